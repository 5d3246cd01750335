/* Host-side construction of TMA tensor maps for the KV cache.  The driver's
 * encoder is fetched through the runtime (cudaGetDriverEntryPoint), so the
 * library links against cudart only. */
#pragma once

#include <cuda.h>

#include "wst_common.cuh"

namespace wst {

/* fp16 tensor of rank 3 to 5, innermost dimension contiguous, tiles laid out in
 * shared memory with the 128-byte swizzle.  dims/box are in elements, innermost
 * first; strides_bytes[i] is the byte stride of dimension i+1.  Out-of-range
 * parts of a tile read as zero.  Returns WST_OK or sets the error text. */
wst_status_t make_kv_tensor_map(CUtensorMap *out, const void *base, int rank,
                                const uint64_t *dims, const uint64_t *strides_bytes,
                                const uint32_t *box);

/* Small per-thread cache in front of the encoder: the same (pointer, shape) pair
 * comes back every decode step of every layer. */
/* rank 3: contiguous caches (d0 = head_dim, d1 = rows, d2 = planes), box 64 x b1;
 * rank 4: page pool (d0 = head_dim, d1 = 16, d2 = n_kv, d3 = pages), box 64 x 16;
 * rank 5: page pool of head_dim 128 with both 128-byte halves of a page in one box
 *         (d2 = n_kv, d3 = pages; d0, d1, b1 as for rank 4) */
struct KvMapKey {
  const void *base;
  uint64_t d0, d1, d2, d3;
  uint32_t b1;
  uint32_t rank;
};
wst_status_t cached_kv_tensor_map(CUtensorMap *out, const KvMapKey &key);

}  // namespace wst
