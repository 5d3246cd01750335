#include "tensor_map.cuh"

#include <cudaTypedefs.h>

#include <cstring>
#include <mutex>

namespace wst {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                              const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encoder() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(p);
    } else {
      cudaGetLastError();
    }
  });
  return fn;
}

}  // namespace

wst_status_t make_kv_tensor_map(CUtensorMap *out, const void *base, int rank,
                                const uint64_t *dims, const uint64_t *strides_bytes,
                                const uint32_t *box) {
  EncodeFn fn = encoder();
  if (!fn) return fail(WST_ERR_UNSUPPORTED_ARCH, "cuTensorMapEncodeTiled is not available");
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) s[i] = strides_bytes[i];
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, static_cast<cuuint32_t>(rank),
                  const_cast<void *>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(WST_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return WST_OK;
}

wst_status_t cached_kv_tensor_map(CUtensorMap *out, const KvMapKey &key) {
  struct Slot {
    KvMapKey key;
    CUtensorMap map;
    bool used;
  };
  constexpr int kSlots = 128;
  static thread_local Slot slots[kSlots];
  uint64_t h = reinterpret_cast<uint64_t>(key.base) >> 8;
  h ^= key.d1 * 0x9E3779B97F4A7C15ull;
  h ^= (key.d2 + 31 * key.d3 + 977 * key.b1) * 0xC2B2AE3D27D4EB4Full;
  Slot &s = slots[(h ^ (h >> 29)) % kSlots];
  if (s.used && std::memcmp(&s.key, &key, sizeof(KvMapKey)) == 0) {
    *out = s.map;
    return WST_OK;
  }
  wst_status_t st;
  if (key.rank == 5) {
    /* page pool [pages][n_kv][16][128] seen as (64 columns, 16 rows, 2 column halves,
     * n_kv, pages): one box is both 128-byte halves of a page's 16 rows of one KV head,
     * 4 KB per request, laid down as [half][16 rows][128 B] */
    uint64_t dims[5] = {64, 16, 2, key.d2, key.d3};
    uint64_t strides[4] = {256, 128, 4096, key.d2 * 4096};
    uint32_t box[5] = {64, 16, 2, 1, 1};
    st = make_kv_tensor_map(out, key.base, 5, dims, strides, box);
  } else {
    uint64_t dims[4] = {key.d0, key.d1, key.d2, key.d3};
    uint64_t strides[3] = {key.d0 * 2, key.d0 * key.d1 * 2, key.d0 * key.d1 * key.d2 * 2};
    uint32_t box[4] = {64, key.b1, 1, 1};
    st = make_kv_tensor_map(out, key.base, static_cast<int>(key.rank), dims, strides, box);
  }
  if (st != WST_OK) return st;
  std::memset(&s.key, 0, sizeof(KvMapKey));
  s.key = key;
  s.map = *out;
  s.used = true;
  return WST_OK;
}

}  // namespace wst
