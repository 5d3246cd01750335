/* Launch interface of the split-KV "row block" attention kernel (kernel sets 2
 * and 4): a small block of query rows -- the heads of one GQA group for one or
 * a few tokens -- against a long stretch of one KV head's cache.  Shared by the
 * decode, small-chunk and paged-verify entry points. */
#pragma once

#include "wst_common.cuh"

namespace wst {

constexpr int kRowsTile = 64;       /* cache positions per pipeline stage */
constexpr int kRowsMaxSplits = 64;  /* upper bound on sequence slices */
constexpr int kRowsRingBytes = 196608; /* shared memory of the K/V ring: 6 stages at head_dim 128 */

/* Measurement knobs of the row-block kernel (wst_b200_set_tuning); -1 / 0 = automatic. */
struct RowsTuning {
  int decode_splits = 0;  /* slices of a decode launch (0: one per SM and KV head) */
  int early_depth = -1;   /* tiles requested at once ahead of the grid dependency */
  int ring_stages = 0;    /* ring depth in use (0: all the shared memory holds) */
  int verify_ctas = 0;    /* persistent CTAs of the ragged verify kernel (0: one per SM) */
  int fp8_kernel = 0;     /* decode over the e4m3 cache: 0 by cache length, 1 row-block kernel,
                             2 tensor-memory kernel */
};
RowsTuning &rows_tuning();

/* Whether a decode launch may request cache tiles before the launch ahead of it in
 * the stream has finished (wst_b200_set_decode_overlap; on by default). */
bool decode_overlap_allowed();
void set_decode_overlap(bool on);

struct RowsLaunch {
  /* queries: q of (token t, head h) at q + t*q_tok_stride + h*hd, fp32 */
  const float *q = nullptr;
  long long q_tok_stride = 0;
  /* cache: contiguous [n_seq][n_kv][max_seq][hd] (n_seq = 1 for the drop-in
   * entry points) or the page pool [n_pool_pages][n_kv][16][hd] */
  const __half *k = nullptr;
  const __half *v = nullptr;
  bool paged = false;
  int max_seq = 0;        /* contiguous: rows per head; paged: max_pages*16 */
  const int32_t *page_table = nullptr;
  int max_pages = 0, n_pool_pages = 0;
  /* positions: sequence s starts its tokens at pos0 = pos0_dev ? pos0_dev[s]
   * (+ pos0_bias) : pos0_val; token j sees [0, clamp(pos0 + j + 1, 0, max_seq)) */
  const int32_t *pos0_dev = nullptr;
  int pos0_bias = 0;
  bool clamp_pos0_nonneg = false;  /* decode cursor: max(*pos, 0) */
  int pos0_val = 0;
  /* tokens: cu_tokens ? ragged [n_seq+1] : n_tok for the single sequence */
  const int32_t *cu_tokens = nullptr;
  int n_seq = 1;
  int n_tok = 1;          /* max tokens of any sequence */
  int tok_seq_stride = 0; /* no cu_tokens: sequence s owns tokens [s*stride, s*stride + n_tok) */
  int n_q = 0, n_kv = 0, hd = 0;
  float scale = 1.f;
  /* Decode contract: of the rows this launch reads, the launch right before it in
   * the stream can have written only the newest one (row pos0); the kernel may
   * then request the older tiles before that launch has finished. */
  bool newest_row_only = false;
  /* split scratch, floats: n_units * n_splits * rows_valid_max * (hd+2) */
  float *scratch = nullptr;
  long long scratch_floats = 0;
  int want_splits = 0;    /* 0 = pick from the SM count */
  int max_len = 0;        /* upper bound on any sequence's visible length */
  /* output: fp16 [token][n_q*hd], or (partial mode) fp32 [n_q][hd+2] triples */
  void *out = nullptr;
  bool partial_out = false;
  /* KV sequence sharded over `world` GPUs: the per-head triples are exchanged through
   * the ranks' mailboxes inside the kernel and `out` is the merged fp16 result
   * (one token, one sequence, scratch given) */
  const void *mailboxes = nullptr; /* device array of `world` mailbox addresses */
  void *xstate = nullptr;          /* this rank's per-head call counters */
  int rank = 0, world = 1;
  /* fp8 cache (contiguous, head_dim 128, one row block of at most 16 rows): k and v point
   * at e4m3 bytes [n_seq][n_kv][max_seq][hd]; a stored value times k_scale / v_scale is
   * the key / value */
  bool kv8 = false;
  float k_scale = 1.f, v_scale = 1.f;
  const char *name = "attention";
};

/* True if the tensor-core kernel can take this shape. */
bool rows_kernel_supports(int n_q, int n_kv, int hd, const void *k, const void *v);

/* Slices the kernel will use for a given shape on the current device. */
int rows_pick_splits(int n_units, int max_len, int sm_count);

/* Floats of scratch a launch with `splits` slices needs. */
long long rows_scratch_floats(int n_units_times_rows, int splits, int hd);

wst_status_t launch_rows(const RowsLaunch &L);

/* The slice merge on its own (the tcgen05 kernel's sliced form writes the same
 * scratch rows: acc[hd] | m | l | 2 pad per query row, log2 units). */
struct SplitMerge {
  const float *scratch = nullptr;
  void *out = nullptr;
  const int32_t *cu_tokens = nullptr;
  int n_tok = 1, tok_seq_stride = 0;
  int n_q = 0, n_kv = 0, hd = 0;
  int n_splits = 1, n_rowblk = 1, tpb = 1, rows_cap = 1, n_units = 1;
  /* slices per unit in device memory (the scratch keeps n_splits slots per unit), or
   * null: every unit has n_splits slices */
  const int *slice_counts = nullptr;
  bool partial_out = false;
  /* cross-GPU exchange inside the merge (world > 1; one token, one sequence) */
  const void *mailboxes = nullptr;
  void *xstate = nullptr;
  int rank = 0, world = 1;
  const char *name = "attention";
};
wst_status_t launch_split_merge(const SplitMerge &m);

/* Decode over the e4m3 cache with both contractions on tcgen05 (attn_decode_tc.cu):
 * head_dim 128, one token, at most 16 query heads per KV head, contiguous cache. */
wst_status_t launch_decode_fp8_tc(const RowsLaunch &L);

/* Portable CUDA-core kernel for head widths the tensor-core kernel does not
 * take (any head_dim % 32 == 0 up to 256, contiguous cache, no split). */
wst_status_t launch_simple(const RowsLaunch &L);

}  // namespace wst
