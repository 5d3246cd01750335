/* Launch interface of the chunked-prefill attention kernel (kernel set 3):
 * causal attention of a chunk of query tokens against the KV cache with both
 * contractions on the 5th-generation tensor cores (tcgen05, accumulators in
 * tensor memory, operands staged by TMA). */
#pragma once

#include "wst_common.cuh"

namespace wst {

struct PrefillLaunch {
  const float *qkv = nullptr;  /* [n][q_tok_stride] fp32, q of head h at h*hd */
  long long q_tok_stride = 0;
  bool q16 = false;            /* the q rows are fp16 (stride in halves): qkv points at them */
  const __half *k = nullptr;   /* [n_kv][max_seq][hd] */
  const __half *v = nullptr;
  __half *out = nullptr;       /* [n][n_q*hd] */
  int n_q = 0, n_kv = 0, hd = 0;
  int pos0 = 0, n = 0, max_seq = 0;
  /* batch: n_seq sequences with caches [n_seq][n_kv][max_seq][hd]; sequence s owns
   * tokens s*n .. s*n+n-1 of qkv and out (or cu_tokens[s] .. cu_tokens[s+1]-1, with n
   * the largest count); chunk starts in device memory (null = pos0 for all) */
  int n_seq = 1;
  const int32_t *pos0_dev = nullptr;
  const int32_t *cu_tokens = nullptr;
  /* paged cache instead: pool [n_pool_pages][n_kv][16][hd], page_table [n_seq][max_pages],
   * max_seq = max_pages * 16 */
  const int32_t *page_table = nullptr;
  int max_pages = 0, n_pool_pages = 0;
  /* few query rows against a long prefix: cut the KV range into n_splits slices
   * (needs n * gqa <= 128 and scratch of n_seq*n_kv*n_splits*n*gqa*(hd+4) floats) */
  int n_splits = 0;
  int max_len = 0; /* sliced mode: upper bound on any sequence's visible length (0: max_seq) */
  /* sliced mode: false = slices are runs of ceil(max_len tiles / n_splits) tiles (equal
   * work per CTA whatever the sequence lengths); true = every query tile cuts its own
   * visible prefix into n_splits equal runs (lengths unknown to the host) */
  bool even_slices = false;
  float *scratch = nullptr;
  long long scratch_floats = 0;
  float scale = 1.f;
  int span_ctas = 0;  /* launch_verify_span: CTAs to use (0: one per SM) */
  int force_pair = 0; /* 0 = automatic, 1 = two query tiles per CTA, -1 = one */
  const char *name = "attention";
};

/* True if the tcgen05 kernel takes this shape and the chunk is large enough
 * for 128-row tiles to pay. */
bool prefill_kernel_supports(int n_q, int n_kv, int hd, int n);

/* True if the sliced form (all query rows of a unit in one tile) takes the shape. */
bool prefill_split_supports(int n_q, int n_kv, int hd, int n_tok_max);

wst_status_t launch_prefill(const PrefillLaunch &P);

/* Ragged paged verify (every unit's query rows in one 128-row tile, prefill_split_supports):
 * the KV tiles of all (sequence, KV head) units end to end, cut into one equal span per
 * persistent CTA, + the slice-merge kernel.  Needs P.page_table, P.cu_tokens, P.pos0_dev,
 * P.scratch and P.max_len. */
wst_status_t launch_verify_span(const PrefillLaunch &P);

}  // namespace wst
