/* Whetstone attention path for NVIDIA B200 (sm_100a): the drop-in C ABI.
 *
 * Every function here keeps the name, argument order, argument meaning, return
 * convention and error behaviour of the entry point of the same name in the
 * Whetstone engine's kernel library, so that the engine's FFI layer
 * (crates/whetstone-kernels/src/ffi.rs) binds to this library unchanged.  Each
 * declaration cites the line of crates/whetstone-kernels/cuda/whetstone.h it
 * replaces.  Entry points that have no counterpart there are in
 * whetstone_b200.h.
 *
 * Conventions (whetstone.h:3-9, common.cuh:17-54):
 *   - plain C types only; tensors are `void *` DEVICE pointers unless the name
 *     ends in _host;
 *   - every entry returns wst_status_t and never aborts, throws or longjmps;
 *   - on failure a message is left in a thread-local buffer, see wst_last_error;
 *   - argument errors return WST_ERR_INVALID_ARG before anything is launched;
 *   - kernels are enqueued on the calling thread's stream (the per-thread default
 *     stream unless wst_b200_set_stream changed it); nothing synchronises, and
 *     after its first call on a device no entry point allocates, so a whole
 *     decode step can be captured into a CUDA graph.
 */

#ifndef WHETSTONE_B200_DROPIN_H
#define WHETSTONE_B200_DROPIN_H

#include <stddef.h>
#include <stdint.h>

/* Exported from the shared library even when it is built with hidden default
 * visibility. */
#if defined(__GNUC__)
#define WST_API __attribute__((visibility("default")))
#else
#define WST_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: whetstone.h:21-28. */
typedef enum {
  WST_OK = 0,
  WST_ERR_CUDA = 1,
  WST_ERR_INVALID_ARG = 2,
  WST_ERR_UNSUPPORTED_ARCH = 3,
  WST_ERR_OOM = 4,
  WST_ERR_SHAPE = 5,
} wst_status_t;

/* Message of the calling thread's last failure; never NULL.  whetstone.h:78. */
WST_API const char *wst_last_error(void);

/* ----------------------------------------------------- device and memory */
/* Thin runtime wrappers, whetstone.h:72-76, 82-94.  Provided so that a host
 * program can drive the attention path with this library alone. */
WST_API wst_status_t wst_device_count(int32_t *out_count);
WST_API wst_status_t wst_device_set(int32_t ordinal);
WST_API wst_status_t wst_device_synchronize(void);
WST_API wst_status_t wst_malloc(void **out_ptr, size_t bytes);
WST_API wst_status_t wst_free(void *ptr);
WST_API wst_status_t wst_memset(void *dst, int32_t value, size_t bytes);
WST_API wst_status_t wst_memcpy_h2d(void *dst, const void *src_host, size_t bytes);
WST_API wst_status_t wst_memcpy_d2h(void *dst_host, const void *src, size_t bytes);
WST_API wst_status_t wst_memcpy_d2d(void *dst, const void *src, size_t bytes);

/* ------------------------------------------- graphs, events, the cursor */
/* whetstone.h:270-285.  Capture is thread-local on the calling thread's
 * stream; events are recorded into that stream. */
WST_API wst_status_t wst_graph_capture_begin(void);
WST_API wst_status_t wst_graph_capture_end(void **out_exec);
WST_API wst_status_t wst_graph_launch(void *exec);
WST_API wst_status_t wst_graph_destroy(void *exec);
WST_API wst_status_t wst_stream_sync(void);
WST_API wst_status_t wst_event_create(void **out);
WST_API wst_status_t wst_event_record(void *ev);
WST_API wst_status_t wst_event_elapsed_ms(void *a, void *b, float *out);
WST_API wst_status_t wst_event_destroy(void *ev);

/* *pos = min(*pos + 1, max_seq) as a stream-ordered node.  whetstone.h:285,
 * cuda/decode.cu:215-226. */
WST_API wst_status_t wst_advance_pos(void *pos, int32_t max_seq);

/* ------------------------------------------------ single-token (decode) */

/* Fused per-head RMSNorm (optional) + half-rotation RoPE + KV-cache append for
 * the one new token at *pos.  whetstone.h:225-228, cuda/decode.cu:112-208.
 *
 *   qkv        [n_q + 2*n_kv][head_dim] float; q is normed+rotated in place,
 *              k is normed+rotated and narrowed to half into the cache, v is
 *              narrowed to half into the cache untouched
 *   k_cache    [n_kv][max_seq][head_dim] half, row *pos is written
 *   v_cache    same
 *   cos_tab, sin_tab  [max_seq][head_dim/2] float
 *   pos        device int32, clamped to [0, max_seq-1] inside the kernel
 *   q_norm_w, k_norm_w  [head_dim] half gains, or NULL for no QK-norm
 */
WST_API wst_status_t wst_rope_cache(void *qkv, void *k_cache, void *v_cache, const void *cos_tab,
                            const void *sin_tab, int32_t n_q, int32_t n_kv,
                            int32_t head_dim, const void *pos, int32_t max_seq,
                            const void *q_norm_w, const void *k_norm_w, float eps);

/* GQA attention of one query token over cache rows [0, clamp(*pos)+1).
 * whetstone.h:242-245, cuda/attention.cu:57-247.
 *
 *   q          [n_q][head_dim] float (the leading part of qkv, after RoPE)
 *   partials   scratch of wst_attn_partial_floats() floats
 *   out        [n_q][head_dim] half
 *   scale      multiplies the scores (callers pass 1/sqrt(head_dim))
 * Requires n_q % n_kv == 0, head_dim % 32 == 0, head_dim <= 256.
 *
 * Stream-order precondition (this library only; the engine's kernel has none): the
 * kernel is launched with programmatic stream serialization and asks for cache rows
 * below *pos before the launches ahead of it in the stream have finished.  So,
 * between the last ordinary kernel launch (one without that attribute: every
 * launch of the engine today) that wrote rows [0, *pos) of this layer's k_cache /
 * v_cache and this call, the stream may hold only launches that write no such row:
 * this library's wst_rope_cache (it writes row *pos alone, and the kernel re-reads
 * that row after its dependency has resolved), wst_attn_decode of other layers,
 * GEMVs and the like.  The engine's call order (qkv GEMV, wst_rope_cache,
 * wst_attn_decode: crates/whetstone-core/src/engine.rs:526-536) satisfies it.  A
 * host that rewrites older rows right before a decode (restoring a cache from a
 * snapshot, say) either synchronises first or switches the early requests off
 * with wst_b200_set_decode_overlap(0). */
WST_API wst_status_t wst_attn_decode(const void *q, const void *k_cache, const void *v_cache,
                             void *partials, void *out, int32_t n_q, int32_t n_kv,
                             int32_t head_dim, const void *pos, int32_t max_seq,
                             float scale);

/* Floats of split scratch wst_attn_decode needs for one layer.
 * whetstone.h:248, cuda/attention.cu:251-253. */
WST_API int32_t wst_attn_partial_floats(int32_t n_q, int32_t head_dim, int32_t max_seq);

/* --------------------------------------------------- multi-token (chunk) */

/* The same fused RoPE/norm/append for tokens j in [0, n) at cache rows pos0+j.
 * whetstone.h:355-359, cuda/chunk_ops.cu:101-181.
 *   qkv   [n][(n_q + 2*n_kv) * head_dim] float, token-major
 * Requires pos0 >= 0 and pos0 + n <= max_seq. */
WST_API wst_status_t wst_rope_cache_chunk(void *qkv, void *k_cache, void *v_cache,
                                  const void *cos_tab, const void *sin_tab, int32_t n_q,
                                  int32_t n_kv, int32_t head_dim, int32_t pos0, int32_t n,
                                  int32_t max_seq, const void *q_norm_w,
                                  const void *k_norm_w, float eps);

/* Causal attention of a chunk: query j sees cache rows [0, pos0 + j].  Used for
 * both chunked prefill and speculative verification.
 * whetstone.h:360-362, cuda/chunk_ops.cu:187-291.
 *   qkv   as above (q of token j, head h at j*stride + h*head_dim)
 *   out   [n][n_q * head_dim] half
 * A few tokens against a long prefix are cut into slices of the KV range; their
 * partial rows go to a 16 MiB workspace the library keeps per host thread and
 * device, allocated by the thread's first such call (an ordinary call, not one under
 * capture) or by wst_b200_reserve_chunk_workspace (whetstone_b200.h).  Without one
 * the call still runs, unsplit, returns WST_OK and says so in wst_last_error(). */
WST_API wst_status_t wst_attn_chunk(const void *qkv, const void *k_cache, const void *v_cache,
                            void *out, int32_t n_q, int32_t n_kv, int32_t head_dim,
                            int32_t pos0, int32_t n, int32_t max_seq, float scale);

/* ---- the projection either side of the attention path ------------------------ */

/* y[j][r] = sum_c x[j][c] * w[r][c] (+ bias[r]) for j < n, r < out_f; with accum != 0
 * the result is added to what y holds (the o_proj form: straight into the residual).
 * whetstone.h:313-317, cuda/chunk_gemm.cu:178-258 and :340-365.
 *   w     [out_f][in_f] half        x  [n][in_f] half, token-major
 *   bias  [out_f] half or null      y  [n][out_f] float
 * Any n is one launch.  Products and sums are fp32 (the engine's kernel rounds groups
 * of four products to fp16 first), so results agree with the engine's to its own
 * rounding, inside the 2e-3 relative bound of its tests. */
WST_API wst_status_t wst_gemm_fp16(const void *w, const void *x, const void *bias, void *y,
                           int32_t in_f, int32_t out_f, int32_t n, int32_t accum);

/* The same projection with weights in the engine's hierarchical int4 format
 * (whetstone.h:313-315, cuda/chunk_gemm.cu:61-176, cuda/hier.cuh:8-13):
 *   qw  [out_f][in_f/32] 16-byte words: 32 nibbles q, weight c of a group in bits 4c..4c+3
 *   si  [out_f][in_f/32] bytes: ls | lm << 4, two 4-bit scale indices per group
 *   sb  [out_f] half2 (d, dmin)            w = q * (d * ls) - dmin * lm
 * in_f a multiple of 32.  The engine's kernel covers 16 tokens per pass and re-reads the
 * weights for every pass; here the weight tile is unpacked to fp16 in shared memory by
 * sixteen warps of the CTA and the contraction runs on the tensor cores for any n.  Each
 * weight is evaluated in fp32 and rounded to fp16 once (the engine keeps q exact and
 * rounds partial dot products to fp16 instead, and sits three to six times further from
 * the exact product); inside the 3e-3 relative bound of the engine's test at its shape
 * (tests/chunk_kernels.rs:114-167). */
WST_API wst_status_t wst_gemm_int4_hier(const void *qw, const void *si, const void *sb,
                                const void *x, const void *bias, void *y, int32_t in_f,
                                int32_t out_f, int32_t n, int32_t accum);

/* Tokens per weight pass, which the engine takes as its prefill chunk width
 * (whetstone.h:311, src/chunk.rs:20): 512 here, 16 in the engine's kernels. */
WST_API int32_t wst_chunk_max_tokens(void);

#ifdef __cplusplus
}
#endif

#endif /* WHETSTONE_B200_DROPIN_H */
