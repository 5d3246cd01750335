/* Whetstone attention path for NVIDIA B200: entry points that have no
 * counterpart in the engine's own kernel library.
 *
 * The engine runs one sequence with a contiguous KV cache on one GPU
 * (crates/whetstone-core/src/engine.rs:264-286,
 * crates/whetstone-kernels/src/decode.rs:162-212).  Batches, a paged cache and a
 * KV sequence sharded over several GPUs are therefore additions; they follow the
 * same rules as whetstone.h (plain C types, device pointers unless named _host,
 * wst_status_t + wst_last_error, nothing allocated per call, launches on the
 * calling thread's stream).
 */

#ifndef WHETSTONE_B200_EXT_H
#define WHETSTONE_B200_EXT_H

#include "whetstone.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------- plumbing */

/* Library version, "major.minor.patch". */
WST_API const char *wst_b200_version(void);

/* Stream used by every later call of THIS thread (a cudaStream_t).  NULL
 * restores the per-thread default stream, which is what the engine's library is
 * compiled to use (crates/whetstone-kernels/build.rs:133-138). */
WST_API wst_status_t wst_b200_set_stream(void *stream);

/* Kernels bound every wait on a barrier; one that ran out of time records a
 * nonzero code in a per-device word instead of hanging.  This synchronises the
 * calling thread's stream, returns that word in *out_code and clears it. */
WST_API wst_status_t wst_b200_device_error(uint32_t *out_code);

/* Which kernel family the attention entry points use:
 *   0 = automatic (default)
 *   1 = force the portable CUDA-core kernel
 *   2 = wst_attn_chunk: force the split-KV mma.sync kernel
 *   3 = wst_attn_chunk: force the tcgen05 prefill kernel (one query tile per CTA);
 *       wst_attn_verify_paged: one CTA per slice of the KV range instead of one
 *       persistent CTA per SM
 *   4 = wst_attn_chunk: force the tcgen05 prefill kernel with two query tiles per CTA
 * A debugging aid for A/B checks; process-wide. */
WST_API wst_status_t wst_b200_set_kernel_choice(int32_t choice);

/* Measurement knobs of the decode kernel, process-wide; value -1 or 0 restores the
 * default.  Results do not depend on them beyond fp32 summation order.
 *   key 1  slices of the KV sequence per KV head (default: SMs / KV heads)
 *   key 2  cache tiles requested at once before the launch ahead has finished
 *   key 4  stages of the shared-memory ring in use (head_dim 128: 2..6; at 3 or
 *          fewer, two blocks of consecutive launches share an SM)
 *   key 5  persistent CTAs of wst_attn_verify_paged (default: one per SM)
 *   key 6  kernel of wst_b200_attn_decode_fp8: 0 by the cache's capacity, 1 the row-block
 *          kernel (mma.sync), 2 the tensor-memory kernel (tcgen05) */
WST_API wst_status_t wst_b200_set_tuning(int32_t key, int32_t value);

/* 0: wst_attn_decode (and wst_b200_attn_decode_fp8) waits for everything ahead of it in
 * the stream before it asks for any cache row (no stream-order precondition, see
 * whetstone.h); 1 (default): it asks for the rows below the cursor early.  Process-wide. */
WST_API wst_status_t wst_b200_set_decode_overlap(int32_t on);

/* Allocates the calling thread's 16 MiB split workspace of wst_attn_chunk /
 * wst_attn_chunk_batch on the current device now (once; later calls return at
 * once), so that no chunk call ever has to: call it at start-up, outside any
 * capture.  WST_ERR_OOM with the reason if it cannot be had. */
WST_API wst_status_t wst_b200_reserve_chunk_workspace(void);

/* --------------------------------------------------------- RoPE table */

/* cos/sin tables [max_seq][head_dim/2] float, angles evaluated in double on the
 * host: the definition the engine uses (RopeTable::with_scaling,
 * crates/whetstone-kernels/src/decode.rs:95-147).
 *   scaling_kind 0: inv_freq[j] = theta^(-j/half)
 *   scaling_kind 1: the Llama-3 piecewise schedule (decode.rs:64-86, 110-130)
 *                   with factor / low_freq_factor / high_freq_factor /
 *                   original_max_position
 * Both outputs are HOST buffers of max_seq * head_dim/2 floats. */
WST_API wst_status_t wst_rope_table_host(float *cos_host, float *sin_host, int32_t max_seq,
                                 int32_t head_dim, double theta, int32_t scaling_kind,
                                 double factor, double low_freq_factor,
                                 double high_freq_factor, int32_t original_max_position);

/* ------------------------------- decode over a KV sequence shard (multi-GPU) */

/* Like wst_attn_decode over cache rows [0, *len), but stops before the
 * normalisation: writes, per query head, the running maximum (natural-log
 * units), the denominator and head_dim numerators -- the (m, l, acc) triple of
 * cuda/attention.cu:50-55 -- so that shards of one sequence held by different
 * GPUs can be combined after an all-gather.
 *   len          device int32, rows of THIS cache that are valid (0 allowed;
 *                clamped to [0, max_seq])
 *   partials     scratch of wst_attn_partial_floats() floats
 *   out_partial  [n_q][head_dim + 2] float */
WST_API wst_status_t wst_attn_decode_partial(const void *q, const void *k_cache, const void *v_cache,
                                     void *partials, void *out_partial, int32_t n_q,
                                     int32_t n_kv, int32_t head_dim, const void *len,
                                     int32_t max_seq, float scale);

/* Combines n_parts partial sets [n_parts][n_q][head_dim + 2] (as gathered from
 * the shards) into out [n_q][head_dim] half: the merge of
 * cuda/attention.cu:170-193 across GPUs instead of across slices. */
WST_API wst_status_t wst_attn_merge_partials(const void *parts, void *out, int32_t n_parts,
                                     int32_t n_q, int32_t head_dim);

/* The same merge with the exchange inside the kernel, for the GPUs of one box:
 * every rank stores its triples into all ranks' mailboxes over NVLink -- plain peer
 * stores of 8-byte {value, tag} packets, valid when the tag is the call's -- and
 * merges the packets that arrive in its own mailbox, polling each for at most about
 * a second.  No NCCL call, no fence and no host step between
 * wst_attn_decode_partial and the fp16 result.
 *   my_triples  [n_q][head_dim + 2] float, this rank's wst_attn_decode_partial output
 *   out         [n_q][head_dim] half (every rank gets the full result)
 *   mailboxes   DEVICE array of `world` pointers; entry g = rank g's mailbox,
 *               8-byte packets [2][world][n_q][head_dim + 2], zeroed once before the
 *               first call, mapped into this process (wst_b200_ipc_import)
 *   state       this rank's uint32[n_q] call counters, zeroed once before the first call
 * Every rank must make the same sequence of calls.  A wait that runs out sets the
 * device error word (wst_b200_device_error) and leaves that head's `out` unwritten. */
WST_API wst_status_t wst_attn_exchange_merge(const void *my_triples, void *out,
                                             const void *mailboxes, void *state, int32_t rank,
                                             int32_t world, int32_t n_q, int32_t head_dim);

/* wst_attn_decode_partial and the exchange as ONE call, for the GPUs of one box: the
 * kernel that merges the slices of this rank's shard (one block per query head, the
 * head's triple in registers) stores that triple into the other ranks' mailboxes
 * (plain peer stores over NVLink, 8-byte {value, tag} packets), waits -- each packet
 * for at most about a second -- for theirs in its own mailbox, and writes the fp16
 * result.  Two launches per layer and rank (slices, merge + exchange) where
 * wst_attn_decode_partial + wst_attn_exchange_merge take three and a round trip
 * through memory more; no NCCL call, no host step.
 *   len         device int32: valid rows of THIS rank's shard (as wst_attn_decode_partial)
 *   partials    scratch of wst_attn_partial_floats() floats
 *   out         [n_q][head_dim] half (every rank gets the full result)
 *   mailboxes, state, rank, world   as for wst_attn_exchange_merge; the two entry
 *               points may share them as long as every rank makes the same sequence
 *               of calls
 * Needs head_dim 64 or 128 and at most 32 query heads per KV head
 * (WST_ERR_SHAPE otherwise: use wst_attn_decode_partial + wst_attn_exchange_merge). */
WST_API wst_status_t wst_attn_decode_sharded(const void *q, const void *k_cache,
                                             const void *v_cache, void *partials, void *out,
                                             int32_t n_q, int32_t n_kv, int32_t head_dim,
                                             const void *len, int32_t max_seq, float scale,
                                             const void *mailboxes, void *state, int32_t rank,
                                             int32_t world);

/* One device buffer shared by the processes of a box (one process per GPU).  The
 * owner exports a 64-byte handle of a buffer from wst_malloc; another process
 * imports it with its own device current and gets an address its kernels can use
 * (peer access between the two GPUs is enabled by the import); close before exit. */
WST_API wst_status_t wst_b200_ipc_export(const void *dev_ptr, void *handle64_out_host);
WST_API wst_status_t wst_b200_ipc_import(const void *handle64_host, void **out_dev_ptr);
WST_API wst_status_t wst_b200_ipc_close(void *dev_ptr);

/* cudaDeviceEnablePeerAccess from the current device to peer_device ("already
 * enabled" is not an error); fails if the two cannot be peers. */
WST_API wst_status_t wst_b200_enable_peer_access(int32_t peer_device);

/* --------------------------------------------- decode without a scratch buffer */

/* wst_attn_decode for callers that cannot provide (or allocate) the split
 * scratch: same arguments minus `partials`, same result.  It has no counterpart
 * in the engine's library.  Hosts that gave all their device memory to a pool
 * at start-up, or that are in a phase where they may not call cudaMalloc, still
 * need the sequence split to fill the GPU; here the slices' partial results go
 * to an array built into the library (2 MiB of device memory per GPU, held from
 * load to exit).
 *
 *   - No call allocates or frees device memory.  The array itself is part of the
 *     library's device image: the CUDA driver sets that image up (and with it the
 *     2 MiB) when the library's kernels are first used on a device.  A host that
 *     hands all device memory to its own pool should therefore make one call of
 *     this entry point (or any attention call of this library) per device BEFORE
 *     the pool takes the memory, or load the library with
 *     CUDA_MODULE_LOADING=EAGER.
 *   - Limit: n_q * min(64, ceil(max_seq / 64)) * (head_dim + 4) floats must not
 *     exceed 524288 (e.g. 28 heads of 128 at any context: 236544).  Larger shapes
 *     are refused with WST_ERR_INVALID_ARG; use wst_attn_decode for them.
 *   - The first call on a device looks up the array's device address; make that
 *     call an ordinary one, before any stream capture.
 *   - All calls share the one array and it keeps whatever the last call left in
 *     it.  Nothing in it has to start at zero -- every slot is written before
 *     it is read within a call -- but two calls that overlap on the GPU (two
 *     streams, two threads) would write over each other: run them one after
 *     the other. */
WST_API wst_status_t wst_attn_decode_noscratch(const void *q, const void *k_cache,
                                               const void *v_cache, void *out, int32_t n_q,
                                               int32_t n_kv, int32_t head_dim, const void *pos,
                                               int32_t max_seq, float scale);

/* ---------------------------------------- several sequences, contiguous caches */

/* The chunk entry points for a batch of n_seq sequences that each process n
 * tokens in this step (batched chunked prefill).  One launch covers the whole
 * batch, so the GPU is filled by (sequence, KV head, query tile) units instead of
 * one sequence's worth.  No counterpart in the engine, which runs one sequence.
 *   qkv       [n_seq][n][(n_q + 2*n_kv) * head_dim] float
 *   k_cache   [n_seq][n_kv][max_seq][head_dim] half (v_cache the same)
 *   seq_pos0  device int32 [n_seq]: cache row of each sequence's first token;
 *             rows are clamped to the cache like the single-sequence kernels do
 *   out       [n_seq][n][n_q * head_dim] half
 * Token j of sequence s sees rows [0, seq_pos0[s] + j] of its own cache. */
WST_API wst_status_t wst_rope_cache_chunk_batch(void *qkv, void *k_cache, void *v_cache,
                                                const void *cos_tab, const void *sin_tab,
                                                const void *seq_pos0, int32_t n_seq, int32_t n_q,
                                                int32_t n_kv, int32_t head_dim, int32_t n,
                                                int32_t max_seq, const void *q_norm_w,
                                                const void *k_norm_w, float eps);
WST_API wst_status_t wst_attn_chunk_batch(const void *qkv, const void *k_cache,
                                          const void *v_cache, void *out, const void *seq_pos0,
                                          int32_t n_seq, int32_t n_q, int32_t n_kv,
                                          int32_t head_dim, int32_t n, int32_t max_seq,
                                          float scale);

/* ---- 8-bit KV cache (on the engine's roadmap, docs/ROADMAP.md:206) ---------------- */

/* The cache holds e4m3 bytes, [n_kv][max_seq][head_dim]; a stored byte times k_scale
 * (v_scale) is the key (value).  Half the bytes of the fp16 cache per decoded token.
 *
 * wst_b200_rope_cache_fp8: kernel set 1 with that cache -- norm, rotation and the q
 * write-back exactly as wst_rope_cache / wst_rope_cache_chunk; k and v rows are stored as
 * round-to-nearest-even e4m3 of value / scale, saturating at +-448.  `pos` non-null: one
 * token at the device cursor (n = 1, pos0 ignored); `pos` null: n tokens at rows pos0...
 * head_dim 64, 128 or 256.
 *
 * wst_b200_attn_decode_fp8: wst_attn_decode over that cache (head_dim 128, at most 16
 * query heads per KV head).  The raw tiles are streamed by TMA and converted to fp16 in
 * shared memory (every e4m3 number is an fp16 number, so the attention arithmetic is that
 * of the fp16 path on the dequantized cache); k_scale is folded into the query scale,
 * v_scale into the output.  A cache of 12288 rows or more goes to the tensor-memory kernel
 * (tcgen05.mma for both contractions, a block-wide conversion by dedicated warps), a
 * smaller one to the row-block kernel, where every consumer warp converts its own 16
 * positions of a tile.  Like wst_attn_decode, the call assumes that the launch right
 * before it in the stream writes no cache row but the one at *pos.  The two NaN bytes of
 * e4m3 (0x7f, 0xff) must not occur in rows [0, *pos]: the append never writes them (it
 * saturates), and the kernels do not agree on what they read them as.  Rows past *pos may
 * hold anything.  `partials`: wst_attn_partial_floats as for wst_attn_decode. */
WST_API wst_status_t wst_b200_rope_cache_fp8(void *qkv, void *k_cache8, void *v_cache8,
                                             const void *cos_tab, const void *sin_tab, int32_t n_q,
                                             int32_t n_kv, int32_t head_dim, const void *pos,
                                             int32_t pos0, int32_t n, int32_t max_seq,
                                             const void *q_norm_w, const void *k_norm_w, float eps,
                                             float k_scale, float v_scale);
WST_API wst_status_t wst_b200_attn_decode_fp8(const void *q, const void *k_cache8,
                                              const void *v_cache8, void *partials, void *out,
                                              int32_t n_q, int32_t n_kv, int32_t head_dim,
                                              const void *pos, int32_t max_seq, float scale,
                                              float k_scale, float v_scale);

/* ---- the projection fused with kernel set 1 ------------------------------------ */

/* The qkv projection of a chunk step with the rotation, the head norm and the cache
 * append in its epilogue: what wst_gemm_fp16 + wst_rope_cache_chunk_batch do in two
 * launches with a [tokens][(n_q + 2 n_kv) * head_dim] fp32 buffer written and read back
 * in between.  Here an accumulator tile of 128 tokens x 256 features is whole heads of
 * whole tokens (two heads of 128, four of 64): a thread holds a head of its token in
 * registers, norms it (q and k heads, if gains are given), rotates it at the token's
 * cache position and stores fp16 -- q heads to q_out, k and v heads to the token's row
 * of the batched cache.  No counterpart in the engine, which runs the two steps one
 * after the other (engine.rs:796-809).
 *   w         [(n_q + 2 n_kv) * head_dim][in_f] half     x  [n_seq * n][in_f] half
 *   bias      [(n_q + 2 n_kv) * head_dim] half or null
 *   q_out     [n_seq * n][n_q * head_dim] half: the rotated (and normed) queries, the
 *             input of wst_b200_attn_chunk_batch_q16
 *   k_cache, v_cache, cos_tab, sin_tab, seq_pos0, gains, eps: as for
 *             wst_rope_cache_chunk_batch; table_len = rows of cos/sin
 * head_dim 64 or 128; in_f a multiple of 8; 16-byte aligned buffers. */
WST_API wst_status_t wst_b200_qkv_rope_append_batch(
    const void *w, const void *x, const void *bias, void *q_out, void *k_cache, void *v_cache,
    const void *cos_tab, const void *sin_tab, const void *seq_pos0, int32_t in_f, int32_t n_seq,
    int32_t n, int32_t n_q, int32_t n_kv, int32_t head_dim, int32_t max_seq, int32_t table_len,
    const void *q_norm_w, const void *k_norm_w, float eps);

/* The same with the qkv weights in the engine's hierarchical int4 format (qw, si, sb as
 * for wst_gemm_int4_hier in whetstone.h; in_f a multiple of 32). */
WST_API wst_status_t wst_b200_qkv_int4_rope_append_batch(
    const void *qw, const void *si, const void *sb, const void *x, const void *bias, void *q_out,
    void *k_cache, void *v_cache, const void *cos_tab, const void *sin_tab, const void *seq_pos0,
    int32_t in_f, int32_t n_seq, int32_t n, int32_t n_q, int32_t n_kv, int32_t head_dim,
    int32_t max_seq, int32_t table_len, const void *q_norm_w, const void *k_norm_w, float eps);

/* wst_attn_chunk_batch over fp16 query rows [n_seq * n][n_q * head_dim] (q_out above)
 * instead of the fp32 projection buffer.  Taken by the tensor-core kernels only: chunks
 * of at least 64 query rows per KV head, else WST_ERR_SHAPE. */
WST_API wst_status_t wst_b200_attn_chunk_batch_q16(const void *q16, const void *k_cache,
                                                   const void *v_cache, void *out,
                                                   const void *seq_pos0, int32_t n_seq, int32_t n_q,
                                                   int32_t n_kv, int32_t head_dim, int32_t n,
                                                   int32_t max_seq, float scale);

/* ------------------------------------------------ paged cache, many sequences */

/* Paged KV pool: [n_pool_pages][n_kv][page_size][head_dim] half for K and for V.
 * page_table [n_seq][max_pages] int32 maps (sequence, position / page_size) to
 * a pool page.  Tokens of all sequences are packed token-major:
 * sequence s owns tokens cu_tokens[s] .. cu_tokens[s+1]-1, which sit at cache
 * positions seq_pos0[s] + j.  page_size must be 16. */

/* Fused QK-norm + RoPE + append for a ragged batch (the batched form of
 * wst_rope_cache_chunk).
 *   qkv        [total_tokens][(n_q + 2*n_kv) * head_dim] float
 *   cos/sin    [table_len][head_dim/2] float; positions are clamped to the table */
WST_API wst_status_t wst_rope_cache_paged(void *qkv, void *k_pool, void *v_pool, const void *cos_tab,
                                  const void *sin_tab, const void *page_table,
                                  const void *seq_pos0, const void *cu_tokens, int32_t n_seq,
                                  int32_t total_tokens, int32_t max_pages, int32_t page_size,
                                  int32_t n_pool_pages, int32_t n_q, int32_t n_kv,
                                  int32_t head_dim, int32_t table_len, const void *q_norm_w,
                                  const void *k_norm_w, float eps);

/* Ragged multi-token attention for speculative verification: token j of
 * sequence s sees positions [0, seq_pos0[s] + j] of that sequence's pages (the
 * batched, paged form of wst_attn_chunk).
 *   max_tokens_per_seq  upper bound on cu_tokens[s+1]-cu_tokens[s]
 *   max_len             upper bound on seq_pos0[s] + tokens of s (sizes the grid)
 *   scratch             wst_attn_verify_scratch_floats() floats
 *   out                 [total_tokens][n_q * head_dim] half */
WST_API wst_status_t wst_attn_verify_paged(const void *qkv, const void *k_pool, const void *v_pool,
                                   const void *page_table, const void *seq_pos0,
                                   const void *cu_tokens, void *scratch, void *out,
                                   int32_t n_seq, int32_t total_tokens,
                                   int32_t max_tokens_per_seq, int32_t max_pages,
                                   int32_t page_size, int32_t n_pool_pages, int32_t n_q,
                                   int32_t n_kv, int32_t head_dim, int32_t max_len,
                                   float scale);

WST_API int64_t wst_attn_verify_scratch_floats(int32_t n_seq, int32_t max_tokens_per_seq, int32_t n_q,
                                       int32_t n_kv, int32_t head_dim, int32_t max_len);

/* ----------------------------- host side: paged KV-cache manager and scheduler */

/* Bookkeeping for many sequences over one pool of 16-token pages: which pages a
 * sequence owns, how many rows of them are committed context, and the host arrays
 * (page_table, seq_pos0, cu_tokens) that wst_rope_cache_paged and
 * wst_attn_verify_paged take.  It stands where the engine has one contiguous cache
 * and one cursor (crates/whetstone-kernels/src/decode.rs:162-212,
 * crates/whetstone-core/src/engine.rs:264-286, 865-880) and follows the engine's
 * speculative loop (crates/whetstone-core/src/speculate.rs:185-256): reserve rows,
 * launch append + attention, commit what was accepted, rewind over what was not --
 * rejected rows are not erased, the next append writes over them.  The C++ classes
 * are in whetstone_b200/host/paged_kv.hpp; these are their C bindings.  Host work
 * only: no call here touches a GPU; a manager is used from one thread at a time.
 *
 *   wst_pkv_create      pool of n_pool_pages pages, no sequence longer than max_len
 *   wst_pkv_open/close  a new empty sequence (ids are reused) / all its pages back
 *   wst_pkv_query       length and page count of `seq` (seq < 0: skip) and the
 *                       pool's free pages; any out pointer may be NULL
 *   wst_pkv_reserve     room for n_tokens more rows; WST_ERR_OOM and no change if the
 *                       pool is short, WST_ERR_SHAPE past max_len
 *   wst_pkv_commit      n_tokens reserved rows now count as context
 *   wst_pkv_rewind      context length back to pos (<= length); pages stay mapped
 *   wst_pkv_trim        pages beyond length + keep_tokens go back to the pool
 *   wst_pkv_schedule    from n_waiting (seq, n_tokens) requests picks this step's
 *                       batch, longest context first, within max_tokens_per_step,
 *                       max_sequences_per_step and the pool's free pages; writes the
 *                       chosen requests' indices in launch order
 *   wst_pkv_build_step  reserves every entry's rows (all or none: WST_ERR_OOM leaves
 *                       the manager unchanged) and fills the HOST arrays
 *                       page_table [n_seq][max_pages], seq_pos0 [n_seq],
 *                       cu_tokens [n_seq + 1]; totals_out4 = total_tokens,
 *                       max_tokens_per_seq, max_len, max_pages
 *   wst_pkv_assign_units  deals the n_seq * n_kv (batch slot, KV head) units to
 *                       `world` GPUs, heaviest first to the least loaded rank;
 *                       rank_of_unit_out[slot * n_kv + kv_head] */
WST_API wst_status_t wst_pkv_create(int32_t n_pool_pages, int32_t max_len, void **out_mgr);
WST_API wst_status_t wst_pkv_destroy(void *mgr);
WST_API wst_status_t wst_pkv_open(void *mgr, int32_t *out_seq);
WST_API wst_status_t wst_pkv_close(void *mgr, int32_t seq);
WST_API wst_status_t wst_pkv_query(void *mgr, int32_t seq, int32_t *out_length,
                                   int32_t *out_pages, int32_t *out_free_pages);
WST_API wst_status_t wst_pkv_reserve(void *mgr, int32_t seq, int32_t n_tokens);
WST_API wst_status_t wst_pkv_commit(void *mgr, int32_t seq, int32_t n_tokens);
WST_API wst_status_t wst_pkv_rewind(void *mgr, int32_t seq, int32_t pos);
WST_API wst_status_t wst_pkv_trim(void *mgr, int32_t seq, int32_t keep_tokens,
                                  int32_t *out_returned);
WST_API wst_status_t wst_pkv_schedule(void *mgr, const int32_t *seqs, const int32_t *n_tokens,
                                      int32_t n_waiting, int32_t max_tokens_per_step,
                                      int32_t max_sequences_per_step, int32_t *chosen_out,
                                      int32_t *n_chosen_out);
WST_API wst_status_t wst_pkv_build_step(void *mgr, const int32_t *seqs, const int32_t *n_tokens,
                                        int32_t n_seq, int32_t *page_table_host,
                                        int32_t *seq_pos0_host, int32_t *cu_tokens_host,
                                        int32_t *totals_out4);
WST_API wst_status_t wst_pkv_assign_units(const int32_t *seq_pos0_host,
                                          const int32_t *cu_tokens_host, int32_t n_seq,
                                          int32_t n_kv, int32_t world, int32_t *rank_of_unit_out);

#ifdef __cplusplus
}
#endif

#endif /* WHETSTONE_B200_EXT_H */
