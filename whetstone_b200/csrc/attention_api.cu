/* C-ABI entry points of the attention kernels: argument checks (same rules and
 * messages' meaning as cuda/attention.cu:219-247 and cuda/chunk_ops.cu:267-291
 * of the engine), kernel selection, and the small cross-GPU merge kernel. */

#include <atomic>
#include <mutex>

#include "attn_prefill.cuh"
#include "attn_rows.cuh"
#include "wst_ptx.cuh"

namespace wst {
namespace {

std::atomic<int> g_kernel_choice{0};

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

/* wst_attn_chunk has no scratch argument (the engine's chunk kernel never
 * splits the sequence), but a handful of draft tokens against a long prefix
 * must be split to fill the GPU.  The slices' partial rows go to a workspace of
 * fixed size (16 MiB) that the library keeps per host thread and device (the engine
 * drives a GPU from one thread, on that thread's stream); one thread that switches
 * streams with wst_b200_set_stream shares its workspace between them and must not let
 * two such chunk calls overlap on the GPU.  It is allocated by
 * wst_b200_reserve_chunk_workspace, or by the thread's first chunk call that wants
 * it -- which, as for every lazily initialised part of this ABI, has to be an
 * ordinary (not graph-captured) call.  When there is none and none can be had
 * (capture in progress, out of memory), the call still runs, unsplit, and says so in
 * the thread's error text.  Never freed: it lives as long as the process. */
constexpr long long kChunkWorkspaceFloats = 4ll << 20; /* 16 MiB */

/* Returns nullptr (and the reason) when no workspace exists and none can be made. */
float *chunk_workspace(const char **why) {
  static thread_local float *ws[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *why = "cudaGetDevice failed";
    return nullptr;
  }
  if (ws[dev]) return ws[dev];
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(current_stream(), &cap);
  if (cap != cudaStreamCaptureStatusNone) {
    *why = "the stream is being captured and this thread has no workspace yet";
    return nullptr;
  }
  void *p = nullptr;
  if (cudaMalloc(&p, kChunkWorkspaceFloats * sizeof(float)) != cudaSuccess) {
    cudaGetLastError();
    *why = "cudaMalloc of the 16 MiB workspace failed";
    return nullptr;
  }
  ws[dev] = static_cast<float *>(p);
  return ws[dev];
}

/* Records, without failing the call, that a launch ran unsplit for want of a workspace. */
void note_unsplit(const char *who, const char *why) {
  fail(WST_OK, "%s: ran without splitting the KV range (%s); call "
               "wst_b200_reserve_chunk_workspace once outside any capture", who, why);
}

/* Slices of the KV range for a chunk launch of `tiles` (unit, query tile) pairs
 * against at most `len` positions: none when the tiles fill the GPU by themselves or
 * the prefix is short; else enough to fill it, in runs of at least two KV tiles. */
int chunk_slices(int sm_count, long long tiles, int len) {
  if (tiles <= 0 || tiles * 2 > sm_count || len <= 512) return 1;
  long long s = sm_count / tiles;
  const long long kv_tiles = (len + 127) / 128;
  if (s > kv_tiles / 2) s = kv_tiles / 2;
  if (s > kRowsMaxSplits) s = kRowsMaxSplits;
  return s < 2 ? 1 : static_cast<int>(s);
}

int max_splits_for(int max_seq) {
  int t = (max_seq + kRowsTile - 1) / kRowsTile;
  if (t > kRowsMaxSplits) t = kRowsMaxSplits;
  return t < 1 ? 1 : t;
}

/* Shared checks of the decode-shaped entry points. */
wst_status_t check_decode_shape(const char *who, int32_t n_q, int32_t n_kv, int32_t head_dim,
                                int32_t max_seq) {
  if (!(n_q > 0 && n_kv > 0 && head_dim > 0))
    return fail(WST_ERR_INVALID_ARG, "%s: non-positive shape", who);
  if (n_q % n_kv != 0)
    return fail(WST_ERR_INVALID_ARG, "%s: query heads must be a multiple of key/value heads", who);
  if (head_dim % 32 != 0)
    return fail(WST_ERR_INVALID_ARG, "%s: head_dim must be a multiple of the warp size", who);
  if (head_dim > 256) return fail(WST_ERR_INVALID_ARG, "%s: head_dim too large", who);
  if (max_seq <= 0) return fail(WST_ERR_INVALID_ARG, "%s: empty cache", who);
  return WST_OK;
}

wst_status_t decode_common(const char *who, const void *q, const void *k_cache,
                           const void *v_cache, void *partials, void *out, int32_t n_q,
                           int32_t n_kv, int32_t head_dim, const void *pos, int32_t max_seq,
                           float scale, bool len_is_count, bool partial_out,
                           const void *mailboxes = nullptr, void *xstate = nullptr, int rank = 0,
                           int world = 1) {
  RowsLaunch L;
  L.name = who;
  L.q = static_cast<const float *>(q);
  L.q_tok_stride = 0;
  L.k = static_cast<const __half *>(k_cache);
  L.v = static_cast<const __half *>(v_cache);
  L.max_seq = max_seq;
  L.pos0_dev = static_cast<const int32_t *>(pos);
  if (len_is_count) {
    L.pos0_bias = -1; /* `len` counts rows: the last visible one is len-1 */
    L.clamp_pos0_nonneg = false;
  } else {
    L.clamp_pos0_nonneg = true; /* seq = max(*pos, 0) + 1 */
  }
  L.n_seq = 1;
  L.n_tok = 1;
  L.newest_row_only = true;
  L.n_q = n_q;
  L.n_kv = n_kv;
  L.hd = head_dim;
  L.scale = scale;
  L.scratch = static_cast<float *>(partials);
  L.scratch_floats = static_cast<long long>(n_q) * max_splits_for(max_seq) * (head_dim + 4);
  L.max_len = max_seq;
  L.out = out;
  L.partial_out = partial_out;
  L.mailboxes = mailboxes;
  L.xstate = xstate;
  L.rank = rank;
  L.world = world;
  if (g_kernel_choice.load() != 1 && rows_kernel_supports(n_q, n_kv, head_dim, k_cache, v_cache) &&
      aligned16(q))
    return launch_rows(L);
  if (world > 1)
    return fail(WST_ERR_SHAPE, "%s: needs head_dim 64 or 128 and 16-byte aligned buffers", who);
  return launch_simple(L);
}

/* Split scratch for wst_attn_decode_noscratch.  It lives in the library's own
 * device image instead of coming from the caller: some hosts may not allocate
 * device memory at all once they are running -- an engine that handed its whole
 * budget to a pool at start-up, or code that is inside a region (a capture, a
 * latency-critical loop) where cudaMalloc is off limits -- and the engine's
 * decode entry point cannot run without a scratch buffer.  2 MiB per GPU that
 * loads the library, held until the process exits.
 *
 * The array's NAME is only a host-side handle.  Its device address is asked for
 * once per device, with that device current (cudaGetSymbolAddress), and that
 * address is what the kernels receive. */
constexpr long long kBuiltinScratchFloats = 512ll * 1024;
static __device__ __align__(256) float g_builtin_scratch[kBuiltinScratchFloats];

wst_status_t builtin_scratch(float **out) {
  static float *ptrs[64] = {};
  static std::mutex mu;
  int dev = 0;
  WST_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(WST_ERR_CUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_builtin_scratch);
    if (e != cudaSuccess) return cuda_fail("cudaGetSymbolAddress(built-in scratch)", e);
    ptrs[dev] = static_cast<float *>(p);
  }
  *out = ptrs[dev];
  return WST_OK;
}

__global__ void merge_partials_kernel(const float *__restrict__ parts, __half *__restrict__ out,
                                      int n_parts, int n_q, int hd) {
  const int head = blockIdx.x;
  const int stride = hd + 2;
  float big = -INFINITY;
  for (int g = 0; g < n_parts; ++g)
    big = fmaxf(big, parts[(static_cast<long long>(g) * n_q + head) * stride]);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int g = 0; g < n_parts; ++g) {
      const float *t = parts + (static_cast<long long>(g) * n_q + head) * stride;
      if (t[0] == -INFINITY) continue; /* an empty shard contributes nothing */
      const float f = expf(t[0] - big);
      num = fmaf(t[2 + d], f, num);
      den = fmaf(t[1], f, den);
    }
    out[static_cast<long long>(head) * hd + d] = __float2half_rn(den > 0.f ? num / den : 0.f);
  }
}

/* ---------------------------------------------------------------------------
 * Cross-GPU merge through peer memory (the KV sequence of one long context is
 * sharded over the GPUs of a box; each rank has its heads' (m, l, acc) triples).
 * One block per query head; no block waits for another block of its own grid.
 *
 * Every float travels as an 8-byte packet {value, tag} written with ONE 64-bit store, so a
 * packet is valid exactly when its tag is this call's tag: no fence, no separate
 * flag, no ordering between packets.  The block stores its head's triple into every
 * rank's mailbox (plain stores to peer memory over NVLink), then reads the same
 * head's packets of all ranks from its OWN mailbox, polling -- bounded -- each packet
 * it needs until the tag is there, and merges.  The tag is a per-head call counter
 * kept in device memory (graph replays advance it).  Mailboxes exist twice, used by
 * tag parity: a rank can publish call t+2 only after it has received everybody's
 * t+1, which they sent after reading t.  Every rank runs its own launch on its own
 * GPU; nothing here waits for another launch on the same GPU. */
struct ExchangeArgs {
  const float *mine;        /* [n_q][hd+2] */
  __half *out;              /* [n_q][hd] */
  uint2 *const *mailboxes;  /* [world] -> packets [2][world][n_q][hd+2] on rank g */
  unsigned int *state;      /* this rank: per-head call counters [n_q] */
  unsigned int *err_word;
  int rank, world, n_q, hd;
};

__device__ __forceinline__ void st_packet(uint2 *p, float value, unsigned int tag) {
  const unsigned long long pk = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(value);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(pk) : "memory");
}
/* value of a packet once its tag has arrived; false after about a second */
__device__ __forceinline__ bool wait_packet(const uint2 *p, unsigned int tag, float *value) {
  auto load = [p]() {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
  };
  unsigned long long v = load();
  if (static_cast<unsigned int>(v >> 32) != tag) {
    const long long t0 = clock64();
    do {
      if (clock64() - t0 > ptx::kWaitCycleLimit) return false;
      v = load();
    } while (static_cast<unsigned int>(v >> 32) != tag);
  }
  *value = __uint_as_float(static_cast<unsigned int>(v));
  return true;
}

__global__ void __launch_bounds__(128) exchange_merge_kernel(const ExchangeArgs a) {
  /* the next kernel in the stream may start its prologue; this one needs the
   * triples its predecessor wrote */
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x, tid = threadIdx.x;
  const int stride = a.hd + 2;
  const unsigned int tag = a.state[head] + 1u;
  const int par = static_cast<int>(tag & 1u);

  /* 1. publish */
  const float *src = a.mine + static_cast<long long>(head) * stride;
  const long long slot = (static_cast<long long>(par) * a.world + a.rank) * a.n_q + head;
  for (int i = tid; i < stride; i += blockDim.x) {
    const float v = src[i];
    for (int g = 0; g < a.world; ++g) st_packet(a.mailboxes[g] + slot * stride + i, v, tag);
  }

  /* 2. merge this head's triples of all ranks as they arrive in this GPU's mailbox */
  const uint2 *box = a.mailboxes[a.rank] +
                     (static_cast<long long>(par) * a.world * a.n_q + head) * stride;
  const long long rank_stride = static_cast<long long>(a.n_q) * stride;
  bool ok = true;
  float big = -INFINITY;
  for (int g = 0; ok && g < a.world; ++g) {
    float m;
    ok = wait_packet(box + g * rank_stride, tag, &m);
    big = fmaxf(big, m);
  }
  for (int d = tid; ok && d < a.hd; d += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int g = 0; g < a.world; ++g) {
      const uint2 *t = box + g * rank_stride;
      float m, l, acc;
      ok = wait_packet(t, tag, &m) && wait_packet(t + 1, tag, &l) && wait_packet(t + 2 + d, tag, &acc);
      if (!ok) break;
      if (m == -INFINITY) continue; /* an empty shard contributes nothing */
      const float f = expf(m - big);
      num = fmaf(acc, f, num);
      den = fmaf(l, f, den);
    }
    if (ok)
      a.out[static_cast<long long>(head) * a.hd + d] = __float2half_rn(den > 0.f ? num / den : 0.f);
  }
  if (!ok) atomicCAS(a.err_word, 0u, 0x401u);
  __syncthreads(); /* every thread has read the counter and is done with the call */
  if (tid == 0) a.state[head] = tag;
}

}  // namespace
}  // namespace wst

using namespace wst;

extern "C" wst_status_t wst_b200_set_kernel_choice(int32_t choice) {
  WST_CHECK_ARG(choice >= 0 && choice <= 4, "wst_b200_set_kernel_choice: unknown choice");
  g_kernel_choice.store(choice);
  return WST_OK;
}

extern "C" wst_status_t wst_b200_set_tuning(int32_t key, int32_t value) {
  RowsTuning &t = rows_tuning();
  switch (key) {
    case 1: t.decode_splits = value; break;
    case 2: t.early_depth = value; break;
    case 4: t.ring_stages = value; break;
    case 5: t.verify_ctas = value; break;
    case 6: t.fp8_kernel = value; break;
    default: return fail(WST_ERR_INVALID_ARG, "wst_b200_set_tuning: unknown key %d", key);
  }
  return WST_OK;
}

extern "C" wst_status_t wst_b200_set_decode_overlap(int32_t on) {
  set_decode_overlap(on != 0);
  return WST_OK;
}

extern "C" wst_status_t wst_b200_reserve_chunk_workspace(void) {
  const char *why = "";
  if (!chunk_workspace(&why))
    return fail(WST_ERR_OOM, "wst_b200_reserve_chunk_workspace: %s", why);
  return WST_OK;
}

extern "C" int32_t wst_attn_partial_floats(int32_t n_q, int32_t head_dim, int32_t max_seq) {
  if (n_q <= 0 || head_dim <= 0 || max_seq <= 0) return 0;
  const long long f = static_cast<long long>(n_q) * max_splits_for(max_seq) * (head_dim + 4);
  return f > 0x7fffffffLL ? 0x7fffffff : static_cast<int32_t>(f);
}

extern "C" wst_status_t wst_attn_decode(const void *q, const void *k_cache, const void *v_cache,
                                        void *partials, void *out, int32_t n_q, int32_t n_kv,
                                        int32_t head_dim, const void *pos, int32_t max_seq,
                                        float scale) {
  WST_CHECK_ARG(q && k_cache && v_cache && out && pos && partials,
                "wst_attn_decode: null pointer");
  wst_status_t st = check_decode_shape("wst_attn_decode", n_q, n_kv, head_dim, max_seq);
  if (st != WST_OK) return st;
  return decode_common("wst_attn_decode", q, k_cache, v_cache, partials, out, n_q, n_kv,
                       head_dim, pos, max_seq, scale, false, false);
}

extern "C" wst_status_t wst_b200_attn_decode_fp8(const void *q, const void *k_cache8,
                                                 const void *v_cache8, void *partials, void *out,
                                                 int32_t n_q, int32_t n_kv, int32_t head_dim,
                                                 const void *pos, int32_t max_seq, float scale,
                                                 float k_scale, float v_scale) {
  const char *who = "wst_b200_attn_decode_fp8";
  WST_CHECK_ARG(q && k_cache8 && v_cache8 && out && pos && partials,
                "wst_b200_attn_decode_fp8: null pointer");
  wst_status_t st = check_decode_shape(who, n_q, n_kv, head_dim, max_seq);
  if (st != WST_OK) return st;
  WST_CHECK_ARG(k_scale > 0.f && v_scale > 0.f, "wst_b200_attn_decode_fp8: scales must be positive");
  if (head_dim != 128 || n_q / n_kv > 16 || !aligned16(q) || !aligned16(k_cache8) ||
      !aligned16(v_cache8))
    return fail(WST_ERR_SHAPE,
                "%s: needs head_dim 128, at most 16 query heads per KV head and 16-byte aligned "
                "buffers", who);
  RowsLaunch L;
  L.name = who;
  L.q = static_cast<const float *>(q);
  L.k = static_cast<const __half *>(k_cache8);
  L.v = static_cast<const __half *>(v_cache8);
  L.kv8 = true;
  L.k_scale = k_scale;
  L.v_scale = v_scale;
  L.max_seq = max_seq;
  L.pos0_dev = static_cast<const int32_t *>(pos);
  L.clamp_pos0_nonneg = true; /* seq = max(*pos, 0) + 1 */
  L.n_seq = 1;
  L.n_tok = 1;
  L.n_q = n_q;
  L.n_kv = n_kv;
  L.hd = head_dim;
  L.scale = scale;
  L.scratch = static_cast<float *>(partials);
  L.scratch_floats = static_cast<long long>(n_q) * max_splits_for(max_seq) * (head_dim + 4);
  L.max_len = max_seq;
  L.out = out;
  /* The tensor-memory kernel pays about a microsecond more per launch and 0.9 us per 128-row
   * tile and slice where the row-block kernel pays 1.4: level at 12288 rows, ahead beyond.
   * The cursor lives on the device, so the choice goes by the cache's capacity. */
  const int pick = rows_tuning().fp8_kernel;
  if (pick == 2 || (pick == 0 && max_seq >= 12288)) return launch_decode_fp8_tc(L);
  return launch_rows(L);
}

extern "C" wst_status_t wst_attn_decode_noscratch(const void *q, const void *k_cache,
                                                  const void *v_cache, void *out, int32_t n_q,
                                                  int32_t n_kv, int32_t head_dim,
                                                  const void *pos, int32_t max_seq,
                                                  float scale) {
  WST_CHECK_ARG(q && k_cache && v_cache && out && pos, "wst_attn_decode_noscratch: null pointer");
  wst_status_t st = check_decode_shape("wst_attn_decode_noscratch", n_q, n_kv, head_dim, max_seq);
  if (st != WST_OK) return st;
  const long long need = static_cast<long long>(n_q) * max_splits_for(max_seq) * (head_dim + 4);
  if (need > kBuiltinScratchFloats)
    return fail(WST_ERR_INVALID_ARG,
                "wst_attn_decode_noscratch: this shape needs %lld floats of split scratch, the "
                "built-in array holds %lld; use wst_attn_decode with a caller buffer",
                need, kBuiltinScratchFloats);
  float *scratch = nullptr;
  st = builtin_scratch(&scratch);
  if (st != WST_OK) return st;
  return decode_common("wst_attn_decode_noscratch", q, k_cache, v_cache, scratch, out, n_q,
                       n_kv, head_dim, pos, max_seq, scale, false, false);
}

extern "C" wst_status_t wst_attn_decode_partial(const void *q, const void *k_cache,
                                                const void *v_cache, void *partials,
                                                void *out_partial, int32_t n_q, int32_t n_kv,
                                                int32_t head_dim, const void *len,
                                                int32_t max_seq, float scale) {
  WST_CHECK_ARG(q && k_cache && v_cache && out_partial && len && partials,
                "wst_attn_decode_partial: null pointer");
  wst_status_t st = check_decode_shape("wst_attn_decode_partial", n_q, n_kv, head_dim, max_seq);
  if (st != WST_OK) return st;
  return decode_common("wst_attn_decode_partial", q, k_cache, v_cache, partials, out_partial,
                       n_q, n_kv, head_dim, len, max_seq, scale, true, true);
}

extern "C" wst_status_t wst_attn_decode_sharded(const void *q, const void *k_cache,
                                                const void *v_cache, void *partials, void *out,
                                                int32_t n_q, int32_t n_kv, int32_t head_dim,
                                                const void *len, int32_t max_seq, float scale,
                                                const void *mailboxes, void *state,
                                                int32_t rank, int32_t world) {
  WST_CHECK_ARG(q && k_cache && v_cache && out && len && partials && mailboxes && state,
                "wst_attn_decode_sharded: null pointer");
  WST_CHECK_ARG(world >= 1 && world <= 32 && rank >= 0 && rank < world,
                "wst_attn_decode_sharded: rank / world out of range");
  wst_status_t st = check_decode_shape("wst_attn_decode_sharded", n_q, n_kv, head_dim, max_seq);
  if (st != WST_OK) return st;
  /* the kernel counts rows like wst_attn_decode_partial: `len`, not a cursor */
  return decode_common("wst_attn_decode_sharded", q, k_cache, v_cache, partials, out, n_q, n_kv,
                       head_dim, len, max_seq, scale, /*len_is_count=*/true,
                       /*partial_out=*/false, mailboxes, state, rank, world);
}

extern "C" wst_status_t wst_attn_merge_partials(const void *parts, void *out, int32_t n_parts,
                                                int32_t n_q, int32_t head_dim) {
  WST_CHECK_ARG(parts && out, "wst_attn_merge_partials: null pointer");
  WST_CHECK_ARG(n_parts > 0 && n_q > 0 && head_dim > 0,
                "wst_attn_merge_partials: non-positive shape");
  const int threads = head_dim < 256 ? ((head_dim + 31) / 32) * 32 : 256;
  merge_partials_kernel<<<n_q, threads, 0, current_stream()>>>(
      static_cast<const float *>(parts), static_cast<__half *>(out), n_parts, n_q, head_dim);
  WST_LAUNCHED("wst_attn_merge_partials");
  return WST_OK;
}

extern "C" wst_status_t wst_attn_exchange_merge(const void *my_triples, void *out,
                                                const void *mailboxes, void *state,
                                                int32_t rank, int32_t world, int32_t n_q,
                                                int32_t head_dim) {
  WST_CHECK_ARG(my_triples && out && mailboxes && state, "wst_attn_exchange_merge: null pointer");
  WST_CHECK_ARG(world >= 1 && world <= 32 && rank >= 0 && rank < world,
                "wst_attn_exchange_merge: rank / world out of range");
  WST_CHECK_ARG(n_q > 0 && head_dim > 0, "wst_attn_exchange_merge: non-positive shape");
  ExchangeArgs a{};
  a.mine = static_cast<const float *>(my_triples);
  a.out = static_cast<__half *>(out);
  a.mailboxes = static_cast<uint2 *const *>(mailboxes);
  a.state = static_cast<unsigned int *>(state);
  a.err_word = device_error_word();
  if (!a.err_word) return WST_ERR_CUDA;
  a.rank = rank;
  a.world = world;
  a.n_q = n_q;
  a.hd = head_dim;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(n_q));
  cfg.blockDim = dim3(128);
  cfg.stream = current_stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, exchange_merge_kernel, a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(WST_ERR_CUDA, "wst_attn_exchange_merge (launch): %s (%s)", cudaGetErrorString(e),
                cudaGetErrorName(e));
  return WST_OK;
}

extern "C" wst_status_t wst_b200_enable_peer_access(int32_t peer_device) {
  int dev = 0;
  WST_CUDA(cudaGetDevice(&dev));
  if (peer_device == dev) return WST_OK;
  int can = 0;
  WST_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can)
    return fail(WST_ERR_CUDA, "device %d cannot access device %d as a peer", dev, peer_device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return WST_OK;
  }
  if (e != cudaSuccess) return cuda_fail("cudaDeviceEnablePeerAccess", e);
  return WST_OK;
}

extern "C" wst_status_t wst_attn_chunk(const void *qkv, const void *k_cache,
                                       const void *v_cache, void *out, int32_t n_q,
                                       int32_t n_kv, int32_t head_dim, int32_t pos0, int32_t n,
                                       int32_t max_seq, float scale) {
  WST_CHECK_ARG(qkv && k_cache && v_cache && out, "wst_attn_chunk: null pointer");
  WST_CHECK_ARG(n_q > 0 && n_kv > 0 && head_dim > 0 && n > 0,
                "wst_attn_chunk: non-positive shape");
  WST_CHECK_ARG(n_q % n_kv == 0,
                "wst_attn_chunk: query heads must be a multiple of key/value heads");
  WST_CHECK_ARG(head_dim % 32 == 0, "wst_attn_chunk: head_dim must be a multiple of the warp size");
  WST_CHECK_ARG(head_dim <= 256, "wst_attn_chunk: head_dim too large");
  WST_CHECK_ARG(pos0 >= 0 && static_cast<long long>(pos0) + n <= max_seq,
                "wst_attn_chunk: chunk runs past cache");

  const int choice = g_kernel_choice.load();
  const bool tc_ok = choice != 1 && rows_kernel_supports(n_q, n_kv, head_dim, k_cache, v_cache) &&
                     aligned16(qkv);

  /* 128-row tcgen05 tiles when the chunk is large enough to fill the GPU with
   * them (or the prefix is short enough that it does not matter); a few tokens
   * against a long prefix go to the split-KV kernel instead. */
  bool use_prefill = tc_ok && choice != 2 && prefill_kernel_supports(n_q, n_kv, head_dim, n);
  int splits = 1;
  if (use_prefill && choice != 3 && choice != 4) {
    DeviceFacts facts;
    if (!device_facts(&facts)) return WST_ERR_CUDA;
    const int gqa = n_q / n_kv;
    splits = chunk_slices(facts.sm_count, (static_cast<long long>(n) * gqa + 127) / 128 * n_kv,
                          pos0 + n);
    /* at most one mma.sync row tile per KV head against a long prefix: the decode
     * kernel's row-block form streams that better than a 128-row tcgen05 tile */
    if (splits > 1 && n * gqa <= 16) use_prefill = false;
  }
  if (use_prefill) {
    PrefillLaunch P;
    P.name = "wst_attn_chunk";
    P.qkv = static_cast<const float *>(qkv);
    P.q_tok_stride = static_cast<long long>(n_q + 2 * n_kv) * head_dim;
    P.k = static_cast<const __half *>(k_cache);
    P.v = static_cast<const __half *>(v_cache);
    P.out = static_cast<__half *>(out);
    P.n_q = n_q; P.n_kv = n_kv; P.hd = head_dim;
    P.pos0 = pos0; P.n = n; P.max_seq = max_seq; P.scale = scale;
    P.force_pair = choice == 4 ? 1 : (choice == 3 ? -1 : 0);
    if (splits > 1) {
      const char *why = "";
      P.scratch = chunk_workspace(&why);
      P.scratch_floats = P.scratch ? kChunkWorkspaceFloats : 0;
      P.n_splits = splits;
      P.max_len = pos0 + n;
      if (!P.scratch) note_unsplit("wst_attn_chunk", why);
    }
    return launch_prefill(P);
  }

  RowsLaunch L;
  L.name = "wst_attn_chunk";
  L.q = static_cast<const float *>(qkv);
  L.q_tok_stride = static_cast<long long>(n_q + 2 * n_kv) * head_dim;
  L.k = static_cast<const __half *>(k_cache);
  L.v = static_cast<const __half *>(v_cache);
  L.max_seq = max_seq;
  L.pos0_val = pos0;
  L.n_seq = 1;
  L.n_tok = n;
  L.n_q = n_q;
  L.n_kv = n_kv;
  L.hd = head_dim;
  L.scale = scale;
  L.max_len = pos0 + n;
  L.out = out;
  if (!tc_ok) return launch_simple(L);
  {
    const char *why = "";
    L.scratch = chunk_workspace(&why);
    L.scratch_floats = L.scratch ? kChunkWorkspaceFloats : 0;
    if (!L.scratch && pos0 + n > 2 * kRowsTile) note_unsplit("wst_attn_chunk", why);
  }
  return launch_rows(L);
}

/* wst_attn_chunk_batch and its form with fp16 query rows (q16: `qkv` is a packed
 * [tokens][n_q * head_dim] half buffer, as the fused projection leaves it). */
static wst_status_t chunk_batch_common(const void *qkv, bool q16, const void *k_cache,
                                       const void *v_cache, void *out, const void *seq_pos0,
                                       int32_t n_seq, int32_t n_q, int32_t n_kv, int32_t head_dim,
                                       int32_t n, int32_t max_seq, float scale) {
  WST_CHECK_ARG(qkv && k_cache && v_cache && out && seq_pos0, "wst_attn_chunk_batch: null pointer");
  WST_CHECK_ARG(n_q > 0 && n_kv > 0 && head_dim > 0 && n > 0 && n_seq > 0,
                "wst_attn_chunk_batch: non-positive shape");
  WST_CHECK_ARG(n_q % n_kv == 0,
                "wst_attn_chunk_batch: query heads must be a multiple of key/value heads");
  WST_CHECK_ARG(n <= max_seq, "wst_attn_chunk_batch: chunk longer than the cache");
  if (!rows_kernel_supports(n_q, n_kv, head_dim, k_cache, v_cache) || !aligned16(qkv) ||
      !aligned16(out))
    return fail(WST_ERR_SHAPE,
                "wst_attn_chunk_batch: needs head_dim 64 or 128, at most 64 query heads per KV "
                "head and 16-byte aligned buffers");
  const long long q_stride =
      q16 ? static_cast<long long>(n_q) * head_dim : static_cast<long long>(n_q + 2 * n_kv) * head_dim;
  const int choice = g_kernel_choice.load();
  bool use_prefill = choice != 2 && prefill_kernel_supports(n_q, n_kv, head_dim, n);
  if (use_prefill && choice != 3 && choice != 4 && !q16) {
    const int gqa = n_q / n_kv;
    use_prefill = (static_cast<long long>(n) * gqa + 127) / 128 * n_kv * n_seq >= 32;
  }
  if (q16 && !use_prefill)
    return fail(WST_ERR_SHAPE,
                "wst_b200_attn_chunk_batch_q16: fp16 query rows are taken by the tensor-core "
                "kernels only (chunks of at least 128 query rows per KV head)");
  if (use_prefill) {
    PrefillLaunch P;
    P.name = "wst_attn_chunk_batch";
    P.qkv = static_cast<const float *>(qkv);
    P.q16 = q16;
    P.q_tok_stride = q_stride;
    P.k = static_cast<const __half *>(k_cache);
    P.v = static_cast<const __half *>(v_cache);
    P.out = static_cast<__half *>(out);
    P.pos0_dev = static_cast<const int32_t *>(seq_pos0);
    P.n_seq = n_seq;
    P.n_q = n_q; P.n_kv = n_kv; P.hd = head_dim;
    P.n = n; P.max_seq = max_seq; P.scale = scale;
    P.force_pair = choice == 4 ? 1 : (choice == 3 ? -1 : 0);
    if (choice != 3 && choice != 4) {
      /* too few (unit, query tile) pairs to fill the GPU: cut every tile's visible
       * prefix into equal slices (the chunk starts are device data, so the cut is made
       * in the kernel, per tile) */
      DeviceFacts facts;
      if (!device_facts(&facts)) return WST_ERR_CUDA;
      const int gqa = n_q / n_kv;
      const int splits = chunk_slices(
          facts.sm_count, (static_cast<long long>(n) * gqa + 127) / 128 * n_kv * n_seq, max_seq);
      if (splits > 1) {
        const char *why = "";
        P.scratch = chunk_workspace(&why);
        P.scratch_floats = P.scratch ? kChunkWorkspaceFloats : 0;
        P.n_splits = splits;
        P.even_slices = true;
        if (!P.scratch) note_unsplit("wst_attn_chunk_batch", why);
      }
    }
    return launch_prefill(P);
  }
  /* few tokens per sequence: the split-KV kernel, one grid over all sequences.
   * Token t of sequence s sits at row s*n + t of qkv and out. */
  RowsLaunch L;
  L.name = "wst_attn_chunk_batch";
  L.q = static_cast<const float *>(qkv);
  L.q_tok_stride = q_stride;
  L.k = static_cast<const __half *>(k_cache);
  L.v = static_cast<const __half *>(v_cache);
  L.max_seq = max_seq;
  L.pos0_dev = static_cast<const int32_t *>(seq_pos0);
  L.clamp_pos0_nonneg = true;
  L.n_seq = n_seq;
  L.n_tok = n;
  L.tok_seq_stride = n;
  L.n_q = n_q;
  L.n_kv = n_kv;
  L.hd = head_dim;
  L.scale = scale;
  L.max_len = max_seq;
  L.out = out;
  {
    const char *why = "";
    L.scratch = chunk_workspace(&why);
    L.scratch_floats = L.scratch ? kChunkWorkspaceFloats : 0;
    if (!L.scratch && max_seq > 2 * kRowsTile) note_unsplit("wst_attn_chunk_batch", why);
  }
  return launch_rows(L);
}

extern "C" wst_status_t wst_attn_chunk_batch(const void *qkv, const void *k_cache,
                                             const void *v_cache, void *out,
                                             const void *seq_pos0, int32_t n_seq, int32_t n_q,
                                             int32_t n_kv, int32_t head_dim, int32_t n,
                                             int32_t max_seq, float scale) {
  return chunk_batch_common(qkv, false, k_cache, v_cache, out, seq_pos0, n_seq, n_q, n_kv, head_dim,
                            n, max_seq, scale);
}

extern "C" wst_status_t wst_b200_attn_chunk_batch_q16(const void *q16, const void *k_cache,
                                                      const void *v_cache, void *out,
                                                      const void *seq_pos0, int32_t n_seq,
                                                      int32_t n_q, int32_t n_kv, int32_t head_dim,
                                                      int32_t n, int32_t max_seq, float scale) {
  return chunk_batch_common(q16, true, k_cache, v_cache, out, seq_pos0, n_seq, n_q, n_kv, head_dim,
                            n, max_seq, scale);
}

extern "C" int64_t wst_attn_verify_scratch_floats(int32_t n_seq, int32_t max_tokens_per_seq,
                                                  int32_t n_q, int32_t n_kv, int32_t head_dim,
                                                  int32_t max_len) {
  if (n_seq <= 0 || max_tokens_per_seq <= 0 || n_q <= 0 || n_kv <= 0 || head_dim <= 0 ||
      max_len <= 0 || n_q % n_kv != 0)
    return 0;
  /* every (sequence, KV head, row block) may be cut into the maximum number of
   * slices; rows per block never exceed 64 */
  const int gqa = n_q / n_kv;
  const long long rows_total =
      static_cast<long long>(n_seq) * n_kv *
      (static_cast<long long>(max_tokens_per_seq) * gqa + 63);
  return rows_total * max_splits_for(max_len) * (head_dim + 4);
}

extern "C" wst_status_t wst_attn_verify_paged(const void *qkv, const void *k_pool,
                                              const void *v_pool, const void *page_table,
                                              const void *seq_pos0, const void *cu_tokens,
                                              void *scratch, void *out, int32_t n_seq,
                                              int32_t total_tokens, int32_t max_tokens_per_seq,
                                              int32_t max_pages, int32_t page_size,
                                              int32_t n_pool_pages, int32_t n_q, int32_t n_kv,
                                              int32_t head_dim, int32_t max_len, float scale) {
  WST_CHECK_ARG(qkv && k_pool && v_pool && page_table && seq_pos0 && cu_tokens && scratch && out,
                "wst_attn_verify_paged: null pointer");
  WST_CHECK_ARG(n_seq > 0 && total_tokens > 0 && max_tokens_per_seq > 0 && n_q > 0 && n_kv > 0,
                "wst_attn_verify_paged: non-positive shape");
  WST_CHECK_ARG(n_q % n_kv == 0,
                "wst_attn_verify_paged: query heads must be a multiple of key/value heads");
  WST_CHECK_ARG(page_size == 16, "wst_attn_verify_paged: page_size must be 16");
  WST_CHECK_ARG(max_pages > 0 && n_pool_pages > 0 && max_len > 0,
                "wst_attn_verify_paged: empty page table or pool");
  WST_CHECK_ARG(static_cast<long long>(max_pages) * page_size >= max_len,
                "wst_attn_verify_paged: page table shorter than max_len");
  if (!rows_kernel_supports(n_q, n_kv, head_dim, k_pool, v_pool) || !aligned16(qkv))
    return fail(WST_ERR_SHAPE,
                "wst_attn_verify_paged: needs head_dim 64 or 128, at most 64 query heads per "
                "KV head and 16-byte aligned buffers");
  if (g_kernel_choice.load() != 2 &&
      prefill_split_supports(n_q, n_kv, head_dim, max_tokens_per_seq)) {
    /* all query rows of a (sequence, KV head) unit fit one 128-row tcgen05 tile */
    DeviceFacts facts;
    if (!device_facts(&facts)) return WST_ERR_CUDA;
    PrefillLaunch P;
    P.name = "wst_attn_verify_paged";
    P.qkv = static_cast<const float *>(qkv);
    P.q_tok_stride = static_cast<long long>(n_q + 2 * n_kv) * head_dim;
    P.k = static_cast<const __half *>(k_pool);
    P.v = static_cast<const __half *>(v_pool);
    P.out = static_cast<__half *>(out);
    P.pos0_dev = static_cast<const int32_t *>(seq_pos0);
    P.cu_tokens = static_cast<const int32_t *>(cu_tokens);
    P.page_table = static_cast<const int32_t *>(page_table);
    P.max_pages = max_pages;
    P.n_pool_pages = n_pool_pages;
    P.n_seq = n_seq;
    P.n_q = n_q; P.n_kv = n_kv; P.hd = head_dim;
    P.n = max_tokens_per_seq;
    P.max_seq = max_pages * page_size;
    P.scale = scale;
    P.scratch = static_cast<float *>(scratch);
    P.scratch_floats =
        wst_attn_verify_scratch_floats(n_seq, max_tokens_per_seq, n_q, n_kv, head_dim, max_len);
    P.max_len = max_len;
    /* the span kernel needs room for at least two slices per unit in the scratch
     * (a tiny batch against a short prefix has less: the sliced schedule takes it) */
    const long long units = static_cast<long long>(n_seq) * n_kv;
    const long long slice_floats =
        units * max_tokens_per_seq * (n_q / n_kv) * (static_cast<long long>(head_dim) + 4);
    const bool span_fits = (P.scratch_floats - units) / slice_floats >= 2;
    if (g_kernel_choice.load() != 3 && span_fits) {
      /* one persistent CTA per SM over equal spans of all units' KV tiles */
      P.span_ctas = rows_tuning().verify_ctas;
      return launch_verify_span(P);
    }
    /* kernel choice 3: one CTA per slice of about 2048 positions (contiguous runs of 16
     * tiles), the older schedule: sequences get as many working CTAs as their length
     * asks for; more, shorter slices only when the batch is too small to fill the GPU */
    int splits = facts.sm_count / (n_seq * n_kv);
    const int by_len = (max_len + 2047) / 2048;
    if (splits < by_len) splits = by_len;
    const int tiles = (max_len + 127) / 128;
    if (splits > tiles) splits = tiles;
    if (splits > kRowsMaxSplits) splits = kRowsMaxSplits;
    P.n_splits = splits < 1 ? 1 : splits;
    return launch_prefill(P);
  }
  RowsLaunch L;
  L.name = "wst_attn_verify_paged";
  L.q = static_cast<const float *>(qkv);
  L.q_tok_stride = static_cast<long long>(n_q + 2 * n_kv) * head_dim;
  L.k = static_cast<const __half *>(k_pool);
  L.v = static_cast<const __half *>(v_pool);
  L.paged = true;
  L.max_seq = max_pages * page_size;
  L.page_table = static_cast<const int32_t *>(page_table);
  L.max_pages = max_pages;
  L.n_pool_pages = n_pool_pages;
  L.pos0_dev = static_cast<const int32_t *>(seq_pos0);
  L.cu_tokens = static_cast<const int32_t *>(cu_tokens);
  L.n_seq = n_seq;
  L.n_tok = max_tokens_per_seq;
  L.n_q = n_q;
  L.n_kv = n_kv;
  L.hd = head_dim;
  L.scale = scale;
  L.scratch = static_cast<float *>(scratch);
  L.scratch_floats =
      wst_attn_verify_scratch_floats(n_seq, max_tokens_per_seq, n_q, n_kv, head_dim, max_len);
  L.max_len = max_len;
  L.out = out;
  return launch_rows(L);
}
