/* Kernel set 1: per-head RMSNorm (optional) + half-rotation RoPE + KV-cache
 * append, for one token (wst_rope_cache), a chunk (wst_rope_cache_chunk) and a
 * ragged batch over a paged cache (wst_rope_cache_paged).
 *
 * The work is pure HBM traffic (read the fused projection once, write q back,
 * write two cache rows), so the layout is chosen for coalescing: one warp owns
 * one (token, head) vector; lane l holds elements [l*E, l*E+E) of the first
 * half and the same elements of the second half -- exactly the pairs the
 * half-rotation couples -- so every load and store of a warp is one contiguous
 * run, the norm's sum of squares is a warp shuffle reduction with no shared
 * memory or block barrier, and a head never leaves registers.
 *
 * Semantics follow cuda/decode.cu:112-178 and cuda/chunk_ops.cu:101-150 of the
 * engine: norm before rotation, per head, q and k with their own fp16 gains, v
 * copied unrotated and un-normed; q written back in place as fp32; k and v
 * narrowed to fp16 into cache row `pos`; positions clamped, never trusted.
 */

#include "attn_rows.cuh"
#include "wst_common.cuh"

namespace wst {
namespace {

constexpr int kWarpsPerBlock = 8;

struct RopeArgs {
  float *qkv;            /* [n_tokens][row_stride] */
  __half *k_cache;       /* contiguous: [n_kv][max_seq][hd]; paged: the pool */
  __half *v_cache;
  const float *cos_tab;  /* [table_len][hd/2] */
  const float *sin_tab;
  const __half *q_gain;  /* [hd] or null */
  const __half *k_gain;
  const int32_t *pos_dev;     /* decode: device cursor, else null */
  const int32_t *page_table;  /* paged only: [n_seq][max_pages] */
  const int32_t *seq_pos0;    /* paged only: [n_seq] */
  const int32_t *cu_tokens;   /* paged only: [n_seq + 1] */
  int n_q, n_kv, hd;
  int n_tokens;
  int pos0;       /* chunk: position of token 0 */
  int max_seq;    /* contiguous: rows per head */
  int table_len;  /* rows in cos/sin */
  int n_seq, max_pages, page_size, n_pool_pages;
  int n_per_seq; /* contiguous batch: tokens per sequence (0 = single sequence) */
  float eps;
  int trigger_early; /* set by the launcher: single-token append under programmatic launch */
  /* fp8 cache: k_cache / v_cache are e4m3 bytes; a row is stored as value * inv_scale */
  int kv8;
  float k_inv_scale, v_inv_scale;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int E>
__device__ __forceinline__ void load_vec(const float *p, float (&x)[E]) {
  if constexpr (E == 4) {
    float4 t = *reinterpret_cast<const float4 *>(p);
    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
  } else if constexpr (E == 2) {
    float2 t = *reinterpret_cast<const float2 *>(p);
    x[0] = t.x; x[1] = t.y;
  } else {
    x[0] = *p;
  }
}

template <int E>
__device__ __forceinline__ void store_vec(float *p, const float (&x)[E]) {
  if constexpr (E == 4) {
    *reinterpret_cast<float4 *>(p) = make_float4(x[0], x[1], x[2], x[3]);
  } else if constexpr (E == 2) {
    *reinterpret_cast<float2 *>(p) = make_float2(x[0], x[1]);
  } else {
    *p = x[0];
  }
}

template <int E>
__device__ __forceinline__ void store_half_vec(__half *p, const float (&x)[E]) {
  if constexpr (E == 4) {
    __half2 a = __floats2half2_rn(x[0], x[1]);
    __half2 b = __floats2half2_rn(x[2], x[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t *>(&a);
    t.y = *reinterpret_cast<uint32_t *>(&b);
    *reinterpret_cast<uint2 *>(p) = t;
  } else if constexpr (E == 2) {
    *reinterpret_cast<__half2 *>(p) = __floats2half2_rn(x[0], x[1]);
  } else {
    *p = __float2half_rn(x[0]);
  }
}

/* E values -> e4m3 (round to nearest, saturating) at byte offset `at` of an fp8 cache */
template <int E>
__device__ __forceinline__ void store_fp8_vec(__half *cache, long long at, const float (&x)[E],
                                              float inv_scale) {
  uint8_t *dst = reinterpret_cast<uint8_t *>(cache) + at;
  if constexpr (E >= 2) {
#pragma unroll
    for (int e = 0; e < E; e += 2) {
      unsigned short two;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(two) : "f"(x[e] * inv_scale), "f"(x[e + 1] * inv_scale));
      *reinterpret_cast<unsigned short *>(dst + e) = two;
    }
  } else {
    unsigned short two;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(two) : "f"(x[0] * inv_scale), "f"(0.f));
    dst[0] = static_cast<uint8_t>(two & 0xFF);
  }
}

template <int E>
__device__ __forceinline__ void load_gain(const __half *p, float (&g)[E]) {
#pragma unroll
  for (int e = 0; e < E; ++e) g[e] = __half2float(p[e]);
}

/* Where token `tok` lives: its cache position, and for the paged layout the
 * element offset of its row 0 / head 0 in the pool (-1 = do not write). */
struct TokenPlace {
  int pos;             /* cache position (already clamped for contiguous) */
  long long kv_base;   /* element offset of [kvh=0] row for this token, or -1 */
  long long kv_head_stride;
};

template <bool PAGED>
__device__ __forceinline__ TokenPlace place_token(const RopeArgs &a, int tok) {
  TokenPlace t;
  if constexpr (!PAGED) {
    int p;
    long long seq_base = 0;
    if (a.n_per_seq > 0) { /* batch of contiguous caches [n_seq][n_kv][max_seq][hd] */
      const int sq = tok / a.n_per_seq;
      p = a.seq_pos0[sq] + (tok - sq * a.n_per_seq);
      p = p < 0 ? 0 : p;
      seq_base = static_cast<long long>(sq) * a.n_kv * a.max_seq * a.hd;
    } else if (a.pos_dev) {
      p = *a.pos_dev;
      p = p < 0 ? 0 : p;
    } else {
      p = a.pos0 + tok;
    }
    p = p < a.max_seq - 1 ? p : a.max_seq - 1;
    t.pos = p;
    t.kv_base = seq_base + static_cast<long long>(p) * a.hd;
    t.kv_head_stride = static_cast<long long>(a.max_seq) * a.hd;
  } else {
    /* binary search: largest s with cu_tokens[s] <= tok */
    int lo = 0, hi = a.n_seq - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (a.cu_tokens[mid] <= tok) lo = mid; else hi = mid - 1;
    }
    const int s = lo;
    int p = a.seq_pos0[s] + (tok - a.cu_tokens[s]);
    p = p < 0 ? 0 : p;
    t.pos = p;
    const int slot = p / a.page_size;
    t.kv_base = -1;
    t.kv_head_stride = static_cast<long long>(a.page_size) * a.hd;
    if (slot < a.max_pages) {
      const int page = a.page_table[static_cast<long long>(s) * a.max_pages + slot];
      if (page >= 0 && page < a.n_pool_pages) {
        t.kv_base = (static_cast<long long>(page) * a.n_kv * a.page_size + (p % a.page_size)) *
                    a.hd;
      }
    }
  }
  return t;
}

/* Fast path: head_dim = 64 * E, everything in registers. */
template <int E, bool PAGED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rope_append_kernel(const RopeArgs a) {
  /* Under programmatic dependent launch: a single-token append lets the next
   * kernel in the stream (the decode attention, which re-reads the one row
   * written here after its own wait) start its prologue right away. */
  if (a.trigger_early && !PAGED) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  /* paged (verify): the kernel behind reads the batch description and old cache rows
   * before its own dependency resolves, so it is released only now, when everything ahead
   * of this append in the stream has completed */
  if (a.trigger_early && PAGED) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int HD = 64 * E;
  constexpr int HALF = HD / 2;
  const int lane = threadIdx.x & 31;
  const int heads = a.n_q + a.n_kv;
  const long long unit =
      static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (unit >= static_cast<long long>(a.n_tokens) * heads) return;
  const int tok = static_cast<int>(unit / heads);
  const int head = static_cast<int>(unit % heads);

  const TokenPlace place = place_token<PAGED>(a, tok);
  const int tpos = place.pos < a.table_len - 1 ? place.pos : a.table_len - 1;

  float *row = a.qkv + static_cast<long long>(tok) * (a.n_q + 2 * a.n_kv) * HD;
  const bool is_q = head < a.n_q;
  const int kvh = head - a.n_q;
  float *vec = is_q ? row + head * HD : row + (a.n_q + kvh) * HD;
  const __half *gain = is_q ? a.q_gain : a.k_gain;

  const int i0 = lane * E;
  float x1[E], x2[E], c[E], s[E];
  load_vec<E>(vec + i0, x1);
  load_vec<E>(vec + HALF + i0, x2);
  load_vec<E>(a.cos_tab + static_cast<long long>(tpos) * HALF + i0, c);
  load_vec<E>(a.sin_tab + static_cast<long long>(tpos) * HALF + i0, s);

  if (gain) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) ss = fmaf(x1[e], x1[e], fmaf(x2[e], x2[e], ss));
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(HD) + a.eps);
    float g1[E], g2[E];
    load_gain<E>(gain + i0, g1);
    load_gain<E>(gain + HALF + i0, g2);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      x1[e] = x1[e] * inv * g1[e];
      x2[e] = x2[e] * inv * g2[e];
    }
  }

  float y1[E], y2[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    y1[e] = x1[e] * c[e] - x2[e] * s[e];
    y2[e] = x2[e] * c[e] + x1[e] * s[e];
  }

  if (is_q) {
    store_vec<E>(vec + i0, y1);
    store_vec<E>(vec + HALF + i0, y2);
    return;
  }

  if (place.kv_base < 0) return;
  const long long slot = place.kv_base + static_cast<long long>(kvh) * place.kv_head_stride;
  const float *vsrc = row + (a.n_q + a.n_kv + kvh) * HD;
  float v1[E], v2[E];
  load_vec<E>(vsrc + i0, v1);
  load_vec<E>(vsrc + HALF + i0, v2);
  if (a.kv8) { /* element offsets are byte offsets in an e4m3 cache */
    store_fp8_vec<E>(a.k_cache, slot + i0, y1, a.k_inv_scale);
    store_fp8_vec<E>(a.k_cache, slot + HALF + i0, y2, a.k_inv_scale);
    store_fp8_vec<E>(a.v_cache, slot + i0, v1, a.v_inv_scale);
    store_fp8_vec<E>(a.v_cache, slot + HALF + i0, v2, a.v_inv_scale);
    return;
  }
  store_half_vec<E>(a.k_cache + slot + i0, y1);
  store_half_vec<E>(a.k_cache + slot + HALF + i0, y2);
  store_half_vec<E>(a.v_cache + slot + i0, v1);
  store_half_vec<E>(a.v_cache + slot + HALF + i0, v2);
}

/* Chunks: one warp takes G consecutive heads of one token.  With one (token, head)
 * per warp a warp moves 1 KB and leaves, and a chunk of 2048 tokens x 40 heads is
 * 12,288 blocks of 8 KB each: the launch ran at two thirds of the HBM rate, bound
 * by block turnover and by a single dependent load -> reduce -> store chain per warp.
 * Here the loads of all G heads (and of the V rows that go with K heads) are in
 * flight together and the token's cos/sin row is fetched once. */
template <int E, int G>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rope_append_group_kernel(const RopeArgs a) {
  constexpr int HD = 64 * E;
  constexpr int HALF = HD / 2;
  const int lane = threadIdx.x & 31;
  const int heads = a.n_q + a.n_kv;
  const int groups = heads / G; /* the launcher checked heads % G == 0 */
  const long long grp =
      static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (grp >= static_cast<long long>(a.n_tokens) * groups) return;
  const int tok = static_cast<int>(grp / groups);
  const int head0 = static_cast<int>(grp % groups) * G;

  const TokenPlace place = place_token<false>(a, tok);
  const int tpos = place.pos < a.table_len - 1 ? place.pos : a.table_len - 1;
  float *row = a.qkv + static_cast<long long>(tok) * (a.n_q + 2 * a.n_kv) * HD;
  const int i0 = lane * E;

  float x1[G][E], x2[G][E], v1[G][E], v2[G][E], c[E], s[E];
#pragma unroll
  for (int g = 0; g < G; ++g) { /* q heads and k heads are consecutive in the row */
    load_vec<E>(row + (head0 + g) * HD + i0, x1[g]);
    load_vec<E>(row + (head0 + g) * HD + HALF + i0, x2[g]);
  }
  load_vec<E>(a.cos_tab + static_cast<long long>(tpos) * HALF + i0, c);
  load_vec<E>(a.sin_tab + static_cast<long long>(tpos) * HALF + i0, s);
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (head0 + g >= a.n_q) {
      const float *vsrc = row + (head0 + g + a.n_kv) * HD;
      load_vec<E>(vsrc + i0, v1[g]);
      load_vec<E>(vsrc + HALF + i0, v2[g]);
    }
  }

#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int head = head0 + g;
    const bool is_q = head < a.n_q;
    const __half *gain = is_q ? a.q_gain : a.k_gain;
    if (gain) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) ss = fmaf(x1[g][e], x1[g][e], fmaf(x2[g][e], x2[g][e], ss));
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / static_cast<float>(HD) + a.eps);
      float g1[E], g2[E];
      load_gain<E>(gain + i0, g1);
      load_gain<E>(gain + HALF + i0, g2);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        x1[g][e] = x1[g][e] * inv * g1[e];
        x2[g][e] = x2[g][e] * inv * g2[e];
      }
    }
    float y1[E], y2[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      y1[e] = x1[g][e] * c[e] - x2[g][e] * s[e];
      y2[e] = x2[g][e] * c[e] + x1[g][e] * s[e];
    }
    if (is_q) {
      store_vec<E>(row + head * HD + i0, y1);
      store_vec<E>(row + head * HD + HALF + i0, y2);
    } else if (place.kv_base >= 0) {
      const long long slot =
          place.kv_base + static_cast<long long>(head - a.n_q) * place.kv_head_stride;
      if (a.kv8) {
        store_fp8_vec<E>(a.k_cache, slot + i0, y1, a.k_inv_scale);
        store_fp8_vec<E>(a.k_cache, slot + HALF + i0, y2, a.k_inv_scale);
        store_fp8_vec<E>(a.v_cache, slot + i0, v1[g], a.v_inv_scale);
        store_fp8_vec<E>(a.v_cache, slot + HALF + i0, v2[g], a.v_inv_scale);
      } else {
        store_half_vec<E>(a.k_cache + slot + i0, y1);
        store_half_vec<E>(a.k_cache + slot + HALF + i0, y2);
        store_half_vec<E>(a.v_cache + slot + i0, v1[g]);
        store_half_vec<E>(a.v_cache + slot + HALF + i0, v2[g]);
      }
    }
  }
}

/* Any even head_dim: two passes over the vector (the second hits L1). */
template <bool PAGED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rope_append_any_kernel(const RopeArgs a) {
  /* may be launched with programmatic stream serialization like the fast path */
  if (a.trigger_early && !PAGED) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (a.trigger_early && PAGED) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int hd = a.hd, half = hd >> 1;
  const int lane = threadIdx.x & 31;
  const int heads = a.n_q + a.n_kv;
  const long long unit =
      static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (unit >= static_cast<long long>(a.n_tokens) * heads) return;
  const int tok = static_cast<int>(unit / heads);
  const int head = static_cast<int>(unit % heads);

  const TokenPlace place = place_token<PAGED>(a, tok);
  const int tpos = place.pos < a.table_len - 1 ? place.pos : a.table_len - 1;
  const float *ct = a.cos_tab + static_cast<long long>(tpos) * half;
  const float *st = a.sin_tab + static_cast<long long>(tpos) * half;

  float *row = a.qkv + static_cast<long long>(tok) * (a.n_q + 2 * a.n_kv) * hd;
  const bool is_q = head < a.n_q;
  const int kvh = head - a.n_q;
  float *vec = is_q ? row + head * hd : row + (a.n_q + kvh) * hd;
  const __half *gain = is_q ? a.q_gain : a.k_gain;

  float inv = 1.f;
  if (gain) {
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) ss = fmaf(vec[i], vec[i], ss);
    ss = warp_sum(ss);
    inv = rsqrtf(ss / static_cast<float>(hd) + a.eps);
  }
  const bool write_kv = !is_q && place.kv_base >= 0;
  const long long slot =
      write_kv ? place.kv_base + static_cast<long long>(kvh) * place.kv_head_stride : 0;
  for (int i = lane; i < half; i += 32) {
    float x1 = vec[i], x2 = vec[i + half];
    if (gain) {
      x1 = x1 * inv * __half2float(gain[i]);
      x2 = x2 * inv * __half2float(gain[i + half]);
    }
    const float c = ct[i], s = st[i];
    const float y1 = x1 * c - x2 * s;
    const float y2 = x2 * c + x1 * s;
    if (is_q) {
      vec[i] = y1;
      vec[i + half] = y2;
    } else if (write_kv) {
      a.k_cache[slot + i] = __float2half_rn(y1);
      a.k_cache[slot + i + half] = __float2half_rn(y2);
    }
  }
  if (write_kv) {
    const float *vsrc = row + (a.n_q + a.n_kv + kvh) * hd;
    for (int i = lane; i < hd; i += 32) a.v_cache[slot + i] = __float2half_rn(vsrc[i]);
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <bool PAGED>
wst_status_t launch_rope(const RopeArgs &a, const char *name) {
  const long long units = static_cast<long long>(a.n_tokens) * (a.n_q + a.n_kv);
  const long long blocks = (units + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffLL) return fail(WST_ERR_INVALID_ARG, "%s: too many tokens", name);
  const dim3 grid(static_cast<unsigned>(blocks)), block(kWarpsPerBlock * 32);
  cudaStream_t st = current_stream();
  /* The vector path needs 16-byte aligned rows; fp32 rows of 64*E floats and
   * cudaMalloc'd bases give that, an odd caller offset falls back. */
  const bool vec_ok = aligned16(a.qkv) && aligned16(a.k_cache) && aligned16(a.v_cache) &&
                      aligned16(a.cos_tab) && aligned16(a.sin_tab) &&
                      (!a.q_gain || aligned16(a.q_gain)) && (!a.k_gain || aligned16(a.k_gain));
  /* A single-token append (decode) and the ragged paged append (verify) are launched
   * with programmatic stream serialization and let their dependents start early; other
   * appends are ordinary launches, complete before anything after them starts. */
  RopeArgs args = a;
  args.trigger_early = 0;
  if (!PAGED && a.n_tokens == 1 && vec_ok && decode_overlap_allowed()) args.trigger_early = 1;
  /* the ragged paged append: the verify kernel behind it reads, before its own
   * dependency resolves, only what this kernel does not write */
  if (PAGED && decode_overlap_allowed()) args.trigger_early = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = args.trigger_early ? 1 : 0;
  if (a.kv8 && !(vec_ok && (a.hd == 64 || a.hd == 128 || a.hd == 256)))
    return fail(WST_ERR_SHAPE, "%s: the fp8 cache needs head_dim 64, 128 or 256 and aligned buffers",
                name);
  cudaError_t e;
  constexpr int kGroup = 4;
  const bool grouped = !PAGED && vec_ok && a.n_tokens >= 32 && (a.n_q + a.n_kv) % kGroup == 0 &&
                       (a.hd == 64 || a.hd == 128 || a.hd == 256);
  if (grouped) {
    const long long groups = units / kGroup;
    cfg.gridDim = dim3(static_cast<unsigned>((groups + kWarpsPerBlock - 1) / kWarpsPerBlock));
    e = a.hd == 64    ? cudaLaunchKernelEx(&cfg, rope_append_group_kernel<1, kGroup>, args)
        : a.hd == 128 ? cudaLaunchKernelEx(&cfg, rope_append_group_kernel<2, kGroup>, args)
                      : cudaLaunchKernelEx(&cfg, rope_append_group_kernel<4, kGroup>, args);
  } else if (vec_ok && a.hd == 64) {
    e = cudaLaunchKernelEx(&cfg, rope_append_kernel<1, PAGED>, args);
  } else if (vec_ok && a.hd == 128) {
    e = cudaLaunchKernelEx(&cfg, rope_append_kernel<2, PAGED>, args);
  } else if (vec_ok && a.hd == 256) {
    e = cudaLaunchKernelEx(&cfg, rope_append_kernel<4, PAGED>, args);
  } else {
    e = cudaLaunchKernelEx(&cfg, rope_append_any_kernel<PAGED>, args);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(WST_ERR_CUDA, "%s (launch): %s (%s)", name,
                                    cudaGetErrorString(e), cudaGetErrorName(e));
  return WST_OK;
}

}  // namespace
}  // namespace wst

using namespace wst;

extern "C" wst_status_t wst_rope_cache(void *qkv, void *k_cache, void *v_cache,
                                       const void *cos_tab, const void *sin_tab, int32_t n_q,
                                       int32_t n_kv, int32_t head_dim, const void *pos,
                                       int32_t max_seq, const void *q_norm_w,
                                       const void *k_norm_w, float eps) {
  WST_CHECK_ARG(qkv && k_cache && v_cache && cos_tab && sin_tab && pos,
                "wst_rope_cache: null pointer");
  WST_CHECK_ARG(n_q > 0 && n_kv > 0 && head_dim > 0, "wst_rope_cache: non-positive shape");
  WST_CHECK_ARG(head_dim % 2 == 0, "wst_rope_cache: head_dim must be even");
  WST_CHECK_ARG(max_seq > 0, "wst_rope_cache: empty cache");
  WST_CHECK_ARG(head_dim / 2 <= 1024, "wst_rope_cache: head_dim/2 exceeds a block");
  RopeArgs a{};
  a.qkv = static_cast<float *>(qkv);
  a.k_cache = static_cast<__half *>(k_cache);
  a.v_cache = static_cast<__half *>(v_cache);
  a.cos_tab = static_cast<const float *>(cos_tab);
  a.sin_tab = static_cast<const float *>(sin_tab);
  a.q_gain = static_cast<const __half *>(q_norm_w);
  a.k_gain = static_cast<const __half *>(k_norm_w);
  a.pos_dev = static_cast<const int32_t *>(pos);
  a.n_q = n_q; a.n_kv = n_kv; a.hd = head_dim;
  a.n_tokens = 1; a.pos0 = 0; a.max_seq = max_seq; a.table_len = max_seq;
  a.eps = eps;
  return launch_rope<false>(a, "wst_rope_cache");
}

extern "C" wst_status_t wst_rope_cache_chunk(void *qkv, void *k_cache, void *v_cache,
                                             const void *cos_tab, const void *sin_tab,
                                             int32_t n_q, int32_t n_kv, int32_t head_dim,
                                             int32_t pos0, int32_t n, int32_t max_seq,
                                             const void *q_norm_w, const void *k_norm_w,
                                             float eps) {
  WST_CHECK_ARG(qkv && k_cache && v_cache && cos_tab && sin_tab,
                "wst_rope_cache_chunk: null pointer");
  WST_CHECK_ARG(n_q > 0 && n_kv > 0 && head_dim > 0 && n > 0,
                "wst_rope_cache_chunk: non-positive shape");
  WST_CHECK_ARG(head_dim % 2 == 0, "wst_rope_cache_chunk: head_dim must be even");
  WST_CHECK_ARG(pos0 >= 0 && static_cast<long long>(pos0) + n <= max_seq,
                "wst_rope_cache_chunk: chunk runs past the cache");
  WST_CHECK_ARG(head_dim / 2 <= 1024, "wst_rope_cache_chunk: head_dim/2 exceeds a block");
  RopeArgs a{};
  a.qkv = static_cast<float *>(qkv);
  a.k_cache = static_cast<__half *>(k_cache);
  a.v_cache = static_cast<__half *>(v_cache);
  a.cos_tab = static_cast<const float *>(cos_tab);
  a.sin_tab = static_cast<const float *>(sin_tab);
  a.q_gain = static_cast<const __half *>(q_norm_w);
  a.k_gain = static_cast<const __half *>(k_norm_w);
  a.pos_dev = nullptr;
  a.n_q = n_q; a.n_kv = n_kv; a.hd = head_dim;
  a.n_tokens = n; a.pos0 = pos0; a.max_seq = max_seq; a.table_len = max_seq;
  a.eps = eps;
  return launch_rope<false>(a, "wst_rope_cache_chunk");
}

extern "C" wst_status_t wst_rope_cache_paged(void *qkv, void *k_pool, void *v_pool,
                                             const void *cos_tab, const void *sin_tab,
                                             const void *page_table, const void *seq_pos0,
                                             const void *cu_tokens, int32_t n_seq,
                                             int32_t total_tokens, int32_t max_pages,
                                             int32_t page_size, int32_t n_pool_pages,
                                             int32_t n_q, int32_t n_kv, int32_t head_dim,
                                             int32_t table_len, const void *q_norm_w,
                                             const void *k_norm_w, float eps) {
  WST_CHECK_ARG(qkv && k_pool && v_pool && cos_tab && sin_tab && page_table && seq_pos0 &&
                    cu_tokens,
                "wst_rope_cache_paged: null pointer");
  WST_CHECK_ARG(n_q > 0 && n_kv > 0 && head_dim > 0 && n_seq > 0 && total_tokens > 0,
                "wst_rope_cache_paged: non-positive shape");
  WST_CHECK_ARG(head_dim % 2 == 0, "wst_rope_cache_paged: head_dim must be even");
  WST_CHECK_ARG(page_size == 16, "wst_rope_cache_paged: page_size must be 16");
  WST_CHECK_ARG(max_pages > 0 && n_pool_pages > 0 && table_len > 0,
                "wst_rope_cache_paged: empty page table, pool or RoPE table");
  RopeArgs a{};
  a.qkv = static_cast<float *>(qkv);
  a.k_cache = static_cast<__half *>(k_pool);
  a.v_cache = static_cast<__half *>(v_pool);
  a.cos_tab = static_cast<const float *>(cos_tab);
  a.sin_tab = static_cast<const float *>(sin_tab);
  a.q_gain = static_cast<const __half *>(q_norm_w);
  a.k_gain = static_cast<const __half *>(k_norm_w);
  a.page_table = static_cast<const int32_t *>(page_table);
  a.seq_pos0 = static_cast<const int32_t *>(seq_pos0);
  a.cu_tokens = static_cast<const int32_t *>(cu_tokens);
  a.n_q = n_q; a.n_kv = n_kv; a.hd = head_dim;
  a.n_tokens = total_tokens; a.table_len = table_len;
  a.n_seq = n_seq; a.max_pages = max_pages; a.page_size = page_size;
  a.n_pool_pages = n_pool_pages;
  a.eps = eps;
  return launch_rope<true>(a, "wst_rope_cache_paged");
}

extern "C" wst_status_t wst_rope_cache_chunk_batch(void *qkv, void *k_cache, void *v_cache,
                                                   const void *cos_tab, const void *sin_tab,
                                                   const void *seq_pos0, int32_t n_seq,
                                                   int32_t n_q, int32_t n_kv, int32_t head_dim,
                                                   int32_t n, int32_t max_seq,
                                                   const void *q_norm_w, const void *k_norm_w,
                                                   float eps) {
  WST_CHECK_ARG(qkv && k_cache && v_cache && cos_tab && sin_tab && seq_pos0,
                "wst_rope_cache_chunk_batch: null pointer");
  WST_CHECK_ARG(n_q > 0 && n_kv > 0 && head_dim > 0 && n > 0 && n_seq > 0,
                "wst_rope_cache_chunk_batch: non-positive shape");
  WST_CHECK_ARG(head_dim % 2 == 0, "wst_rope_cache_chunk_batch: head_dim must be even");
  WST_CHECK_ARG(n <= max_seq, "wst_rope_cache_chunk_batch: chunk longer than the cache");
  RopeArgs a{};
  a.qkv = static_cast<float *>(qkv);
  a.k_cache = static_cast<__half *>(k_cache);
  a.v_cache = static_cast<__half *>(v_cache);
  a.cos_tab = static_cast<const float *>(cos_tab);
  a.sin_tab = static_cast<const float *>(sin_tab);
  a.q_gain = static_cast<const __half *>(q_norm_w);
  a.k_gain = static_cast<const __half *>(k_norm_w);
  a.seq_pos0 = static_cast<const int32_t *>(seq_pos0);
  a.n_q = n_q; a.n_kv = n_kv; a.hd = head_dim;
  a.n_tokens = n_seq * n; a.max_seq = max_seq; a.table_len = max_seq;
  a.n_seq = n_seq; a.n_per_seq = n;
  a.eps = eps;
  return launch_rope<false>(a, "wst_rope_cache_chunk_batch");
}


/* wst_rope_cache / wst_rope_cache_chunk with an e4m3 cache: k and v rows are stored as
 * round-to-nearest e4m3 of value / scale (saturating at 448); q is written back as fp32
 * exactly as by the fp16 entry points.  No counterpart in the engine (its roadmap names
 * an 8-bit cache, docs/ROADMAP.md:206). */
extern "C" wst_status_t wst_b200_rope_cache_fp8(void *qkv, void *k_cache8, void *v_cache8,
                                                const void *cos_tab, const void *sin_tab,
                                                int32_t n_q, int32_t n_kv, int32_t head_dim,
                                                const void *pos, int32_t pos0, int32_t n,
                                                int32_t max_seq, const void *q_norm_w,
                                                const void *k_norm_w, float eps, float k_scale,
                                                float v_scale) {
  WST_CHECK_ARG(qkv && k_cache8 && v_cache8 && cos_tab && sin_tab,
                "wst_b200_rope_cache_fp8: null pointer");
  WST_CHECK_ARG(n_q > 0 && n_kv > 0 && head_dim > 0 && n > 0 && max_seq > 0,
                "wst_b200_rope_cache_fp8: non-positive shape");
  WST_CHECK_ARG(k_scale > 0.f && v_scale > 0.f, "wst_b200_rope_cache_fp8: scales must be positive");
  WST_CHECK_ARG(pos != nullptr ? n == 1
                               : (pos0 >= 0 && static_cast<long long>(pos0) + n <= max_seq),
                "wst_b200_rope_cache_fp8: one token at the device cursor, or a chunk inside the cache");
  RopeArgs a{};
  a.qkv = static_cast<float *>(qkv);
  a.k_cache = static_cast<__half *>(k_cache8);
  a.v_cache = static_cast<__half *>(v_cache8);
  a.cos_tab = static_cast<const float *>(cos_tab);
  a.sin_tab = static_cast<const float *>(sin_tab);
  a.q_gain = static_cast<const __half *>(q_norm_w);
  a.k_gain = static_cast<const __half *>(k_norm_w);
  a.pos_dev = static_cast<const int32_t *>(pos);
  a.n_q = n_q; a.n_kv = n_kv; a.hd = head_dim;
  a.n_tokens = n; a.pos0 = pos0; a.max_seq = max_seq; a.table_len = max_seq;
  a.eps = eps;
  a.kv8 = 1;
  a.k_inv_scale = 1.f / k_scale;
  a.v_inv_scale = 1.f / v_scale;
  return launch_rope<false>(a, "wst_b200_rope_cache_fp8");
}
