/* Kernel sets 3 and 4: causal chunked-prefill attention, and the ragged paged
 * verify step, on the 5th-generation tensor cores.
 *
 * Query rows are (token, head-in-group) pairs, token-major, 128 per tile -- a tile
 * covers 128/gqa consecutive tokens and all the query heads that share a KV head --
 * and a tile walks its visible prefix in tiles of 128 cache positions.  Per step:
 *
 *   S  = Q K^T   tcgen05.mma (M128 x N128 x K16 steps), K tiles as the B operand in
 *                128-byte-swizzled shared memory (TMA), fp32 accumulator in tensor
 *                memory
 *   softmax      one TMEM lane is one query row, so row maximum and row sum need no
 *                shuffles; fp32, exp2 with scale*log2(e) folded into q; P goes back
 *                into tensor memory as fp16 pairs (tcgen05.st) and is the A operand
 *                of the next MMA: P never crosses shared memory
 *   O += P V     tcgen05.mma (M128 x N(head_dim) x K16 steps) accumulating in
 *                tensor memory across tiles.  The exponent offset of a row moves
 *                only when it has to ("lazy rescale"); then the row's owner
 *                multiplies its O lane in place (tcgen05.ld / tcgen05.st).
 *
 * Two kernels:
 *   attn_prefill_kernel<HD, PAGED>   one tile per CTA.  Q too is a tensor-memory
 *       operand; S double-buffered; two softmax threads per row (8 warps), one MMA
 *       warp, one TMA warp.  Paged caches, ragged batches, and the sliced form
 *       (grid.x = query tiles x slices of the KV range, partial rows for the slice
 *       merge kernel of attn_rows.cu) for launches that cannot fill the GPU.
 *   attn_prefill_pair_kernel<HD>     two tiles of one KV head per CTA, each with a
 *       softmax warpgroup of its own (one thread per row): one tile's softmax runs
 *       under the other tile's MMAs and every K/V tile serves 256 rows.  The
 *       default for launches of at least two waves of tiles.
 * Every wait is bounded.
 *
 * Semantics: cuda/chunk_ops.cu:187-264 of the engine (query j sees cache rows
 * [0, pos0 + j]; fp32 softmax state; fp16 output).
 */

#include "attn_prefill.cuh"
#include "attn_rows.cuh"
#include "tensor_map.cuh"
#include "wst_ptx.cuh"

#include <type_traits>

namespace wst {
namespace {

using namespace ptx;

constexpr float kLog2e = 1.4426950408889634f;

template <int HD>
struct PCfg {
  static constexpr int BN = 128;               /* cache positions per tile */
  static constexpr int NH = HD / 64;           /* 128-byte column halves of a K/V/Q row */
  static constexpr int HALF_BYTES = BN * 128;  /* one half of a tile: 128 rows x 128 B */
  static constexpr int KV_BYTES = NH * HALF_BYTES;
  static constexpr int NSTAGE = HD == 128 ? 3 : 4;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + NSTAGE * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + NSTAGE * KV_BYTES;
  static constexpr int NBAR = 4 * NSTAGE + 2 + 2 + 1 + 1 + 1 + 1;
  /* after the barriers and the tensor-memory slot: three [2][128] float areas through
   * which the two threads of a query row exchange their partial maxima and sums */
  static constexpr int OFF_XCH = OFF_BAR + 256;
  static constexpr int SMEM_BYTES = OFF_XCH + 3 * 2 * 128 * 4 + 64 + 1024; /* + 64: a span's start */
  static constexpr int THREADS = 320; /* 8 softmax warps, the MMA warp, the TMA warp */
  static_assert(NBAR * 8 + 16 <= 256, "barrier area");
  /* tensor-memory columns */
  static constexpr int COL_S = 0;      /* two S buffers of BN fp32 columns */
  static constexpr int COL_O = 2 * BN; /* the output accumulator, HD fp32 columns */
  static constexpr int COL_P = 384;    /* P as the A operand of PV: 128 fp16 = 64 columns */
  static constexpr int COL_Q = 448;    /* Q as the A operand of QK^T: HD fp16 = HD/2 columns */
  static constexpr int TMEM_COLS = 512;
  static_assert(COL_O + HD <= COL_P && COL_Q + HD / 2 <= TMEM_COLS, "tensor-memory map");
};

struct PrefillArgs {
  const float *q;            /* [token][q_tok_stride], sequence s owns tokens s*n .. or cu_tokens */
  long long q_tok_stride;
  int q16;                   /* q is fp16: the pointer is reinterpreted, the stride is in halves */
  __half *out;               /* [token][n_q*hd] */
  float *scratch;            /* split mode: [unit][slice][rows_cap][hd+4] */
  const int32_t *pos0_dev;   /* per-sequence chunk start, or null: pos0 for all */
  const int32_t *cu_tokens;  /* ragged token ranges [n_seq+1], or null: n tokens each */
  const int32_t *page_table; /* paged cache: [n_seq][max_pages] */
  int max_pages, n_pool_pages;
  int n_splits, rows_cap;
  int tiles_per_slice; /* sliced mode: KV tiles per slice; 0 = each query tile cuts its own
                        * prefix into n_splits equal runs */
  int n_q, n_kv, gqa;
  int pos0, n, max_seq;
  int tpt;      /* tokens per 128-row tile = 128 / gqa */
  int n_qtiles;
  float qscale; /* scale * log2(e) */
  unsigned int *err_word;
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}



template <int HD, bool PAGED>
__global__ void __launch_bounds__(PCfg<HD>::THREADS, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap, const PrefillArgs a) {
  using C = PCfg<HD>;
  constexpr int BN = C::BN, NH = C::NH, NSTAGE = C::NSTAGE;
  constexpr int HALF_BYTES = C::HALF_BYTES, KV_BYTES = C::KV_BYTES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto bar = [bar0](int i) { return bar0 + 8u * i; };
  /* barrier indices */
  constexpr int K_FULL = 0, V_FULL = NSTAGE, K_EMPTY = 2 * NSTAGE, V_EMPTY = 3 * NSTAGE;
  constexpr int S_FULL = 4 * NSTAGE, S_FREE = S_FULL + 2, P_READY = S_FREE + 2;
  constexpr int PV_DONE = P_READY + 1, Q_READY = PV_DONE + 1;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + C::OFF_BAR + C::NBAR * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  /* blockIdx.x is the query tile (longest prefixes first) or, when the KV range
   * is cut into slices (few query rows against a long prefix), the slice */
  const int ns = a.n_splits;
  const int split = ns > 1 ? static_cast<int>(blockIdx.x) % ns : 0;
  const int qtile = a.n_qtiles - 1 - static_cast<int>(blockIdx.x) / (ns > 1 ? ns : 1);
  const int kvh = blockIdx.y;
  const int seq = blockIdx.z;

  if (ns > 1 && split > 0) {
    /* A slice past the end of a short sequence has no tiles: publish the empty
     * partial the merge kernel expects and leave before barriers and tensor memory are
     * set up (about half of the CTAs of a ragged batch are of this kind). */
    grid_dependency_wait();
    const int e_pos0 = a.pos0_dev ? max(a.pos0_dev[seq], 0) : a.pos0;
    int e_ntok = a.n;
    if (a.cu_tokens) e_ntok = a.cu_tokens[seq + 1] - a.cu_tokens[seq];
    const int e_tok0 = qtile * a.tpt;
    e_ntok = max(min(a.tpt, e_ntok - e_tok0), 0);
    const int e_kv_end = e_ntok > 0 ? min(e_pos0 + e_tok0 + e_ntok, a.max_seq) : 0;
    const int e_tiles = (e_kv_end + BN - 1) / BN;
    const int e_tps = a.tiles_per_slice > 0 ? a.tiles_per_slice : (e_tiles + ns - 1) / ns;
    if (e_tiles - split * e_tps <= 0) {
      constexpr int V4 = (HD + 4) / 4; /* float4 per scratch row: acc[HD] | m l pad pad */
      const long long unit = (static_cast<long long>(seq) * a.n_kv + kvh) * a.n_qtiles + qtile;
      float4 *dst = reinterpret_cast<float4 *>(a.scratch + (unit * ns + split) * a.rows_cap * (HD + 4));
      const int n4 = e_ntok * a.gqa * V4;
      for (int idx = threadIdx.x; idx < n4; idx += blockDim.x)
        dst[idx] = idx % V4 == V4 - 1 ? make_float4(-INFINITY, 0.f, 0.f, 0.f)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
      return;
    }
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(bar(K_FULL + i), 1);
      mbar_init(bar(V_FULL + i), 1);
      mbar_init(bar(K_EMPTY + i), 1);
      mbar_init(bar(V_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(S_FREE + i), 256);
    }
    mbar_init(bar(P_READY), 256);
    mbar_init(bar(PV_DONE), 1);
    mbar_init(bar(Q_READY), 256);
    mbar_init_fence();
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  constexpr int MMA_WARP = 8, TMA_WARP = 9;
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  grid_dependency_wait();

  /* rows of this tile: row r = (token tok0 + r / gqa, head kvh*gqa + r % gqa) */
  const int pos0 = a.pos0_dev ? max(a.pos0_dev[seq], 0) : a.pos0;
  const int plane = seq * a.n_kv + kvh; /* which [max_seq][hd] slab of a contiguous cache */
  int tok_begin = seq * a.n, n_tok = a.n; /* this sequence's tokens in qkv / out */
  if (a.cu_tokens) {
    tok_begin = a.cu_tokens[seq];
    n_tok = a.cu_tokens[seq + 1] - tok_begin;
  }
  const int tok0 = qtile * a.tpt;
  const int ntok = max(min(a.tpt, n_tok - tok0), 0);
  const int tok_base = tok_begin + tok0;
  const int rows_valid = ntok * a.gqa;
  const int kv_end = ntok > 0 ? min(pos0 + tok0 + ntok, a.max_seq) : 0; /* live rows seen */
  const int lim_min = min(pos0 + tok0 + 1, a.max_seq);
  const int all_tiles = (kv_end + BN - 1) / BN;
  /* this CTA's tiles: all of them, or (sliced) the slice's contiguous run of
   * a.tiles_per_slice tiles -- slices past the end of a short sequence get none and
   * only publish an empty partial, so that the CTAs that do work are equally long
   * whatever the sequence lengths are */
  const int tps = a.tiles_per_slice > 0 ? a.tiles_per_slice : (all_tiles + ns - 1) / (ns > 1 ? ns : 1);
  const int first_tile = split * tps;
  const int slice_cap = split == ns - 1 ? all_tiles : tps; /* the last takes the rest */
  const int n_tiles = ns > 1 ? max(min(all_tiles - first_tile, slice_cap), 0) : all_tiles;
  auto tile_of = [first_tile](int j) { return first_tile + j; };

  if (warp == TMA_WARP) {
    /* ------------------------------------------------------ TMA producer */
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % NSTAGE, round = j / NSTAGE;
        if (j >= NSTAGE && !mbar_wait(bar(K_EMPTY + st), (round - 1) & 1, a.err_word, 0x201u))
          break;
        const int jt = tile_of(j);
        int pages[BN / 16];
        if constexpr (PAGED) {
#pragma unroll
          for (int pg = 0; pg < BN / 16; ++pg) {
            const int slot = jt * (BN / 16) + pg;
            int page = slot < a.max_pages
                           ? a.page_table[static_cast<long long>(seq) * a.max_pages + slot]
                           : -1;
            /* an unmapped slot reads as zeros: coordinate just past the pool */
            pages[pg] = (page < 0 || page >= a.n_pool_pages) ? a.n_pool_pages : page;
          }
        }
        mbar_arrive_expect_tx(bar(K_FULL + st), KV_BYTES);
        if constexpr (PAGED) {
#pragma unroll
          for (int pg = 0; pg < BN / 16; ++pg)
#pragma unroll
            for (int h = 0; h < NH; ++h)
              tma_load_4d(sbase + C::OFF_K + st * KV_BYTES + h * HALF_BYTES + pg * 16 * 128, &kmap,
                          bar(K_FULL + st), h * 64, 0, kvh, pages[pg]);
        } else {
#pragma unroll
          for (int h = 0; h < NH; ++h)
            tma_load_3d(sbase + C::OFF_K + st * KV_BYTES + h * HALF_BYTES, &kmap,
                        bar(K_FULL + st), h * 64, jt * BN, plane);
        }
        if (j >= NSTAGE && !mbar_wait(bar(V_EMPTY + st), (round - 1) & 1, a.err_word, 0x202u))
          break;
        mbar_arrive_expect_tx(bar(V_FULL + st), KV_BYTES);
        if constexpr (PAGED) {
#pragma unroll
          for (int pg = 0; pg < BN / 16; ++pg)
#pragma unroll
            for (int h = 0; h < NH; ++h)
              tma_load_4d(sbase + C::OFF_V + st * KV_BYTES + h * HALF_BYTES + pg * 16 * 128, &vmap,
                          bar(V_FULL + st), h * 64, 0, kvh, pages[pg]);
        } else {
#pragma unroll
          for (int h = 0; h < NH; ++h)
            tma_load_3d(sbase + C::OFF_V + st * KV_BYTES + h * HALF_BYTES, &vmap,
                        bar(V_FULL + st), h * 64, jt * BN, plane);
        }
      }
    }
  } else if (warp == MMA_WARP) {
    /* -------------------------------------------------------- MMA issuer */
    constexpr uint32_t idesc_qk = umma_idesc(128, BN, 0);
    constexpr uint32_t idesc_pv = umma_idesc(128, HD, 1);
    bool ok = mbar_wait(bar(Q_READY), 0, a.err_word, 0x210u);
    tc_fence_after_sync();

    /* One k-step (16 along the contraction) of S(j) = Q K(j)^T and of
     * O += P V(i); each is a 128 x 128 x 16 MMA, 64 clocks of the tensor pipe. */
    const uint32_t k_lo0 = umma_desc_lo(sbase + C::OFF_K, 16);
    const uint32_t v_lo0 = umma_desc_lo(sbase + C::OFF_V, HALF_BYTES);
    auto s_step = [&](int j, int ks) {
      const uint32_t off = (j % NSTAGE) * KV_BYTES + (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
      umma_ts_f16_lohi(tmem + C::COL_S + (j & 1) * BN, tmem + C::COL_Q + ks * 8, k_lo0 + (off >> 4),
                       kDescHi, idesc_qk, ks > 0);
    };
    auto pv_step = [&](int i, int kk) {
      const uint32_t off = (i % NSTAGE) * KV_BYTES + kk * 2048;
      umma_ts_f16_lohi(tmem + C::COL_O, tmem + C::COL_P + kk * 8, v_lo0 + (off >> 4), kDescHi,
                       idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
    };

    /* the first two score tiles */
    for (int j = 0; ok && j < 2 && j < n_tiles; ++j) {
      if (!mbar_wait(bar(K_FULL + j), 0, a.err_word, 0x214u)) { ok = false; break; }
      tc_fence_after_sync();
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) s_step(j, ks);
        umma_commit(bar(S_FULL + j));
        umma_commit(bar(K_EMPTY + j));
      }
      __syncwarp();
    }

    /* step i: O += P(i) V(i) as soon as P(i) arrives, then S(i+2) = Q K(i+2)^T into
     * the score buffer that the softmax of tile i handed back before it sent P(i).
     * The softmax of tile i+1 runs meanwhile on the other score buffer. */
    for (int i = 0; ok && i < n_tiles; ++i) {
      const int st = i % NSTAGE;
      const int j = i + 2;
      const bool has_s = j < n_tiles;
      /* the operands in shared memory arrive long before P: look at their
       * barriers first, so that only P(i) is waited for on the critical path */
      if (!mbar_wait(bar(V_FULL + st), (i / NSTAGE) & 1, a.err_word, 0x212u)) { ok = false; break; }
      if (has_s &&
          !mbar_wait(bar(K_FULL + j % NSTAGE), (j / NSTAGE) & 1, a.err_word, 0x214u)) { ok = false; break; }
      const uint32_t vb = sbase + C::OFF_V + st * KV_BYTES;
      /* Cache rows past the live data can hold any bit pattern and 0 * NaN is
       * NaN: clear them in the last tile before the tensor core reads V. */
      if (tile_of(i) * BN + BN > kv_end) {
        const int first = kv_end - tile_of(i) * BN;
        for (int idx = first * (NH * 8) + lane; idx < BN * NH * 8; idx += 32) {
          const int row = idx / (NH * 8), rest = idx % (NH * 8);
          asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(
                           vb + (rest >> 3) * HALF_BYTES + row * 128 + (rest & 7) * 16),
                       "r"(0u)
                       : "memory");
        }
        fence_async_smem();
        __syncwarp();
      }
      if (!mbar_wait(bar(P_READY), i & 1, a.err_word, 0x211u)) { ok = false; break; }
      tc_fence_after_sync();
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) pv_step(i, k);
        umma_commit(bar(PV_DONE));
        umma_commit(bar(V_EMPTY + st));
      }
      __syncwarp();
      if (has_s) {
        if (!mbar_wait(bar(S_FREE + (j & 1)), ((j >> 1) - 1) & 1, a.err_word, 0x215u)) { ok = false; break; }
        tc_fence_after_sync();
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) s_step(j, k);
          umma_commit(bar(S_FULL + (j & 1)));
          umma_commit(bar(K_EMPTY + j % NSTAGE));
        }
        __syncwarp();
      }
    }
  } else {
    /* ---- softmax + output: two threads per query row, 64 score columns each.
     * One warp per scheduler cannot keep the special-function unit busy (the
     * exponentials and the fp16 packing share it and need about 1000 clocks per
     * 128 x 128 tile; loads, maxima and waits came on top, one after the other);
     * with two warps per scheduler one warp's exponentials fill the other's gaps. */
    constexpr int HB = BN / 2;  /* score columns per thread */
    constexpr int OC = HD / 2;  /* output columns per thread */
    const int wq = warp & 3, half = warp >> 2;
    const int r = wq * 32 + lane; /* query row == TMEM lane */
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    float *xch = reinterpret_cast<float *>(smem + C::OFF_XCH);
    /* the two warps that share 32 rows meet here; every thread of both executes
     * every pair_sync of the kernel, whatever else went wrong */
    auto pair_sync = [wq]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + wq) : "memory"); };
    /* a barrier wait whose verdict is the same in every lane of the warp */
    auto wait_all = [&](int which, uint32_t parity, unsigned code) {
      return __all_sync(0xffffffffu, mbar_wait(bar(which), parity, a.err_word, code)) != 0;
    };

    /* q half-row -> fp16 * scale * log2(e), two per 32-bit column of this row's TMEM lane */
    {
      const bool valid = r < rows_valid && n_tiles > 0; /* a slice without tiles needs no q */
      const float *src = a.q + static_cast<long long>(tok_base + r / a.gqa) * a.q_tok_stride +
                         static_cast<long long>(kvh * a.gqa + r % a.gqa) * HD + half * OC;
      constexpr int QC = OC / 2; /* 32-bit columns this thread writes */
      uint32_t packed[QC];
      const __half *src16 = reinterpret_cast<const __half *>(a.q) +
                            static_cast<long long>(tok_base + r / a.gqa) * a.q_tok_stride +
                            static_cast<long long>(kvh * a.gqa + r % a.gqa) * HD + half * OC;
      /* one loop per source type, so that the row's loads go out together */
      if (valid && a.q16) {
#pragma unroll
        for (int e = 0; e < QC; e += 2) {
          const uint2 h = __ldg(reinterpret_cast<const uint2 *>(src16 + 2 * e));
          const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
          const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&h.y));
          packed[e] = pack_half2(lo.x * a.qscale, lo.y * a.qscale);
          packed[e + 1] = pack_half2(hi.x * a.qscale, hi.y * a.qscale);
        }
      } else {
#pragma unroll
        for (int e = 0; e < QC; e += 2) {
          float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
          if (valid) f = __ldg(reinterpret_cast<const float4 *>(src + 2 * e));
          packed[e] = pack_half2(f.x * a.qscale, f.y * a.qscale);
          packed[e + 1] = pack_half2(f.z * a.qscale, f.w * a.qscale);
        }
      }
      if constexpr (QC == 32)
        tmem_st_32x32(tmem + lane_base + C::COL_Q + half * QC, packed);
      else
        tmem_st_32x16(tmem + lane_base + C::COL_Q + half * QC, packed);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(Q_READY));
    }

    const int lim = r < rows_valid ? min(pos0 + tok0 + r / a.gqa + 1, a.max_seq) : kv_end;
    /* A warp with no valid query row (a short last tile, or a handful of tokens
     * against a long prefix) only keeps the barrier protocol going: its rows of
     * S, P and O hold garbage that no other row depends on and nobody reads. */
    const bool live = wq * 32 < rows_valid;
    float m_ref = -INFINITY; /* exponent offset in use for this row (log2 units) */
    float l_run = 0.f;       /* this thread's share of the row sum */
    bool ok = true;          /* warp-uniform */

    for (int j = 0; j < n_tiles; ++j) {
      if (ok) ok = wait_all(S_FULL + (j & 1), (j >> 1) & 1, 0x220u);
      if (!live) {
        if (ok) {
          mbar_arrive(bar(S_FREE + (j & 1)));
          /* not before the previous tile's P has been consumed: an early arrival
           * would be counted into the phase the live warps have not finished */
          if (j >= 1) ok = wait_all(PV_DONE, (j - 1) & 1, 0x224u);
          if (ok) mbar_arrive(bar(P_READY));
        }
        continue;
      }

      /* this thread's 64 scores into registers, then hand the buffer back at once */
      uint32_t sv[HB];
      float mxh = -INFINITY;
      if (ok) {
        tc_fence_after_sync();
        const uint32_t s_addr = tmem + lane_base + C::COL_S + (j & 1) * BN + half * HB;
#pragma unroll
        for (int c0 = 0; c0 < HB; c0 += 32)
          tmem_ld_32x32(s_addr + c0, *reinterpret_cast<uint32_t(*)[32]>(&sv[c0]));
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(bar(S_FREE + (j & 1)));

        if (tile_of(j) * BN + BN > lim_min) { /* causal edge / end of sequence */
          const int lim_local = lim - tile_of(j) * BN - half * HB;
#pragma unroll
          for (int c = 0; c < HB; ++c)
            if (c >= lim_local) sv[c] = 0xff800000u; /* -inf */
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < HB; c += 8)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mx4[k] = max3(mx4[k], __uint_as_float(sv[c + 2 * k]), __uint_as_float(sv[c + 2 * k + 1]));
        mxh = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      /* the row maximum needs the other half's */
      float *slot = xch + (j & 1) * 256;
      slot[half * 128 + r] = mxh;
      pair_sync();
      const float mx = fmaxf(mxh, slot[(half ^ 1) * 128 + r]);
      if (!ok) continue;

      /* Lazy rescale: keep the old offset unless some row of this warp outgrew
       * it by more than 2^8 (p then stays <= 256, exact enough in fp16 and far
       * from its range); the vote keeps the protocol warp-uniform, and both warps
       * of a pair see the same rows and the same maxima. */
      const bool grow = j == 0 || mx > m_ref + 8.f;
      const bool warp_grow = __any_sync(0xffffffffu, grow);
      const float m_new = warp_grow ? fmaxf(m_ref, mx) : m_ref;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;

      float ps8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < HB; c += 8)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float p = ex2(__uint_as_float(sv[c + k]) - m_use);
          ps8[k] += p;
          sv[c + k] = __float_as_uint(p);
        }
      const float psum = ((ps8[0] + ps8[1]) + (ps8[2] + ps8[3])) + ((ps8[4] + ps8[5]) + (ps8[6] + ps8[7]));
#pragma unroll
      for (int c = 0; c < HB / 2; ++c)
        sv[c] = pack_half2(__uint_as_float(sv[2 * c]), __uint_as_float(sv[2 * c + 1]));

      /* PV of the previous tile must be finished: it reads P and writes O */
      if (j >= 1) ok = wait_all(PV_DONE, (j - 1) & 1, 0x222u);
      if (!ok) continue;
      tmem_st_32x32(tmem + lane_base + C::COL_P + half * (HB / 2),
                    *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));

      if (warp_grow && j > 0) { /* move this thread's half of the O rows to the new offsets */
        tc_fence_after_sync();
        const float factor = ex2(m_ref - m_use); /* 1 for rows that did not move */
#pragma unroll
        for (int c0 = 0; c0 < OC; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + lane_base + C::COL_O + half * OC + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
          tmem_st_32x32(tmem + lane_base + C::COL_O + half * OC + c0, v);
        }
        l_run *= factor;
      }
      m_ref = m_new;
      l_run += psum;

      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(P_READY));
    }
    grid_launch_dependents();

    if (ok && n_tiles > 0) ok = wait_all(PV_DONE, (n_tiles - 1) & 1, 0x223u);
    if (live) {
      /* the row sum is the two threads' shares together */
      float *slot = xch + 512;
      slot[half * 128 + r] = l_run;
      pair_sync();
      l_run += slot[(half ^ 1) * 128 + r];
    }
    if (ok && live && ns > 1) {
      /* one slice of a split KV range: this row's (acc, m, l) for the merge kernel,
       * acc[HD] | m | l | pad pad, log2 units (attn_rows.cu reads the same rows) */
      tc_fence_after_sync();
      const long long unit = (static_cast<long long>(seq) * a.n_kv + kvh) * a.n_qtiles + qtile;
      float *dst = a.scratch + ((unit * ns + split) * a.rows_cap + r) * (HD + 4) + half * OC;
#pragma unroll
      for (int c0 = 0; c0 < OC; c0 += 32) {
        uint32_t v[32];
        if (n_tiles > 0) { /* warp-uniform: the load is a warp-wide instruction */
          tmem_ld_32x32(tmem + lane_base + C::COL_O + half * OC + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (r < rows_valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            *reinterpret_cast<uint4 *>(dst + c0 + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
        }
      }
      if (half == 0 && r < rows_valid)
        *reinterpret_cast<float2 *>(dst + HD) = make_float2(n_tiles > 0 ? m_ref : -INFINITY, l_run);
    } else if (ok && live) {
      tc_fence_after_sync();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __half *dst = a.out + (static_cast<long long>(tok_base + r / a.gqa) * a.n_q +
                             (kvh * a.gqa + r % a.gqa)) * HD + half * OC;
#pragma unroll
      for (int c0 = 0; c0 < OC; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + C::COL_O + half * OC + c0, v);
        tmem_ld_wait();
        if (r < rows_valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 packed;
            packed.x = pack_half2(__uint_as_float(v[8 * g + 0]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
            packed.y = pack_half2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
            packed.z = pack_half2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
            packed.w = pack_half2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
            *reinterpret_cast<uint4 *>(dst + c0 + 8 * g) = packed;
          }
        }
      }
    }
  }

  /* common exit: every role gets here, then the allocating warp frees TMEM */
  tc_fence_before_sync();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}


/* ------------------------------------------------------------------------
 * Two query tiles per CTA: attn_prefill_pair_kernel.
 *
 * A CTA owns TWO 128-row tiles of the same KV head, so every K/V tile fetched from
 * L2 serves 256 query rows.  Each tile has its own softmax warpgroup AND its own
 * MMA-issuing warp; the two tiles share only the K/V ring and the tensor pipe.
 *
 * Tensor memory is exactly full -- S0 S1 O0 O1 at 128 fp32 columns each -- and P_t
 * (fp16) goes over columns 0..63 of S_t, so the scores of tile j+1 cannot be written
 * where P(j) still waits for its MMA.  Were S(j+1) issued whole, after PV(j), every
 * tile would run the chain  softmax -> PV -> S -> softmax  end to end (measured: 4100
 * clocks per KV tile for 2048 clocks of tensor work).  The score MMA is therefore cut
 * in two along the keys:
 *
 *   S_hi(j+1) = Q K(j+1)[64..127]^T -> columns 64..127, issued as soon as the softmax
 *               of tile j has read those columns into registers (HI_FREE);
 *   S_lo(j+1) = Q K(j+1)[0..63]^T   -> columns 0..63, issued behind PV(j), which the
 *               tensor pipe finishes first since it executes in order.
 *
 * The softmax of tile j+1 starts on the upper keys the moment it is done with tile j,
 * and the lower keys arrive while it works; each half is one step of the online
 * softmax (its own maximum, offset kept unless a row grows by more than 2^8).
 * An N = 64 MMA with both operands in shared memory costs 48 clocks, not 32 (the
 * 4 KB Q operand alone takes 32 at 128 bytes per clock), so the scores cost 768
 * clocks per tile where one N = 128 instruction stream costs 512: the tensor pipe
 * has 2560 clocks of work per KV tile and CTA, and that is the new bound.
 *
 * The issuing warps matter as much as the pipe: every wait, election, fence and
 * commit costs the issuing warp 50 to 100 clocks with nothing to overlap it, and one
 * warp driving both tiles spent more time on those than the pipe spent on the MMAs.
 * ---------------------------------------------------------------------- */
template <int HD>
struct P2Cfg {
  static constexpr int BN = 128;
  static constexpr int NH = HD / 64;
  static constexpr int HALF_BYTES = BN * 128;
  static constexpr int Q_BYTES = NH * HALF_BYTES;   /* one query tile */
  static constexpr int KV_BYTES = NH * HALF_BYTES;
  /* K and V tiles go through ONE ring in the order they are fetched, K(0) V(0)
   * K(1) V(1) ...: next to the two query tiles shared memory has room for five
   * 32 KB slots (head_dim 128).  K(j+1) and V(j) are in use during step j, the
   * other three slots are in flight; a tile takes some 2500 clocks to arrive from L2. */
  static constexpr int NSLOT = HD == 128 ? 5 : 8;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_RING = OFF_Q + 2 * Q_BYTES;
  static constexpr int OFF_BAR = OFF_RING + NSLOT * KV_BYTES;
  static constexpr int NBAR = 2 * NSLOT + 2 * 6;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 16 + 1024;
  static constexpr int THREADS = 352; /* 2 x 4 softmax warps, 2 MMA warps, TMA warp */
  static constexpr int COL_S = 0;     /* S_t at COL_S + t*128, P_t over its first 64 columns */
  static constexpr int COL_O = 256;   /* O_t at COL_O + t*128 */
  static constexpr int TMEM_COLS = 512;
};

/* One half (64 keys) of a score row as a step of the online softmax: the offset
 * m_cur moves only if some row of the warp grows by more than 2^8 (or `force`);
 * p = 2^(s - offset) packed to fp16 pairs, returns their fp32 sum.  Subtraction and
 * summation run two lanes wide (f32x2); the 64 exponentials are what bounds it. */
__device__ __forceinline__ float softmax_half(uint32_t (&sv)[64], uint32_t (&pk)[32], float &m_cur,
                                              bool force) {
  float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 64; c += 8)
#pragma unroll
    for (int k = 0; k < 4; ++k)
      mx4[k] = max3(mx4[k], __uint_as_float(sv[c + 2 * k]), __uint_as_float(sv[c + 2 * k + 1]));
  const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
  const bool grow = force || mx > m_cur + 8.f;
  if (__any_sync(0xffffffffu, grow)) m_cur = fmaxf(m_cur, mx);
  const float m_use = m_cur == -INFINITY ? 0.f : m_cur;
  const uint64_t mm = pack_f32x2(m_use, m_use);
  uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float x0, x1;
    unpack_f32x2(sub_f32x2(pack_f32x2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), mm),
                 x0, x1);
    const float p0 = ex2(x0), p1 = ex2(x1);
    acc[i & 3] = add_f32x2(acc[i & 3], pack_f32x2(p0, p1));
    pk[i] = pack_half2(p0, p1);
  }
  float s0, s1;
  unpack_f32x2(add_f32x2(add_f32x2(acc[0], acc[1]), add_f32x2(acc[2], acc[3])), s0, s1);
  return s0 + s1;
}

template <int HD>
__global__ void __launch_bounds__(P2Cfg<HD>::THREADS, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap kmap,
                         const __grid_constant__ CUtensorMap vmap, const PrefillArgs a) {
  using C = P2Cfg<HD>;
  constexpr int BN = C::BN, NH = C::NH, NSLOT = C::NSLOT;
  constexpr int HALF_BYTES = C::HALF_BYTES, KV_BYTES = C::KV_BYTES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto bar = [bar0](int i) { return bar0 + 8u * i; };
  /* ring item 2j is K(j), item 2j+1 is V(j); item i lives in slot i % NSLOT */
  constexpr int FULL = 0, EMPTY = NSLOT;
  constexpr int SHI_FULL = 2 * NSLOT, SLO_FULL = SHI_FULL + 2, HI_FREE = SLO_FULL + 2;
  constexpr int P_READY = HI_FREE + 2, O_DONE = P_READY + 2, Q_READY = O_DONE + 2;
  constexpr int MMA_WARP0 = 8, TMA_WARP = 10;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + C::OFF_BAR + C::NBAR * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_pairs = (a.n_qtiles + 1) >> 1;
  const int pair = n_pairs - 1 - blockIdx.x; /* longest prefixes first */
  const int kvh = blockIdx.y;
  const int seq = blockIdx.z;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSLOT; ++i) {
      mbar_init(bar(FULL + i), 1);
      mbar_init(bar(EMPTY + i), 2); /* one arrival per MMA warp */
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(SHI_FULL + i), 1);
      mbar_init(bar(SLO_FULL + i), 1);
      mbar_init(bar(HI_FREE + i), 128);
      mbar_init(bar(P_READY + i), 128);
      mbar_init(bar(O_DONE + i), 1);
      mbar_init(bar(Q_READY + i), 128);
    }
    mbar_init_fence();
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  if (warp == MMA_WARP0) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  grid_dependency_wait();

  const int pos0 = a.pos0_dev ? max(a.pos0_dev[seq], 0) : a.pos0;
  const int plane = seq * a.n_kv + kvh;
  /* tile t of the pair: tokens tok0_[t] .. tok0_[t] + ntok_[t] - 1; a missing second tile
   * (odd tile count) runs with zero rows over the first tile's range */
  int tok0_[2], ntok_[2], kv_end_[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt = 2 * pair + t;
    tok0_[t] = qt * a.tpt;
    ntok_[t] = qt < a.n_qtiles ? min(a.tpt, a.n - tok0_[t]) : 0;
    kv_end_[t] = ntok_[t] > 0 ? min(pos0 + tok0_[t] + ntok_[t], a.max_seq) : 0;
  }
  if (ntok_[1] == 0) kv_end_[1] = kv_end_[0];
  const int kv_end_all = kv_end_[1];
  /* this warp's tile (warps 0-3 and 8: tile 0; warps 4-7 and 9: tile 1) */
  const int my_t = warp < 8 ? warp >> 2 : (warp - 8) & 1;
  const int my_tok0 = my_t ? tok0_[1] : tok0_[0], my_ntok = my_t ? ntok_[1] : ntok_[0];
  const int my_kv_end = my_t ? kv_end_[1] : kv_end_[0];
  const int my_tiles = (my_kv_end + BN - 1) / BN;
  const int T = (kv_end_all + BN - 1) / BN; /* tile 1 sees at least as far as tile 0 */

  if (warp == TMA_WARP) {
    /* ------------------------------------------------------ TMA producer */
    if (lane == 0) {
      for (int i = 0; i < 2 * T; ++i) {
        const int slot = i % NSLOT, round = i / NSLOT, j = i >> 1;
        if (i >= NSLOT && !mbar_wait(bar(EMPTY + slot), (round - 1) & 1, a.err_word, 0x301u))
          break;
        mbar_arrive_expect_tx(bar(FULL + slot), KV_BYTES);
#pragma unroll
        for (int h = 0; h < NH; ++h)
          tma_load_3d(sbase + C::OFF_RING + slot * KV_BYTES + h * HALF_BYTES, (i & 1) ? &vmap : &kmap,
                      bar(FULL + slot), h * 64, j * BN, plane);
      }
    }
  } else if (warp >= MMA_WARP0) {
    /* ------------------------------------- MMA issuer of tile t = warp - 8 */
    const int t = my_t;
    const int nt = my_tiles;
    constexpr uint32_t idesc_qk = umma_idesc(128, BN / 2, 0);
    constexpr uint32_t idesc_pv = umma_idesc(128, HD, 1);
    bool ok = mbar_wait(bar(Q_READY + t), 0, a.err_word, 0x310u);
    tc_fence_after_sync();
    const uint32_t q_lo = umma_desc_lo(sbase + C::OFF_Q + t * C::Q_BYTES, 16);
    const uint32_t s_col = tmem + C::COL_S + t * 128;

    auto full_wait = [&](int item, unsigned code) {
      return mbar_wait(bar(FULL + item % NSLOT), (item / NSLOT) & 1, a.err_word, code);
    };
    /* S_t(j), keys 64*part .. 64*part+63, into columns 64*part .. of the score buffer */
    auto issue_s = [&](int j, int part) {
      const uint32_t k_lo =
          umma_desc_lo(sbase + C::OFF_RING + ((2 * j) % NSLOT) * KV_BYTES + part * (64 * 128), 16);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          umma_ss_f16_lohi(s_col + part * 64, q_lo + off, k_lo + off, kDescHi, idesc_qk, ks > 0);
        }
        umma_commit(bar((part ? SHI_FULL : SLO_FULL) + t));
        if (part == 0) umma_commit(bar(EMPTY + (2 * j) % NSLOT)); /* this warp is done with K(j) */
      }
      __syncwarp();
    };

    if (ok && nt > 0) {
      ok = full_wait(0, 0x314u);
      tc_fence_after_sync();
      if (ok) {
        issue_s(0, 1);
        issue_s(0, 0);
      }
    }
    for (int j = 0; ok && j < nt; ++j) {
      const bool more = j + 1 < nt;
      if (more) {
        if (!full_wait(2 * j + 2, 0x314u) ||
            !mbar_wait(bar(HI_FREE + t), j & 1, a.err_word, 0x313u)) { ok = false; break; }
        tc_fence_after_sync();
        issue_s(j + 1, 1);
      }
      const int item = 2 * j + 1;
      if (!full_wait(item, 0x312u)) { ok = false; break; }
      const uint32_t vb = sbase + C::OFF_RING + (item % NSLOT) * KV_BYTES;
      /* rows past the live data may hold anything, and 0 * NaN is NaN: clear them
       * (both MMA warps do, whichever comes first; the second writes zeros over zeros) */
      if (j * BN + BN > kv_end_all) {
        const int first = kv_end_all - j * BN;
        for (int idx = first * (NH * 8) + lane; idx < BN * NH * 8; idx += 32) {
          const int row = idx / (NH * 8), rest = idx % (NH * 8);
          asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(
                           vb + (rest >> 3) * HALF_BYTES + row * 128 + (rest & 7) * 16),
                       "r"(0u)
                       : "memory");
        }
        fence_async_smem();
        __syncwarp();
      }
      if (!mbar_wait(bar(P_READY + t), j & 1, a.err_word, 0x311u)) { ok = false; break; }
      tc_fence_after_sync();
      if (elect_one()) { /* O_t += P_t V(j) */
        const uint32_t v_lo = umma_desc_lo(vb, HALF_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          umma_ts_f16_lohi(tmem + C::COL_O + t * 128, s_col + kk * 8, v_lo + ((kk * 2048) >> 4),
                           kDescHi, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        if (!more) umma_commit(bar(O_DONE + t));
        umma_commit(bar(EMPTY + item % NSLOT)); /* this warp is done with V(j) */
      }
      __syncwarp();
      if (more) issue_s(j + 1, 0); /* behind PV(j) in the pipe: P(j) has been read */
    }
    /* tiles that only the other query tile reads: pass their slots on */
    for (int i = 2 * nt; ok && i < 2 * T; ++i) {
      if (!full_wait(i, 0x315u)) break;
      if (elect_one()) mbar_arrive(bar(EMPTY + i % NSLOT));
      __syncwarp();
    }
  } else {
    /* --------------------------- softmax + output: warpgroup t owns tile t */
    const int t = my_t;
    const int r = (warp & 3) * 32 + lane; /* query row == TMEM lane */
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int rows_valid = my_ntok * a.gqa;
    const uint32_t s_col = tmem + lane_base + C::COL_S + t * 128;
    const uint32_t o_col = tmem + lane_base + C::COL_O + t * 128;

    /* q rows -> fp16 * scale * log2(e), in the K-major swizzled operand layout.  A warp
     * stages its 32 rows with whole-row loads (one row of 128 fp32 = one float4 per
     * lane), eight rows in flight; a thread walking its own row alone took several
     * microseconds per CTA before the first MMA could be issued. */
    {
      constexpr int LPR = HD / 4;   /* lanes per row */
      constexpr int RPI = 32 / LPR; /* rows per load instruction */
      const int l = lane % LPR;
      int row = (warp & 3) * 32 + lane / LPR;
      int tok = row / a.gqa, head = row % a.gqa;
      const float *q_tile = a.q + static_cast<long long>(seq * a.n + my_tok0) * a.q_tok_stride +
                            static_cast<long long>(kvh * a.gqa) * HD + 4 * l;
      const __half *q16_tile = reinterpret_cast<const __half *>(a.q) +
                               static_cast<long long>(seq * a.n + my_tok0) * a.q_tok_stride +
                               static_cast<long long>(kvh * a.gqa) * HD + 4 * l;
      uint8_t *q_smem = smem + C::OFF_Q + t * C::Q_BYTES + ((l >> 1) >> 3) * HALF_BYTES + (l & 1) * 8;
      /* one loop per source type: with the choice inside the loop the loads of the eight
       * rows no longer went out together and a launch took 13 us longer */
      auto stage_rows = [&](auto load_row) {
#pragma unroll 8
        for (int i = 0; i < 32 / RPI; ++i) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (row < rows_valid) v = load_row(tok * a.q_tok_stride + head * HD);
          uint2 h;
          h.x = pack_half2(v.x * a.qscale, v.y * a.qscale);
          h.y = pack_half2(v.z * a.qscale, v.w * a.qscale);
          *reinterpret_cast<uint2 *>(q_smem + swz128(row, (l >> 1) & 7)) = h;
          row += RPI;
          head += RPI;
          if (head >= a.gqa) { /* RPI <= 2: one step at most when gqa >= RPI */
            head -= a.gqa;
            ++tok;
            if (head >= a.gqa) { head -= a.gqa; ++tok; }
          }
        }
      };
      if (a.q16) {
        stage_rows([&](long long off) {
          const uint2 h = __ldg(reinterpret_cast<const uint2 *>(q16_tile + off));
          const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
          const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&h.y));
          return make_float4(lo.x, lo.y, hi.x, hi.y);
        });
      } else {
        stage_rows([&](long long off) {
          return __ldg(reinterpret_cast<const float4 *>(q_tile + off));
        });
      }
      fence_async_smem();
      mbar_arrive(bar(Q_READY + t));
    }

    const int lim = r < rows_valid ? min(pos0 + my_tok0 + r / a.gqa + 1, a.max_seq) : my_kv_end;
    const int lim_min = min(pos0 + my_tok0 + 1, a.max_seq);
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < my_tiles; ++j) {
      const bool masked = j * BN + BN > lim_min;
      const int lim_local = lim - j * BN;
      uint32_t sv[64], p_hi[32], p_lo[32];
      float m_cur = m_ref;

      /* keys 64..127: computed while this warpgroup was busy with tile j-1 */
      if (!mbar_wait(bar(SHI_FULL + t), j & 1, a.err_word, 0x320u)) { ok = false; break; }
      tc_fence_after_sync();
      tmem_ld_32x32(s_col + 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld_32x32(s_col + 96, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(HI_FREE + t)); /* S_hi(j+1) may overwrite them now */
      if (masked) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (64 + c >= lim_local) sv[c] = 0xff800000u; /* -inf */
      }
      float sum_hi = softmax_half(sv, p_hi, m_cur, j == 0);
      const float m_mid = m_cur;

      /* keys 0..63: issued behind PV(j-1), so O_t is quiescent once they are here */
      if (!mbar_wait(bar(SLO_FULL + t), j & 1, a.err_word, 0x321u)) { ok = false; break; }
      tc_fence_after_sync();
      tmem_ld_32x32(s_col, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld_32x32(s_col + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_wait();
      if (masked) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (c >= lim_local) sv[c] = 0xff800000u;
      }
      const float sum_lo = softmax_half(sv, p_lo, m_cur, false);
      const float m_use = m_cur == -INFINITY ? 0.f : m_cur;
      if (m_cur != m_mid) {
        /* the offset moved between the halves: bring the upper keys' probabilities
         * to the new one (they are all zero if the upper half was masked out) */
        const float f = m_mid == -INFINITY ? 0.f : ex2(m_mid - m_use);
        const __half2 f2 = __float2half2_rn(f);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const __half2 v = __hmul2(*reinterpret_cast<const __half2 *>(&p_hi[i]), f2);
          p_hi[i] = *reinterpret_cast<const uint32_t *>(&v);
        }
        sum_hi *= f;
      }
      tmem_st_32x32(s_col, p_lo);
      tmem_st_32x32(s_col + 32, p_hi);

      if (__any_sync(0xffffffffu, m_cur != m_ref) && j > 0) {
        const float factor = ex2(m_ref - m_use); /* 1 for rows that did not move */
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(o_col + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
          tmem_st_32x32(o_col + c0, v);
        }
        l_run *= factor;
      }
      m_ref = m_cur;
      l_run += sum_hi + sum_lo;
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(P_READY + t));
    }
    grid_launch_dependents();

    if (ok && my_tiles > 0) ok = mbar_wait(bar(O_DONE + t), 0, a.err_word, 0x323u);
    if (ok && rows_valid > 0) {
      tc_fence_after_sync();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __half *dst = a.out +
                    (static_cast<long long>(seq * a.n + my_tok0 + r / a.gqa) * a.n_q +
                     (kvh * a.gqa + r % a.gqa)) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(o_col + c0, v);
        tmem_ld_wait();
        if (r < rows_valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 packed;
            packed.x = pack_half2(__uint_as_float(v[8 * g + 0]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
            packed.y = pack_half2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
            packed.z = pack_half2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
            packed.w = pack_half2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
            *reinterpret_cast<uint4 *>(dst + c0 + 8 * g) = packed;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == MMA_WARP0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

/* ------------------------------------------------------------------------
 * Ragged paged verify as ONE persistent wave: attn_verify_span_kernel.
 *
 * The (sequence, KV head) units of a ragged batch differ in length by an order of
 * magnitude, and every unit has a single 128-row query tile (a few draft tokens x the
 * heads of the GQA group).  With one CTA per (unit, slice) each CTA pays a prologue
 * (length, page table, first K tile from DRAM, first two score tiles) and an epilogue
 * that nothing else on its SM overlaps, and the last wave is ragged.  Here the KV
 * tiles of ALL units are laid end to end (unit-major) and cut into gridDim.x equal
 * spans; a CTA walks its span, which may cross unit boundaries -- each stretch inside
 * one unit is a "piece" and produces one partial row set (a slice of that unit).  The
 * TMA producer runs ahead across pieces, so the next piece's page ids and first tiles
 * arrive while the current piece is still in its softmax and epilogue; the MMA and
 * softmax warps carry their barrier phases on a tile counter that never restarts.
 * Every CTA streams the same number of tiles (+-1), whatever the lengths are.
 *
 * Same tile pipeline as attn_prefill_kernel (Q and P in tensor memory, two score
 * buffers, two softmax threads per row, lazy rescale); the slices of a unit are
 * merged by attn_merge_kernel, which reads each unit's slice count from the tail of
 * the scratch buffer.
 * ---------------------------------------------------------------------- */
struct SpanArgs {
  const float *q;
  long long q_tok_stride;
  float *scratch;            /* [unit][max_slices][rows_cap][hd+4], then int32 counts[n_units] */
  int *slice_counts;
  const int32_t *pos0_dev;   /* [n_seq] */
  const int32_t *cu_tokens;  /* [n_seq + 1] */
  const int32_t *page_table; /* [n_seq][max_pages] */
  int max_pages, n_pool_pages;
  int n_seq, n_q, n_kv, gqa, max_seq;
  int max_slices, rows_cap;
  int min_span; /* tiles: no unit may be cut into more than max_slices pieces */
  int early;    /* the batch description and the cache rows below every sequence's new
                 * tokens are not written by the launch ahead: read them before the grid
                 * dependency resolves */
  float qscale;
  unsigned int *err_word;
};

/* One stretch of a CTA's span inside one unit. */
struct SpanPiece {
  int seq, kvh, first, n, slice, count; /* count > 0 only on the unit's first piece */
  int pos0, tok_begin, ntok, kv_end;
};

/* What starting a piece costs a CTA, in tiles: the next unit's q has to be fetched and
 * staged and the pipeline refilled while the finished piece's rows are stored (measured:
 * 4 to 5 us per unit boundary against 1.8 us per tile).  The span arithmetic counts every
 * unit as kUnitPad + tiles "slots", so a span with many short units gets fewer real
 * tiles than one inside a long unit, and all CTAs finish together. */
constexpr int kUnitPad = 3;

/* Walks the pieces of a span; every role of the CTA runs its own copy.  Positions are
 * slots: unit u owns slots [start_u, start_u + kUnitPad + tiles_u); the first kUnitPad
 * of them are padding, slot kUnitPad + i is KV tile i. */
struct SpanWalk {
  int seq, kvh, slot; /* where the next piece starts: slot index inside the unit */
  long long g, hi;    /* global slot index of that point, end of the span */
  long long before;   /* slots of all units of earlier sequences */
  int span, cta;
  const SpanArgs *a;

  __device__ __forceinline__ static int seq_tiles(const SpanArgs &a, int s, int *pos0, int *tok_begin,
                                                  int *ntok, int *kv_end) {
    const int b = a.cu_tokens[s];
    const int n = a.cu_tokens[s + 1] - b;
    const int p0 = max(a.pos0_dev[s], 0);
    const int end = n > 0 ? min(p0 + n, a.max_seq) : 0;
    *pos0 = p0;
    *tok_begin = b;
    *ntok = n;
    *kv_end = end;
    return (end + 127) / 128;
  }
  /* slots of one unit of a sequence with t tiles (0 for a sequence without tokens) */
  __device__ __forceinline__ static int unit_slots(int t) { return t > 0 ? t + kUnitPad : 0; }

  __device__ __forceinline__ bool next(SpanPiece *p) {
    while (g < hi && seq < a->n_seq) {
      const int t = seq_tiles(*a, seq, &p->pos0, &p->tok_begin, &p->ntok, &p->kv_end);
      if (t == 0) { /* a sequence without tokens in this step */
        ++seq;
        continue;
      }
      const int us = unit_slots(t);
      const long long left = hi - g;
      const int n_slots = static_cast<int>(min(static_cast<long long>(us - slot), left));
      const long long unit_start = before + static_cast<long long>(kvh) * us;
      /* the real tiles among slots [slot, slot + n_slots) */
      const int first = max(slot - kUnitPad, 0);
      const int last = slot + n_slots - kUnitPad; /* one past */
      const int n = max(last - first, 0);
      /* slices are numbered by the CTAs that hold real tiles of the unit: the first real
       * tile sits at unit_start + kUnitPad */
      const long long first_real = unit_start + kUnitPad;
      p->seq = seq;
      p->kvh = kvh;
      p->first = first;
      p->n = n;
      p->slice = cta - static_cast<int>(first_real / span);
      p->count = (n > 0 && first == 0)
                     ? static_cast<int>((first_real + t - 1) / span - first_real / span) + 1
                     : 0;
      g += n_slots;
      slot += n_slots;
      if (slot == us) {
        slot = 0;
        if (++kvh == a->n_kv) {
          kvh = 0;
          before += static_cast<long long>(a->n_kv) * us;
          ++seq;
        }
      }
      if (n > 0) return true; /* a stretch of padding only is no piece */
    }
    return false;
  }
};

template <int HD>
__global__ void __launch_bounds__(PCfg<HD>::THREADS, 1)
attn_verify_span_kernel(const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap vmap,
                        const __grid_constant__ SpanArgs a) {
  using C = PCfg<HD>;
  constexpr int BN = C::BN, NH = C::NH, NSTAGE = C::NSTAGE;
  constexpr int HALF_BYTES = C::HALF_BYTES, KV_BYTES = C::KV_BYTES;
  /* head_dim 128: a page's two 128-byte halves come in ONE 4 KB box (5-D tensor map;
   * half as many requests per tile, and the TMA unit's rate is per request), which lays
   * a tile down as [page][half][16 rows][128 B] instead of [half][128 rows][128 B].  An
   * 8-row group of one half is then 4096 bytes from the same rows of the next page and
   * 1024 from the other eight rows of its own page, so the score MMA runs as two N = 64
   * halves -- columns 0-63 are rows 0-7 of the eight pages, columns 64-127 rows 8-15 --
   * and P, the mask and the PV k-steps follow that column order. */
  constexpr bool WIDE = HD == 128;
  constexpr uint32_t kDescHiWide = (4096u >> 4) | (1u << 14) | (2u << 29);

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto bar = [bar0](int i) { return bar0 + 8u * i; };
  constexpr int K_FULL = 0, V_FULL = NSTAGE, K_EMPTY = 2 * NSTAGE, V_EMPTY = 3 * NSTAGE;
  constexpr int S_FULL = 4 * NSTAGE, S_FREE = S_FULL + 2, P_READY = S_FREE + 2;
  constexpr int PV_DONE = P_READY + 1, Q_READY = PV_DONE + 1, EPI_DONE = Q_READY + 1;
  static_assert(EPI_DONE < C::NBAR, "barrier area");
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + C::OFF_BAR + C::NBAR * 8);
  /* where this CTA's span starts, written by warp 0: seq, kvh, tile, span, g(lo,hi) lo hi, before */
  long long *walk0 = reinterpret_cast<long long *>(smem + C::OFF_XCH + 3 * 2 * 128 * 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(bar(K_FULL + i), 1);
      mbar_init(bar(V_FULL + i), 1);
      mbar_init(bar(K_EMPTY + i), 1);
      mbar_init(bar(V_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(S_FREE + i), 256);
    }
    mbar_init(bar(P_READY), 256);
    mbar_init(bar(PV_DONE), 1);
    mbar_init(bar(Q_READY), 256);
    mbar_init(bar(EPI_DONE), 256);
    mbar_init_fence();
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  constexpr int MMA_WARP = 8, TMA_WARP = 9;
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  grid_launch_dependents();
  if (warp == 0) { /* towards L2 while the dependency is open: no architectural effect */
    for (int i = lane * 32; i <= a.n_seq; i += 32 * 32) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a.cu_tokens + i));
      if (i < a.n_seq) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.pos0_dev + i));
    }
  }
  /* With `early`, the launch ahead of this one in the stream (the append of this step's
   * tokens) writes only q and the cache rows at and above each sequence's seq_pos0, and
   * nothing writes the batch description (seq_pos0, cu_tokens, page table) any more.  So
   * the span arithmetic, the page ids and every K/V tile that lies wholly below seq_pos0
   * are fetched while that launch and the merge before it are still running; each role
   * waits for the dependency right before it first touches what the append writes. */
  if (!a.early) grid_dependency_wait();

  /* ---- where does this CTA's span start?  warp 0: total tiles, span length, and the
   * (sequence, KV head, tile) at global tile index cta * span */
  if (warp == 0) {
    int pos0, tb, nt, ke;
    long long total = 0;
    for (int s0 = 0; s0 < a.n_seq; s0 += 32) {
      const int s = s0 + lane;
      long long t = s < a.n_seq ? SpanWalk::unit_slots(SpanWalk::seq_tiles(a, s, &pos0, &tb, &nt, &ke)) : 0;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
      total += t;
    }
    total *= a.n_kv;
    long long span = (total + gridDim.x - 1) / gridDim.x;
    if (span < a.min_span) span = a.min_span;
    const long long lo = static_cast<long long>(blockIdx.x) * span;
    const long long hi = min(lo + span, total);
    /* the sequence that holds global tile `lo` */
    long long before = 0;
    int seq = a.n_seq, kvh = 0, tile = 0;
    if (lo < total) {
      for (int s0 = 0; s0 < a.n_seq && seq == a.n_seq; s0 += 32) {
        const int s = s0 + lane;
        const long long mine =
            s < a.n_seq ? static_cast<long long>(a.n_kv) *
                              SpanWalk::unit_slots(SpanWalk::seq_tiles(a, s, &pos0, &tb, &nt, &ke))
                        : 0;
        long long incl = mine;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const long long up = __shfl_up_sync(0xffffffffu, incl, off);
          if (lane >= off) incl += up;
        }
        const bool here = mine > 0 && before + incl - mine <= lo && lo < before + incl;
        const unsigned vote = __ballot_sync(0xffffffffu, here);
        if (vote) {
          const int src = __ffs(vote) - 1;
          const long long start = __shfl_sync(0xffffffffu, before + incl - mine, src);
          const long long t = __shfl_sync(0xffffffffu, mine, src) / a.n_kv;
          seq = s0 + src;
          kvh = static_cast<int>((lo - start) / t);
          tile = static_cast<int>((lo - start) % t);
          before = start;
        } else {
          before += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
    }
    if (lane == 0) {
      walk0[0] = seq;
      walk0[1] = kvh;
      walk0[2] = tile;
      walk0[3] = span;
      walk0[4] = lo;
      walk0[5] = hi;
      walk0[6] = before;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  SpanWalk walk;
  walk.seq = static_cast<int>(walk0[0]);
  walk.kvh = static_cast<int>(walk0[1]);
  walk.slot = static_cast<int>(walk0[2]);
  walk.span = static_cast<int>(walk0[3]);
  walk.g = walk0[4];
  walk.hi = walk0[5];
  walk.before = walk0[6];
  walk.cta = static_cast<int>(blockIdx.x);
  walk.a = &a;
  int n_total = 0; /* KV tiles of this CTA (its span minus the padding slots) */
  {
    SpanWalk count = walk;
    SpanPiece pc;
    while (count.next(&pc)) n_total += pc.n;
  }

  if (n_total == 0) {
    /* nothing to do: fall through to the common exit */
  } else if (warp == TMA_WARP) {
    /* ------------------------------------------------------ TMA producer.
     * A 128-position tile of a paged cache is eight pages for K and eight for V, one
     * box per page and operand (4 KB at head_dim 128, 2 KB at 64).  The whole warp
     * issues them: lanes 0-15 own the K boxes, lanes 16-31 the V boxes,
     * one box per lane, and the two half-warps run their rings independently (K is
     * wanted a tile earlier than V).  Each lane fetches its page id one tile ahead, so
     * no tile waits for a page-table load. */
    {
      constexpr int BOXES = WIDE ? BN / 16 : (BN / 16) * NH; /* per operand */
      const int which = lane >> 4, sub = lane & 15;
      const bool active = sub < BOXES;
      const int pg = WIDE ? sub : sub / NH, h = WIDE ? 0 : sub % NH;
      const unsigned halfmask = which ? 0xffff0000u : 0x0000ffffu;
      const int FULL = which ? V_FULL : K_FULL, EMPTY = which ? V_EMPTY : K_EMPTY;
      const CUtensorMap *map = which ? &vmap : &kmap;
      const uint32_t dst0 = sbase + (which ? C::OFF_V : C::OFF_K) +
                            (WIDE ? pg * 4096 : h * HALF_BYTES + pg * 16 * 128);
      auto page_of = [&](int seq, int jt) {
        const int slot = jt * (BN / 16) + pg;
        int page = (active && slot < a.max_pages)
                       ? a.page_table[static_cast<long long>(seq) * a.max_pages + slot]
                       : -1;
        /* an unmapped slot reads as zeros: coordinate just past the pool */
        return (page < 0 || page >= a.n_pool_pages) ? a.n_pool_pages : page;
      };
      SpanPiece pc;
      int G = 0;
      bool ok = true;
      bool waited = !a.early;
      while (ok && walk.next(&pc)) {
        int page_next = page_of(pc.seq, pc.first);
        for (int j = 0; j < pc.n; ++j, ++G) {
          const int st = G % NSTAGE, round = G / NSTAGE;
          if (!waited && (pc.first + j) * BN + BN > pc.pos0) { /* this tile may hold new rows */
            grid_dependency_wait();
            waited = true;
          }
          const int page = page_next;
          if (j + 1 < pc.n) page_next = page_of(pc.seq, pc.first + j + 1);
          if (G >= NSTAGE) {
            const bool got = mbar_wait(bar(EMPTY + st), (round - 1) & 1, a.err_word, 0x501u + which);
            if (!__all_sync(halfmask, got)) {
              ok = false;
              break;
            }
          }
          if (sub == 0) mbar_arrive_expect_tx(bar(FULL + st), KV_BYTES);
          __syncwarp(halfmask);
          if (active) {
            if constexpr (WIDE)
              tma_load_5d(dst0 + st * KV_BYTES, map, bar(FULL + st), 0, 0, 0, pc.kvh, page);
            else
              tma_load_4d(dst0 + st * KV_BYTES, map, bar(FULL + st), h * 64, 0, pc.kvh, page);
          }
        }
      }
    }
  } else if (warp == MMA_WARP) {
    /* -------------------------------------------------------- MMA issuer.
     * Program over the CTA's tiles g = 0 .. n_total-1, whatever piece they belong to:
     *     S(0) S(1)   then for every g:   PV(g)  S(g+2)
     * S of a piece's first tile waits for that piece's Q; PV of a piece's first tile
     * starts a new accumulation and waits until the epilogue of the piece before has
     * read O. */
    constexpr uint32_t idesc_qk = umma_idesc(128, BN, 0);
    constexpr uint32_t idesc_qk_half = umma_idesc(128, BN / 2, 0);
    constexpr uint32_t idesc_pv = umma_idesc(128, HD, 1);
    const uint32_t k_lo0 = umma_desc_lo(sbase + C::OFF_K, 16);
    const uint32_t v_lo0 = umma_desc_lo(sbase + C::OFF_V, WIDE ? 2048 : HALF_BYTES);
    if (a.early) grid_dependency_wait(); /* Q and P come from threads that waited; be ordered too */
    /* two walkers: one for the S stream (two tiles ahead), one for the PV stream */
    SpanWalk ws = walk, wp = walk;
    SpanPiece ps, pp;
    int s_left = 0, s_piece = -1;  /* tiles left in the S stream's current piece */
    int p_left = 0, p_piece = -1, p_pos = 0;
    bool ok = true;

    auto issue_s = [&](int g) -> bool {
      bool first = false;
      if (s_left == 0) {
        if (!ws.next(&ps)) return false;
        s_left = ps.n;
        ++s_piece;
        first = true;
      }
      --s_left;
      if (first && !mbar_wait(bar(Q_READY), s_piece & 1, a.err_word, 0x510u)) return false;
      if (!mbar_wait(bar(K_FULL + g % NSTAGE), (g / NSTAGE) & 1, a.err_word, 0x514u)) return false;
      if (g >= 2 && !mbar_wait(bar(S_FREE + (g & 1)), ((g >> 1) - 1) & 1, a.err_word, 0x515u))
        return false;
      tc_fence_after_sync();
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          if constexpr (WIDE) {
            const uint32_t off = (g % NSTAGE) * KV_BYTES + (ks >> 2) * 2048 + (ks & 3) * 32;
            umma_ts_f16_lohi(tmem + C::COL_S + (g & 1) * BN, tmem + C::COL_Q + ks * 8,
                             k_lo0 + (off >> 4), kDescHiWide, idesc_qk_half, ks > 0);
            umma_ts_f16_lohi(tmem + C::COL_S + (g & 1) * BN + 64, tmem + C::COL_Q + ks * 8,
                             k_lo0 + ((off + 1024) >> 4), kDescHiWide, idesc_qk_half, ks > 0);
          } else {
            const uint32_t off = (g % NSTAGE) * KV_BYTES + (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
            umma_ts_f16_lohi(tmem + C::COL_S + (g & 1) * BN, tmem + C::COL_Q + ks * 8,
                             k_lo0 + (off >> 4), kDescHi, idesc_qk, ks > 0);
          }
        }
        umma_commit(bar(S_FULL + (g & 1)));
        umma_commit(bar(K_EMPTY + g % NSTAGE));
      }
      __syncwarp();
      return true;
    };
    auto issue_pv = [&](int g) -> bool {
      if (p_left == 0) {
        if (!wp.next(&pp)) return false;
        p_left = pp.n;
        p_pos = 0;
        ++p_piece;
        /* the epilogue of the piece before must have read O */
        if (p_piece > 0 && !mbar_wait(bar(EPI_DONE), (p_piece - 1) & 1, a.err_word, 0x516u))
          return false;
      }
      const int st = g % NSTAGE;
      if (!mbar_wait(bar(V_FULL + st), (g / NSTAGE) & 1, a.err_word, 0x512u)) return false;
      const uint32_t vb = sbase + C::OFF_V + st * KV_BYTES;
      const int jt = pp.first + p_pos;
      /* Cache rows past the live data can hold any bit pattern and 0 * NaN is NaN:
       * clear them in the sequence's last tile before the tensor core reads V. */
      if (jt * BN + BN > pp.kv_end) {
        const int first_dead = pp.kv_end - jt * BN;
        for (int idx = first_dead * (NH * 8) + lane; idx < BN * NH * 8; idx += 32) {
          const int row = idx / (NH * 8), rest = idx % (NH * 8);
          const uint32_t where =
              WIDE ? (row >> 4) * 4096 + (rest >> 3) * 2048 + (row & 15) * 128 + (rest & 7) * 16
                   : (rest >> 3) * HALF_BYTES + row * 128 + (rest & 7) * 16;
          asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(vb + where), "r"(0u)
                       : "memory");
        }
        fence_async_smem();
        __syncwarp();
      }
      if (!mbar_wait(bar(P_READY), g & 1, a.err_word, 0x511u)) return false;
      tc_fence_after_sync();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          /* P columns 16kk .. 16kk+15: (WIDE) rows 0-7 or 8-15 of two neighbouring pages */
          const uint32_t off = WIDE ? st * KV_BYTES + (kk & 3) * 8192 + (kk >> 2) * 1024
                                    : st * KV_BYTES + kk * 2048;
          umma_ts_f16_lohi(tmem + C::COL_O, tmem + C::COL_P + kk * 8, v_lo0 + (off >> 4),
                           WIDE ? kDescHiWide : kDescHi, idesc_pv, (p_pos > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bar(PV_DONE));
        umma_commit(bar(V_EMPTY + st));
      }
      __syncwarp();
      ++p_pos;
      --p_left;
      return true;
    };

    /* A score tile that opens a new piece waits for that piece's Q, which the softmax
     * warps stage only after the last tile of the piece before: such an S is held back
     * behind the next PV (the old piece's last), so that PV and the old piece's epilogue
     * run while Q is on its way instead of after it. */
    int s_next = 0; /* next score tile to issue; runs up to two ahead of the PV stream */
    auto s_opens_piece = [&]() { return s_left == 0; };
    for (; ok && s_next < 2 && s_next < n_total; ++s_next) ok = issue_s(s_next);
    for (int g = 0; ok && g < n_total; ++g) {
      ok = issue_pv(g);
      while (ok && s_next < n_total && s_next <= g + 2) {
        /* two ahead normally; a piece-opening S not before the PV of the tile right
         * before it has been issued */
        if (s_opens_piece() && s_next > g + 1) break;
        ok = issue_s(s_next);
        ++s_next;
      }
    }
  } else {
    /* ---- softmax + partial output: two threads per query row, 64 score columns each */
    constexpr int HB = BN / 2;
    constexpr int OC = HD / 2;
    const int wq = warp & 3, half = warp >> 2;
    const int r = wq * 32 + lane; /* query row == TMEM lane */
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    float *xch = reinterpret_cast<float *>(smem + C::OFF_XCH);
    auto pair_sync = [wq]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + wq) : "memory"); };
    auto wait_all = [&](int which, uint32_t parity, unsigned code) {
      return __all_sync(0xffffffffu, mbar_wait(bar(which), parity, a.err_word, code)) != 0;
    };
    /* q half-row of (piece, row r) -> fp16 * scale * log2(e) into this row's TMEM lane */
    auto stage_q = [&](const SpanPiece &pc) {
      const int rows_valid = pc.ntok * a.gqa;
      const bool valid = r < rows_valid;
      const float *src = a.q + static_cast<long long>(pc.tok_begin + r / a.gqa) * a.q_tok_stride +
                         static_cast<long long>(pc.kvh * a.gqa + r % a.gqa) * HD + half * OC;
      constexpr int QC = OC / 2;
      uint32_t packed[QC];
#pragma unroll
      for (int e = 0; e < QC; e += 2) {
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid) f = __ldg(reinterpret_cast<const float4 *>(src + 2 * e));
        packed[e] = pack_half2(f.x * a.qscale, f.y * a.qscale);
        packed[e + 1] = pack_half2(f.z * a.qscale, f.w * a.qscale);
      }
      if constexpr (QC == 32)
        tmem_st_32x32(tmem + lane_base + C::COL_Q + half * QC, packed);
      else
        tmem_st_32x16(tmem + lane_base + C::COL_Q + half * QC, packed);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(Q_READY));
    };

    if (a.early) grid_dependency_wait(); /* q is what the append ahead of this launch wrote */
    SpanWalk wk = walk;
    SpanPiece pc, nxt;
    bool have = wk.next(&pc);
    if (have) stage_q(pc);
    int G = 0, piece = 0;
    bool ok = true; /* warp-uniform */
    while (have) {
      /* the piece after this one: its q rows towards L2 now, staged when this piece's
       * last score tile has been read */
      const bool more = wk.next(&nxt);
      if (more && r < nxt.ntok * a.gqa) {
        const char *qn = reinterpret_cast<const char *>(
            a.q + static_cast<long long>(nxt.tok_begin + r / a.gqa) * a.q_tok_stride +
            static_cast<long long>(nxt.kvh * a.gqa + r % a.gqa) * HD + half * OC);
#pragma unroll
        for (int b = 0; b < OC * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(qn + b));
      }
      const int rows_valid = pc.ntok * a.gqa;
      const int lim = r < rows_valid ? min(pc.pos0 + r / a.gqa + 1, a.max_seq) : pc.kv_end;
      const int lim_min = min(pc.pos0 + 1, a.max_seq);
      const bool live = wq * 32 < rows_valid;
      float m_ref = -INFINITY, l_run = 0.f;

      for (int j = 0; j < pc.n; ++j, ++G) {
        const int jt = pc.first + j;
        if (ok) ok = wait_all(S_FULL + (G & 1), (G >> 1) & 1, 0x520u);
        if (!live) {
          if (ok) {
            mbar_arrive(bar(S_FREE + (G & 1)));
            if (G >= 1) ok = wait_all(PV_DONE, (G - 1) & 1, 0x524u);
            if (ok) mbar_arrive(bar(P_READY));
          }
          continue;
        }
        uint32_t sv[HB];
        float mxh = -INFINITY;
        if (ok) {
          tc_fence_after_sync();
          const uint32_t s_addr = tmem + lane_base + C::COL_S + (G & 1) * BN + half * HB;
#pragma unroll
          for (int c0 = 0; c0 < HB; c0 += 32)
            tmem_ld_32x32(s_addr + c0, *reinterpret_cast<uint32_t(*)[32]>(&sv[c0]));
          tmem_ld_wait();
          tc_fence_before_sync();
          mbar_arrive(bar(S_FREE + (G & 1)));
          if (jt * BN + BN > lim_min) { /* causal edge / end of sequence */
            if constexpr (WIDE) { /* column c of this half is row 8*half + c%8 of page c/8 */
              const int lim_tile = lim - jt * BN - 8 * half;
#pragma unroll
              for (int c = 0; c < HB; ++c)
                if (16 * (c >> 3) + (c & 7) >= lim_tile) sv[c] = 0xff800000u; /* -inf */
            } else {
              const int lim_local = lim - jt * BN - half * HB;
#pragma unroll
              for (int c = 0; c < HB; ++c)
                if (c >= lim_local) sv[c] = 0xff800000u; /* -inf */
            }
          }
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < HB; c += 8)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mx4[k] = max3(mx4[k], __uint_as_float(sv[c + 2 * k]), __uint_as_float(sv[c + 2 * k + 1]));
          mxh = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        }
        float *slot = xch + (G & 1) * 256;
        slot[half * 128 + r] = mxh;
        pair_sync();
        const float mx = fmaxf(mxh, slot[(half ^ 1) * 128 + r]);
        if (!ok) continue;

        const bool grow = j == 0 || mx > m_ref + 8.f; /* lazy rescale, as in attn_prefill_kernel */
        const bool warp_grow = __any_sync(0xffffffffu, grow);
        const float m_new = warp_grow ? fmaxf(m_ref, mx) : m_ref;
        const float m_use = m_new == -INFINITY ? 0.f : m_new;

        float ps8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < HB; c += 8)
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float p = ex2(__uint_as_float(sv[c + k]) - m_use);
            ps8[k] += p;
            sv[c + k] = __float_as_uint(p);
          }
        const float psum = ((ps8[0] + ps8[1]) + (ps8[2] + ps8[3])) + ((ps8[4] + ps8[5]) + (ps8[6] + ps8[7]));
#pragma unroll
        for (int c = 0; c < HB / 2; ++c)
          sv[c] = pack_half2(__uint_as_float(sv[2 * c]), __uint_as_float(sv[2 * c + 1]));

        /* PV of the tile before must be finished: it reads P and writes O */
        if (G >= 1) ok = wait_all(PV_DONE, (G - 1) & 1, 0x522u);
        if (!ok) continue;
        tmem_st_32x32(tmem + lane_base + C::COL_P + half * (HB / 2),
                      *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        if (warp_grow && j > 0) {
          tc_fence_after_sync();
          const float factor = ex2(m_ref - m_use);
#pragma unroll
          for (int c0 = 0; c0 < OC; c0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem + lane_base + C::COL_O + half * OC + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
            tmem_st_32x32(tmem + lane_base + C::COL_O + half * OC + c0, v);
          }
          l_run *= factor;
        }
        m_ref = m_new;
        l_run += psum;
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(bar(P_READY));
      }

      /* The last S of this piece has been read, so Q is free: stage the next piece's q
       * BEFORE this piece's epilogue -- the MMA warp issues the next piece's first score
       * tile ahead of this piece's last PV and would otherwise wait for Q while the
       * epilogue waits for that PV. */
      if (more) stage_q(nxt);

      /* ---- epilogue: this piece's (acc, m, l) rows for the merge kernel */
      if (ok) ok = wait_all(PV_DONE, (G - 1) & 1, 0x523u);
      if (live) {
        float *slot = xch + 512;
        slot[half * 128 + r] = l_run;
        pair_sync();
        l_run += slot[(half ^ 1) * 128 + r];
        pair_sync(); /* both halves have read before the next piece writes the slot */
      }
      const long long unit = static_cast<long long>(pc.seq) * a.n_kv + pc.kvh;
      if (ok && live) {
        tc_fence_after_sync();
        float *dst = a.scratch + ((unit * a.max_slices + pc.slice) * a.rows_cap + r) * (HD + 4) + half * OC;
#pragma unroll
        for (int c0 = 0; c0 < OC; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + lane_base + C::COL_O + half * OC + c0, v);
          tmem_ld_wait();
          if (r < rows_valid) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<uint4 *>(dst + c0 + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
          }
        }
        if (half == 0 && r < rows_valid)
          *reinterpret_cast<float2 *>(dst + HD) = make_float2(m_ref, l_run);
      }
      if (pc.count > 0 && threadIdx.x == 0) a.slice_counts[unit] = pc.count;
      tc_fence_before_sync();
      mbar_arrive(bar(EPI_DONE)); /* O may be overwritten */
      pc = nxt;
      have = more;
      ++piece;
    }
  }

  /* common exit: every role gets here, then the allocating warp frees TMEM */
  tc_fence_before_sync();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <class Cfg, class Kern, class Args>
wst_status_t launch_kernel(const PrefillLaunch &P, Kern kern, const Args &args,
                           const CUtensorMap &kmap, const CUtensorMap &vmap, dim3 grid) {
  /* the opt-in to > 48 KB of dynamic shared memory is per function and device */
  static thread_local const void *configured_fn[8] = {};
  static thread_local int configured_dev[8] = {};
  int dev = 0;
  WST_CUDA(cudaGetDevice(&dev));
  const void *fn = reinterpret_cast<const void *>(kern);
  bool done = false;
  int free_slot = -1;
  for (int i = 0; i < 8; ++i) {
    if (configured_fn[i] == fn && configured_dev[i] == dev) done = true;
    if (!configured_fn[i] && free_slot < 0) free_slot = i;
  }
  if (!done) {
    WST_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  Cfg::SMEM_BYTES));
    if (free_slot >= 0) {
      configured_fn[free_slot] = fn;
      configured_dev[free_slot] = dev;
    }
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(Cfg::THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = current_stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, kmap, vmap, args);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(WST_ERR_CUDA, "%s (launch): %s (%s)", P.name, cudaGetErrorString(e),
                cudaGetErrorName(e));
  return WST_OK;
}

}  // namespace

bool prefill_kernel_supports(int n_q, int n_kv, int hd, int n) {
  if (hd != 64 && hd != 128) return false;
  if (n_kv <= 0 || n_q % n_kv != 0) return false;
  const int gqa = n_q / n_kv;
  if (gqa > 128) return false;
  /* 128-row tiles pay once the chunk fills at least half of one */
  return static_cast<long long>(n) * gqa >= 64;
}


wst_status_t launch_verify_span(const PrefillLaunch &P) {
  DeviceFacts facts;
  if (!device_facts(&facts)) return WST_ERR_CUDA;
  if (facts.cc_major < 10)
    return fail(WST_ERR_UNSUPPORTED_ARCH, "%s: this library is built for sm_100a only", P.name);
  if (!aligned16(P.qkv) || !aligned16(P.k) || !aligned16(P.v) || !aligned16(P.out) ||
      !aligned16(P.scratch))
    return fail(WST_ERR_INVALID_ARG, "%s: buffers must be 16-byte aligned", P.name);
  const int gqa = P.n_q / P.n_kv;
  const int rows_cap = P.n * gqa;
  const long long units = static_cast<long long>(P.n_seq) * P.n_kv;
  const long long row_floats = static_cast<long long>(rows_cap) * (P.hd + 4);
  /* slices a unit may be cut into: what the scratch holds (after it, one count per unit) */
  long long cap = (P.scratch_floats - units) / (units * row_floats);
  if (cap > kRowsMaxSplits) cap = kRowsMaxSplits;
  if (cap < 2) return fail(WST_ERR_INVALID_ARG, "%s: scratch too small", P.name);
  const int max_tiles = (P.max_len > 0 ? P.max_len : P.max_seq) / 128 + 1;

  if (P.q16) return fail(WST_ERR_SHAPE, "%s: fp16 query rows are not taken by the paged verify", P.name);
  SpanArgs a{};
  a.q = P.qkv;
  a.q_tok_stride = P.q_tok_stride;
  a.scratch = P.scratch;
  a.slice_counts = reinterpret_cast<int *>(P.scratch + units * cap * row_floats);
  a.pos0_dev = P.pos0_dev;
  a.cu_tokens = P.cu_tokens;
  a.page_table = P.page_table;
  a.max_pages = P.max_pages;
  a.n_pool_pages = P.n_pool_pages;
  a.n_seq = P.n_seq;
  a.n_q = P.n_q;
  a.n_kv = P.n_kv;
  a.gqa = gqa;
  a.max_seq = P.max_seq;
  a.max_slices = static_cast<int>(cap);
  a.rows_cap = rows_cap;
  a.min_span = (max_tiles + static_cast<int>(cap) - 2) / (static_cast<int>(cap) - 1);
  if (a.min_span < 1) a.min_span = 1;
  a.qscale = P.scale * kLog2e;
  a.early = decode_overlap_allowed() ? 1 : 0;
  a.err_word = device_error_word();
  if (!a.err_word) return WST_ERR_CUDA;

  CUtensorMap kmap, vmap;
  KvMapKey key{};
  key.d0 = static_cast<uint64_t>(P.hd);
  key.d1 = 16;
  key.d2 = static_cast<uint64_t>(P.n_kv);
  key.d3 = static_cast<uint64_t>(P.n_pool_pages);
  key.b1 = 16;
  key.rank = P.hd == 128 ? 5 : 4; /* head_dim 128: both halves of a page in one box */
  key.base = P.k;
  wst_status_t st = cached_kv_tensor_map(&kmap, key);
  if (st != WST_OK) return st;
  key.base = P.v;
  st = cached_kv_tensor_map(&vmap, key);
  if (st != WST_OK) return st;

  /* one persistent CTA per SM, never more CTAs than there can be tiles */
  long long ctas = facts.sm_count;
  const long long tiles_bound = units * max_tiles;
  if (ctas > tiles_bound) ctas = tiles_bound;
  if (P.span_ctas > 0 && P.span_ctas < ctas) ctas = P.span_ctas;
  const dim3 grid(static_cast<unsigned>(ctas));
  st = P.hd == 128
           ? launch_kernel<PCfg<128>>(P, attn_verify_span_kernel<128>, a, kmap, vmap, grid)
           : launch_kernel<PCfg<64>>(P, attn_verify_span_kernel<64>, a, kmap, vmap, grid);
  if (st != WST_OK) return st;

  SplitMerge m;
  m.scratch = P.scratch;
  m.out = P.out;
  m.cu_tokens = P.cu_tokens;
  m.n_tok = P.n;
  m.tok_seq_stride = 0;
  m.n_q = P.n_q;
  m.n_kv = P.n_kv;
  m.hd = P.hd;
  m.n_splits = static_cast<int>(cap);
  m.slice_counts = a.slice_counts;
  m.n_rowblk = 1;
  m.tpb = P.n;
  m.rows_cap = rows_cap;
  m.n_units = static_cast<int>(units);
  m.name = P.name;
  return launch_split_merge(m);
}

bool prefill_split_supports(int n_q, int n_kv, int hd, int n_tok_max) {
  if (hd != 64 && hd != 128) return false;
  if (n_kv <= 0 || n_q % n_kv != 0) return false;
  /* every query row of a (sequence, KV head) unit in one 128-row tile */
  return static_cast<long long>(n_tok_max) * (n_q / n_kv) <= 128;
}

wst_status_t launch_prefill(const PrefillLaunch &P) {
  DeviceFacts facts;
  if (!device_facts(&facts)) return WST_ERR_CUDA;
  if (facts.cc_major < 10)
    return fail(WST_ERR_UNSUPPORTED_ARCH, "%s: this library is built for sm_100a only", P.name);
  if (!aligned16(P.qkv) || !aligned16(P.k) || !aligned16(P.v) || !aligned16(P.out))
    return fail(WST_ERR_INVALID_ARG, "%s: buffers must be 16-byte aligned", P.name);

  PrefillArgs a{};
  a.q = P.qkv;
  a.q_tok_stride = P.q_tok_stride;
  a.q16 = P.q16 ? 1 : 0;
  a.out = P.out;
  a.scratch = P.scratch;
  a.pos0_dev = P.pos0_dev;
  a.cu_tokens = P.cu_tokens;
  a.page_table = P.page_table;
  a.max_pages = P.max_pages;
  a.n_pool_pages = P.n_pool_pages;
  a.n_q = P.n_q;
  a.n_kv = P.n_kv;
  a.gqa = P.n_q / P.n_kv;
  a.pos0 = P.pos0;
  a.n = P.n;
  a.max_seq = P.max_seq;
  a.tpt = 128 / a.gqa;
  a.n_qtiles = (P.n + a.tpt - 1) / a.tpt;
  a.qscale = P.scale * kLog2e;
  a.err_word = device_error_word();
  if (!a.err_word) return WST_ERR_CUDA;

  /* slices of the KV range: every (unit, query tile) writes one partial per slice */
  int splits = P.n_splits > 0 ? P.n_splits : 1;
  a.rows_cap = (P.n < a.tpt ? P.n : a.tpt) * a.gqa;
  const long long units = static_cast<long long>(P.n_seq) * P.n_kv;
  if (!P.scratch || !aligned16(P.scratch)) splits = 1;
  while (splits > 1 &&
         units * a.n_qtiles * splits * a.rows_cap * (P.hd + 4) > P.scratch_floats)
    --splits;
  a.n_splits = splits;
  const int max_tiles = (P.max_len > 0 ? P.max_len : P.max_seq) / 128 + 1;
  a.tiles_per_slice = splits > 1 && !P.even_slices ? (max_tiles + splits - 1) / splits : 0;

  CUtensorMap kmap, vmap;
  KvMapKey key{};
  key.d0 = static_cast<uint64_t>(P.hd);
  if (P.page_table) {
    key.d1 = 16;
    key.d2 = static_cast<uint64_t>(P.n_kv);
    key.d3 = static_cast<uint64_t>(P.n_pool_pages);
    key.b1 = 16;
    key.rank = 4;
  } else {
    key.d1 = static_cast<uint64_t>(P.max_seq);
    key.d2 = static_cast<uint64_t>(P.n_kv) * P.n_seq;
    key.d3 = 1;
    key.b1 = 128;
    key.rank = 3;
  }
  key.base = P.k;
  wst_status_t st = cached_kv_tensor_map(&kmap, key);
  if (st != WST_OK) return st;
  key.base = P.v;
  st = cached_kv_tensor_map(&vmap, key);
  if (st != WST_OK) return st;

  /* Two query tiles per CTA whenever there are two: every K/V tile fetched from L2
   * serves 256 query rows and one tile's MMAs run under the other's softmax (1117
   * against 841 TFLOP/s on the last chunk of the 4 x 8192-token, 32-head shape).
   * The one-tile kernel takes what is left: launches that finish sooner with one
   * tile per CTA (few tiles), paged caches, ragged batches and the sliced form. */
  /* waves x measured time per KV tile: a CTA with two query tiles takes 1.5 times as
   * long per KV tile as a CTA with one (1.86 against 1.24 us) */
  const long long tiles = units * a.n_qtiles, pairs = units * ((a.n_qtiles + 1) / 2);
  const long long sm = facts.sm_count;
  const bool pays = (pairs + sm - 1) / sm * 3 < (tiles + sm - 1) / sm * 2;
  const bool pair = P.force_pair >= 0 && (P.force_pair > 0 || (a.n_qtiles >= 2 && pays)) &&
                    splits == 1 && !P.page_table && !P.cu_tokens;
  const unsigned gx = splits > 1 ? a.n_qtiles * splits : (pair ? (a.n_qtiles + 1) / 2 : a.n_qtiles);
  const dim3 grid(gx, static_cast<unsigned>(P.n_kv), static_cast<unsigned>(P.n_seq));
  if (pair)
    st = P.hd == 128
             ? launch_kernel<P2Cfg<128>>(P, attn_prefill_pair_kernel<128>, a, kmap, vmap, grid)
             : launch_kernel<P2Cfg<64>>(P, attn_prefill_pair_kernel<64>, a, kmap, vmap, grid);
  else if (P.page_table)
    st = P.hd == 128
             ? launch_kernel<PCfg<128>>(P, attn_prefill_kernel<128, true>, a, kmap, vmap, grid)
             : launch_kernel<PCfg<64>>(P, attn_prefill_kernel<64, true>, a, kmap, vmap, grid);
  else
    st = P.hd == 128
             ? launch_kernel<PCfg<128>>(P, attn_prefill_kernel<128, false>, a, kmap, vmap, grid)
             : launch_kernel<PCfg<64>>(P, attn_prefill_kernel<64, false>, a, kmap, vmap, grid);
  if (st != WST_OK || splits == 1) return st;

  SplitMerge m;
  m.scratch = P.scratch;
  m.out = P.out;
  m.cu_tokens = P.cu_tokens;
  m.n_tok = P.n;
  m.tok_seq_stride = P.cu_tokens ? 0 : P.n;
  m.n_q = P.n_q;
  m.n_kv = P.n_kv;
  m.hd = P.hd;
  m.n_splits = splits;
  m.n_rowblk = a.n_qtiles;
  m.tpb = a.tpt;
  m.rows_cap = a.rows_cap;
  m.n_units = static_cast<int>(units * a.n_qtiles);
  m.name = P.name;
  return launch_split_merge(m);
}

}  // namespace wst
