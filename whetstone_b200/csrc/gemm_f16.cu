/* The multi-token projection either side of the attention path:
 *
 *     y[j][r] (+)= sum_c x[j][c] * w[r][c] + bias[r]        j < n tokens, r < out_f
 *
 * x [n][in_f] and w [out_f][in_f] fp16, y [n][out_f] fp32 -- wst_gemm_fp16 of the
 * engine (cuda/chunk_gemm.cu:178-258, dispatch :340-365).  The engine's kernel keeps
 * the weights outermost and covers at most 16 tokens per pass; every weight row is a
 * warp's dot product in half2.  Here any number of tokens is one launch:
 *
 *   both operands are K-major, so a 128-token x BN-feature tile is
 *   tcgen05.mma.kind::f16 M128 x N(BN) x K16 straight from the TMA-filled,
 *   128-byte-swizzled stages (x tile 16 KB + w tile BN*128 B per 64 columns of K);
 *   fp32 accumulators in tensor memory, TWO of them, so the epilogue of one tile
 *   (tensor memory -> registers -> + bias (+ y) -> global) runs under the main loop
 *   of the next; persistent CTAs, one per SM, walk the tiles token-tile fastest so
 *   that the CTAs running at the same time share a weight tile in L2.
 *
 *   BN = 256 for real chunks (A 4 KB + B 8 KB of shared memory per 128-clock MMA,
 *   96 bytes per clock); BN = 32, 48 or 64 when the token count is small and the
 *   launch is a stream of the weights: as many CTAs as there are SMs pull on HBM.
 *
 * Products are exact in fp32 and accumulated in fp32 (the engine's kernel rounds
 * every group of four products to fp16 first): results differ from the engine's by
 * its own rounding, well inside the 2e-3 relative bound its tests use
 * (tests/chunk_kernels.rs:44-49).
 *
 * Shapes the tensor maps cannot describe (in_f not a multiple of 8, unaligned
 * bases) go to a plain warp-per-output kernel.
 */

#include <initializer_list>

#include "tensor_map.cuh"
#include "wst_common.cuh"
#include "wst_ptx.cuh"

namespace wst {
namespace {

using namespace ptx;

/* BN feature rows per tile; KS 64-column slabs of K per pipeline stage; RB token rows
 * fetched per tile (the MMA is always M = 128: with RB < 128 the tensor core reads
 * whatever follows the fetched rows in shared memory, and the accumulator rows that
 * come of it belong to tokens that do not exist and are never stored). */
template <int BN, int KS, int RB>
struct GCfg {
  static constexpr int BM = 128, BK = 64 * KS;
  static constexpr int A_SLAB = RB * 128, B_SLAB = BN * 128;
  static constexpr int A_BYTES = KS * A_SLAB;
  static constexpr int B_BYTES = KS * B_SLAB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NSTAGE = (200 * 1024) / STAGE_BYTES < 8 ? (200 * 1024) / STAGE_BYTES : 8;
  static constexpr int OFF_BAR = NSTAGE * STAGE_BYTES;
  static constexpr int NBAR = 2 * NSTAGE + 4;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 16 + 1024;
  static constexpr int ACC_STRIDE = BN <= 32 ? 32 : BN <= 64 ? 64 : 256; /* columns per accumulator */
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  static_assert(RB % 8 == 0 && NSTAGE >= 2, "stage geometry");
  /* the M = 128 read of the last slab of the last stage stays inside the ring */
  static_assert(KS == 1 ? RB == 128 : 128 * 128 <= A_SLAB + B_BYTES, "over-read leaves the ring");
};

struct GemmArgs {
  const __half *bias;
  float *y;
  int in_f, out_f, n, accum;
  int m_tiles, n_tiles;
  unsigned int *err_word;
  /* the fused form (ROPE): the tile's columns are whole heads of the qkv row; they are
   * normed, rotated and stored where the attention reads them instead of going to y */
  /* the int4 form (INT4): the weights come packed, one 16-byte word of 32 nibbles and one
   * byte of two 4-bit scale indices per group of 32 along K, one (d, dmin) pair per row */
  const uint4 *qw;       /* [out_f][in_f / 32] */
  const uint8_t *si;     /* [out_f][in_f / 32]: ls | lm << 4 */
  const __half2 *sb;     /* [out_f]: (d, dmin) */
  __half *q_out;         /* [n][n_q * hd] */
  __half *k_cache;       /* [n_seq][n_kv][max_seq][hd] */
  __half *v_cache;
  const float *cos_tab;  /* [table_len][hd / 2] */
  const float *sin_tab;
  const __half *q_gain;  /* [hd] or null */
  const __half *k_gain;
  const int32_t *seq_pos0; /* [n_seq] */
  int n_q, n_kv, hd, n_per_seq, max_seq, table_len;
  float eps;
};

/* Epilogue of the fused form for one head of one token: HD accumulator columns from
 * tensor memory (+ bias) -> per-head RMS norm with fp16 gains (q and k heads, if gains
 * are given) -> half-rotation RoPE at the token's position -> fp16, to the q buffer or
 * to the token's cache row; v heads are narrowed and stored as they are.  The
 * arithmetic is that of rope_append_kernel (norm before rotation, x * inv * gain,
 * cuda/decode.cu:112-178 and cuda/chunk_ops.cu:101-150 of the engine). */
template <int HD>
__device__ __forceinline__ void rope_head_epilogue(const GemmArgs &a, uint32_t tmem_head, int head,
                                                   int tpos, long long kv_row, int tok, bool valid) {
  float x[HD];
#pragma unroll
  for (int c0 = 0; c0 < HD; c0 += 32) {
    uint32_t v[32];
    tmem_ld_32x32(tmem_head + c0, v);
    tmem_ld_wait();
#pragma unroll
    for (int e = 0; e < 32; ++e) x[c0 + e] = __uint_as_float(v[e]);
  }
  if (!valid) return;
  if (a.bias) {
#pragma unroll
    for (int e = 0; e < HD; e += 2) {
      const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(a.bias + head * HD + e));
      x[e] += b.x;
      x[e + 1] += b.y;
    }
  }
  constexpr int HALF = HD / 2;
  const bool is_q = head < a.n_q, is_k = !is_q && head < a.n_q + a.n_kv;
  __half *dst;
  if (is_q) {
    dst = a.q_out + (static_cast<long long>(tok) * a.n_q + head) * HD;
  } else {
    const int kvh = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
    dst = (is_k ? a.k_cache : a.v_cache) + kv_row + static_cast<long long>(kvh) * a.max_seq * HD;
  }
  if (is_q || is_k) {
    const __half *gain = is_q ? a.q_gain : a.k_gain;
    if (gain) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < HALF; ++e) ss = fmaf(x[e], x[e], fmaf(x[e + HALF], x[e + HALF], ss));
      const float inv = rsqrtf(ss / static_cast<float>(HD) + a.eps);
#pragma unroll
      for (int e = 0; e < HD; e += 2) {
        const float2 g = __half22float2(*reinterpret_cast<const __half2 *>(gain + e));
        x[e] = x[e] * inv * g.x;
        x[e + 1] = x[e + 1] * inv * g.y;
      }
    }
    const float4 *ct = reinterpret_cast<const float4 *>(a.cos_tab + static_cast<long long>(tpos) * HALF);
    const float4 *st = reinterpret_cast<const float4 *>(a.sin_tab + static_cast<long long>(tpos) * HALF);
#pragma unroll
    for (int e = 0; e < HALF; e += 4) {
      const float4 c = __ldg(ct + e / 4), sn = __ldg(st + e / 4);
      const float cc[4] = {c.x, c.y, c.z, c.w}, ss4[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x1 = x[e + k], x2 = x[e + k + HALF];
        x[e + k] = x1 * cc[k] - x2 * ss4[k];
        x[e + k + HALF] = x2 * cc[k] + x1 * ss4[k];
      }
    }
  }
#pragma unroll
  for (int e = 0; e < HD; e += 8) {
    uint4 o;
    o.x = pack_half2(x[e], x[e + 1]);
    o.y = pack_half2(x[e + 2], x[e + 3]);
    o.z = pack_half2(x[e + 4], x[e + 5]);
    o.w = pack_half2(x[e + 6], x[e + 7]);
    *reinterpret_cast<uint4 *>(dst + e) = o;
  }
}

/* Threads of a CTA: 4 epilogue warps, the MMA warp, the TMA warp, and for the int4 form
 * sixteen warps that unpack the weight tile into shared memory. */
constexpr int kUnpackThreads = 512;
constexpr int gemm_threads(bool int4) { return int4 ? 192 + kUnpackThreads : 192; }

template <int BN, int KS, int RB, bool ROPE, bool INT4>
__global__ void __launch_bounds__(gemm_threads(INT4), 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                const GemmArgs a) {
  using C = GCfg<BN, KS, RB>;
  constexpr int NSTAGE = C::NSTAGE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto bar = [bar0](int i) { return bar0 + 8u * i; };
  constexpr int FULL = 0, EMPTY = NSTAGE, ACC_FULL = 2 * NSTAGE, ACC_EMPTY = ACC_FULL + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + C::OFF_BAR + C::NBAR * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(bar(FULL + i), INT4 ? 1 + kUnpackThreads / 32 : 1); /* the TMA lane (+ the unpacking warps) */
      mbar_init(bar(EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(ACC_FULL + i), 1);
      mbar_init(bar(ACC_EMPTY + i), 128);
    }
    mbar_init_fence();
    tma_prefetch_desc(&xmap);
    if constexpr (!INT4) tma_prefetch_desc(&wmap);
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  grid_dependency_wait();

  const int n_tiles_total = a.m_tiles * a.n_tiles;
  const int k_blocks = (a.in_f + C::BK - 1) / C::BK;
  /* tile i of this CTA is global tile blockIdx.x + i * gridDim.x: token tile fastest */

  if (warp == 5) {
    /* ------------------------------------------------------ TMA producer */
    if (lane == 0) {
      int it = 0; /* stage uses so far */
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x) {
        const int m0 = (tile % a.m_tiles) * C::BM, n0 = (tile / a.m_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int st = it % NSTAGE;
          if (it >= NSTAGE &&
              !mbar_wait(bar(EMPTY + st), ((it / NSTAGE) - 1) & 1, a.err_word, 0x601u)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(bar(FULL + st), INT4 ? C::A_BYTES : C::STAGE_BYTES);
          if constexpr (INT4) { /* the weight tile comes from the unpacking warps */
            tma_load_3d(sbase + st * C::STAGE_BYTES, &xmap, bar(FULL + st), kb * C::BK, m0, 0);
          } else if constexpr (KS == 1) { /* maps over [rows][in_f]: columns past in_f read as zero */
            tma_load_3d(sbase + st * C::STAGE_BYTES, &xmap, bar(FULL + st), kb * C::BK, m0, 0);
            tma_load_3d(sbase + st * C::STAGE_BYTES + C::A_BYTES, &wmap, bar(FULL + st), kb * C::BK,
                        n0, 0);
          } else { /* maps over [in_f / 64][rows][64]: KS slabs per request */
            tma_load_3d(sbase + st * C::STAGE_BYTES, &xmap, bar(FULL + st), 0, m0, kb * KS);
            tma_load_3d(sbase + st * C::STAGE_BYTES + C::A_BYTES, &wmap, bar(FULL + st), 0, n0,
                        kb * KS);
          }
        }
      }
    }
  } else if (warp >= 6) {
    /* ---------------------- int4 weights -> fp16 tile in the operand layout
     * (cuda/hier.cuh:8-13, the arithmetic of cuda/chunk_gemm.cu:121-132).  A thread takes
     * the groups g = tid, tid + 512, ... of the stage: row g / 2 of the tile, 32-column
     * half g % 2 of the 64-column k-block = four 16-byte chunks of the row's 128 swizzled
     * bytes. */
    if constexpr (INT4) {
      /* The packed words of a group are one dependent load from DRAM; a thread that asked
       * for them only when their stage fell free spent a memory latency per k-block (228 us
       * for the projection that takes 101 with fp16 weights).  So each thread keeps the
       * words of its groups for the next kAhead k-blocks in registers. */
      constexpr int kAhead = 4;
      constexpr int G = 2 * BN / kUnpackThreads > 0 ? 2 * BN / kUnpackThreads : 1;
      const int tid = threadIdx.x - 6 * 32;
      const int vec_per_row = a.in_f / 32;
      const int my_tiles = blockIdx.x < n_tiles_total
                               ? (n_tiles_total - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1
                               : 0;
      const int total = my_tiles * k_blocks;
      struct Raw { /* as loaded: nothing may depend on these before their stage is unpacked */
        uint4 w;
        unsigned idx;
        __half2 dd;
      };
      Raw ahead[kAhead][G];
      /* the fetch cursor walks (tile, k-block) in the order of the stages; everything that
       * needs a division is recomputed once per tile (the unpacking warps are bound by the
       * instructions they issue: with the tile and k-block derived from the stage counter
       * by three divisions per k-block, the address arithmetic cost as much as the
       * unpacking) */
      int f_left = total, f_kb = 0, f_tile = blockIdx.x;
      size_t f_at[G];   /* group index of (row, half) at k-block 0 of the cursor's tile */
      bool f_row_ok[G];
      int f_grow[G];
      auto fetch_tile = [&]() {
        const int n0 = (f_tile / a.m_tiles) * BN;
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const int g = tid + j * kUnpackThreads;
          const int grow = n0 + (g >> 1);
          f_row_ok[j] = g < 2 * BN && grow < a.out_f;
          f_grow[j] = grow;
          f_at[j] = static_cast<size_t>(grow) * vec_per_row + (g & 1);
        }
      };
      fetch_tile();
      auto fetch = [&](Raw (&dst)[G]) {
#pragma unroll
        for (int j = 0; j < G; ++j) {
          dst[j].w = make_uint4(0u, 0u, 0u, 0u);
          dst[j].idx = 0u;
          dst[j].dd = __float2half2_rn(0.f); /* past the last row or the last group: zeros */
          const int v = f_kb * 2 + ((tid + j * kUnpackThreads) & 1);
          if (f_left > 0 && f_row_ok[j] && v < vec_per_row) {
            const size_t at = f_at[j] + 2 * f_kb;
            dst[j].w = __ldg(a.qw + at);
            dst[j].idx = __ldg(a.si + at);
            dst[j].dd = __ldg(a.sb + f_grow[j]);
          }
        }
        --f_left;
        if (++f_kb == k_blocks) {
          f_kb = 0;
          f_tile += gridDim.x;
          if (f_left > 0) fetch_tile();
        }
      };
      auto unpack = [&](int it, const Raw (&src)[G]) -> bool {
        const int st = it % NSTAGE;
        if (it >= NSTAGE && !mbar_wait(bar(EMPTY + st), ((it / NSTAGE) - 1) & 1, a.err_word, 0x605u))
          return false;
        uint8_t *btile = smem + st * C::STAGE_BYTES + C::A_BYTES;
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const int g = tid + j * kUnpackThreads;
          if (g < 2 * BN) {
            const int row = g >> 1, half = g & 1;
            const uint32_t words[4] = {src[j].w.x, src[j].w.y, src[j].w.z, src[j].w.w};
            /* A nibble q dropped into byte 2 of 0x3F000000 is the float 0.5 + q / 256, one
             * byte permute per weight; then w = q s - dmin lm = (256 s) f - (128 s + dmin lm)
             * with s = d * ls is ONE fp32 fma per weight, and the result is rounded to fp16
             * once -- the only difference from the exact weight, random in sign.  (In half2
             * arithmetic, (q * ls) * d - fp16(lm * dmin), the rounded offset is common to the
             * 32 weights of a group and adds up along the group: 9.7e-3 from the exact
             * product on the engine's test case where this form has 1.3e-3 and the engine's
             * own kernel 7.7e-3, for 6 % less time.) */
            const float2 dd = __half22float2(src[j].dd);
            const float s1 = dd.x * static_cast<float>(src[j].idx & 0xFu); /* d * ls */
            const float sc = 256.0f * s1;
            const float mt = fmaf(-128.0f, s1, -dd.y * static_cast<float>(src[j].idx >> 4));
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) { /* 8 weights = one 16-byte chunk per word */
              const uint32_t even = words[wi] & 0x0F0F0F0Fu, odd = (words[wi] >> 4) & 0x0F0F0F0Fu;
              uint32_t o[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) { /* weights 2i (low nibble of byte i) and 2i + 1 */
                const float f0 = __uint_as_float(__byte_perm(even, 0x3F000000u, 0x7044u | (i << 8)));
                const float f1 = __uint_as_float(__byte_perm(odd, 0x3F000000u, 0x7044u | (i << 8)));
                o[i] = pack_half2(fmaf(f0, sc, mt), fmaf(f1, sc, mt));
              }
              *reinterpret_cast<uint4 *>(btile + swz128(row, half * 4 + wi)) =
                  make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
        /* one arrival per warp: 256 arrivals on one barrier word took longer than the
         * unpacking itself */
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FULL + st));
        return true;
      };
#pragma unroll
      for (int u = 0; u < kAhead; ++u) fetch(ahead[u]);
      bool ok = true;
      for (int it0 = 0; ok && it0 < total; it0 += kAhead) {
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
          if (it0 + u < total) {
            ok = ok && unpack(it0 + u, ahead[u]);
            fetch(ahead[u]);
          }
        }
      }
    }
  } else if (warp == 4) {
    /* -------------------------------------------------------- MMA issuer */
    constexpr uint32_t idesc = umma_idesc(128, BN, 0);
    int it = 0, local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles_total; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      /* the epilogue of the tile two back has emptied this accumulator */
      if (local >= 2 &&
          !mbar_wait(bar(ACC_EMPTY + buf), ((local >> 1) - 1) & 1, a.err_word, 0x602u)) break;
      tc_fence_after_sync();
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int st = it % NSTAGE;
        if (!mbar_wait(bar(FULL + st), (it / NSTAGE) & 1, a.err_word, 0x603u)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a_lo = umma_desc_lo(sbase + st * C::STAGE_BYTES, 16);
        const uint32_t b_lo = umma_desc_lo(sbase + st * C::STAGE_BYTES + C::A_BYTES, 16);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < C::BK / 16; ++ks) {
            const uint32_t a_off = ((ks >> 2) * C::A_SLAB + (ks & 3) * 32) >> 4;
            const uint32_t b_off = ((ks >> 2) * C::B_SLAB + (ks & 3) * 32) >> 4;
            umma_ss_f16_lohi(tmem + buf * C::ACC_STRIDE, a_lo + a_off, b_lo + b_off, kDescHi, idesc,
                             (kb > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(bar(EMPTY + st));
          if (kb == k_blocks - 1) umma_commit(bar(ACC_FULL + buf));
        }
        __syncwarp();
      }
    }
  } else {
    /* --------------------------------------- epilogue: thread r owns token row r */
    const int r = warp * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const bool vec = (a.out_f & 3) == 0;
    int local = 0;
    for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % a.m_tiles) * C::BM, n0 = (tile / a.m_tiles) * BN;
      if (!mbar_wait_idle(bar(ACC_FULL + buf), (local >> 1) & 1, a.err_word, 0x604u)) break;
      tc_fence_after_sync();
      const int row = m0 + r;
      if constexpr (ROPE) {
        /* the token's sequence, cache position (clamped, never trusted) and cache row */
        const bool valid = row < a.n;
        const int sq = valid ? row / a.n_per_seq : 0;
        int pos = valid ? a.seq_pos0[sq] + (row - sq * a.n_per_seq) : 0;
        pos = pos < 0 ? 0 : pos;
        pos = pos < a.max_seq - 1 ? pos : a.max_seq - 1;
        const int tpos = pos < a.table_len - 1 ? pos : a.table_len - 1;
        const long long kv_row =
            (static_cast<long long>(sq) * a.n_kv * a.max_seq + pos) * static_cast<long long>(a.hd);
        const uint32_t acc = tmem + lane_base + buf * C::ACC_STRIDE;
        if (a.hd == 128) {
#pragma unroll 1
          for (int h = 0; h < BN / 128; ++h) {
            const int head = (n0 >> 7) + h;
            rope_head_epilogue<128>(a, acc + h * 128, head, tpos, kv_row, row,
                                    valid && head * 128 < a.out_f);
          }
        } else {
#pragma unroll 1
          for (int h = 0; h < BN / 64; ++h) {
            const int head = (n0 >> 6) + h;
            rope_head_epilogue<64>(a, acc + h * 64, head, tpos, kv_row, row,
                                   valid && head * 64 < a.out_f);
          }
        }
        tc_fence_before_sync();
        mbar_arrive(bar(ACC_EMPTY + buf));
        continue;
      }
      float *yrow = a.y + static_cast<long long>(row) * a.out_f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + buf * C::ACC_STRIDE + c0, v);
        tmem_ld_wait();
        const int col0 = n0 + c0;
        if (row < a.n && col0 < a.out_f) {
          if (vec && c0 + 32 <= BN && col0 + 32 <= a.out_f) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              float4 o = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                     __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
              if (a.bias) {
                const uint2 b = __ldg(reinterpret_cast<const uint2 *>(a.bias + col0 + e));
                const float2 b0 = __half22float2(*reinterpret_cast<const __half2 *>(&b.x));
                const float2 b1 = __half22float2(*reinterpret_cast<const __half2 *>(&b.y));
                o.x += b0.x; o.y += b0.y; o.z += b1.x; o.w += b1.y;
              }
              float4 *dst = reinterpret_cast<float4 *>(yrow + col0 + e);
              if (a.accum) {
                const float4 old = *dst;
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *dst = o;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              if (c0 + e < BN && col0 + e < a.out_f) {
                float o = __uint_as_float(v[e]);
                if (a.bias) o += __half2float(a.bias[col0 + e]);
                if (a.accum) o += yrow[col0 + e];
                yrow[col0 + e] = o;
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar(ACC_EMPTY + buf));
    }
    grid_launch_dependents();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

/* Any shape: one warp per (token, output feature), fp32 accumulation. */
__global__ void __launch_bounds__(256)
gemm_f16_plain_kernel(const __half *w, const __half *x, const __half *bias, float *y, int in_f,
                      int out_f, int n, int accum) {
  const long long unit = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (unit >= static_cast<long long>(n) * out_f) return;
  const int lane = threadIdx.x & 31;
  const int j = static_cast<int>(unit / out_f), r = static_cast<int>(unit % out_f);
  const __half *wr = w + static_cast<long long>(r) * in_f;
  const __half *xr = x + static_cast<long long>(j) * in_f;
  float acc = 0.f;
  for (int c = lane; c < in_f; c += 32) acc = fmaf(__half2float(wr[c]), __half2float(xr[c]), acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    if (bias) acc += __half2float(bias[r]);
    float *dst = y + static_cast<long long>(j) * out_f + r;
    *dst = accum ? *dst + acc : acc;
  }
}

/* The operand maps.  KS == 1: [rows][in_f] as it lies, box 64 columns x `box_rows`.
 * KS > 1 (in_f a multiple of 64): the same memory as [in_f / 64][rows][64] -- slab,
 * row, column -- so that one request brings KS slabs. */
wst_status_t operand_map(CUtensorMap *out, const void *base, int in_f, int rows, int box_rows,
                         int ks) {
  if (ks == 1) {
    KvMapKey key{};
    key.rank = 3;
    key.base = base;
    key.d0 = static_cast<uint64_t>(in_f);
    key.d1 = static_cast<uint64_t>(rows);
    key.d2 = 1;
    key.d3 = 1;
    key.b1 = static_cast<uint32_t>(box_rows);
    return cached_kv_tensor_map(out, key);
  }
  struct Slot {
    const void *base;
    int in_f, rows, box_rows, ks;
    CUtensorMap map;
    bool used;
  };
  static thread_local Slot slots[16];
  const uint64_t h = (reinterpret_cast<uint64_t>(base) >> 8) ^ (static_cast<uint64_t>(rows) * 0x9E3779B97F4A7C15ull);
  Slot &sl = slots[(h ^ (h >> 31)) % 16];
  if (sl.used && sl.base == base && sl.in_f == in_f && sl.rows == rows && sl.box_rows == box_rows &&
      sl.ks == ks) {
    *out = sl.map;
    return WST_OK;
  }
  const uint64_t dims[3] = {64, static_cast<uint64_t>(rows), static_cast<uint64_t>(in_f / 64)};
  const uint64_t strides[2] = {static_cast<uint64_t>(in_f) * 2, 128};
  const uint32_t box[3] = {64, static_cast<uint32_t>(box_rows), static_cast<uint32_t>(ks)};
  const wst_status_t st = make_kv_tensor_map(out, base, 3, dims, strides, box);
  if (st != WST_OK) return st;
  sl = Slot{base, in_f, rows, box_rows, ks, *out, true};
  return WST_OK;
}

template <int BN, int KS, int RB, bool ROPE = false, bool INT4 = false>
wst_status_t launch_gemm(const void *w, const void *x, GemmArgs a, int sm_count) {
  using C = GCfg<BN, KS, RB>;
  CUtensorMap xmap, wmap;
  wst_status_t st = operand_map(&xmap, x, a.in_f, a.n, RB, KS);
  if (st != WST_OK) return st;
  if (INT4) {
    wmap = xmap; /* not used: the weight tile is unpacked by the CTA itself */
  } else {
    st = operand_map(&wmap, w, a.in_f, a.out_f, BN, KS);
    if (st != WST_OK) return st;
  }
  static thread_local int configured_dev = -1;
  int dev = 0;
  WST_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    WST_CUDA(cudaFuncSetAttribute(gemm_f16_kernel<BN, KS, RB, ROPE, INT4>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured_dev = dev;
  }
  a.m_tiles = (a.n + C::BM - 1) / C::BM;
  a.n_tiles = (a.out_f + BN - 1) / BN;
  const long long tiles = static_cast<long long>(a.m_tiles) * a.n_tiles;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles < sm_count ? tiles : sm_count));
  cfg.blockDim = dim3(gemm_threads(INT4));
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = current_stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_f16_kernel<BN, KS, RB, ROPE, INT4>, xmap, wmap, a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("wst_gemm_fp16 (launch)", e);
  return WST_OK;
}

template <int KS, int RB>
wst_status_t launch_narrow(int bn, const void *w, const void *x, const GemmArgs &a, int sm_count) {
  switch (bn) {
    case 32: return launch_gemm<32, KS, RB>(w, x, a, sm_count);
    case 48: return launch_gemm<48, KS, RB>(w, x, a, sm_count);
    default: return launch_gemm<64, KS, RB>(w, x, a, sm_count);
  }
}

}  // namespace
}  // namespace wst

using namespace wst;

extern "C" wst_status_t wst_gemm_fp16(const void *w, const void *x, const void *bias, void *y,
                                      int32_t in_f, int32_t out_f, int32_t n, int32_t accum) {
  WST_CHECK_ARG(w && x && y, "wst_gemm_fp16: null pointer");
  WST_CHECK_ARG(in_f > 0 && out_f > 0, "wst_gemm_fp16: non-positive dimension");
  WST_CHECK_ARG(n > 0, "wst_gemm_fp16: n must be positive");
  DeviceFacts facts;
  if (!device_facts(&facts)) return WST_ERR_CUDA;

  const bool tma_ok = in_f % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                      (!bias || (reinterpret_cast<uintptr_t>(bias) & 7) == 0) && facts.cc_major >= 10;
  if (!tma_ok) {
    const long long units = static_cast<long long>(n) * out_f;
    const long long blocks = (units + 7) / 8;
    WST_CHECK_ARG(blocks <= 0x7fffffffLL, "wst_gemm_fp16: too many outputs");
    gemm_f16_plain_kernel<<<static_cast<unsigned>(blocks), 256, 0, current_stream()>>>(
        static_cast<const __half *>(w), static_cast<const __half *>(x),
        static_cast<const __half *>(bias), static_cast<float *>(y), in_f, out_f, n, accum);
    WST_LAUNCHED("wst_gemm_fp16");
    return WST_OK;
  }

  unsigned int *err_word = device_error_word();
  if (!err_word) return WST_ERR_CUDA;
  GemmArgs a{};
  a.bias = static_cast<const __half *>(bias);
  a.y = static_cast<float *>(y);
  a.in_f = in_f;
  a.out_f = out_f;
  a.n = n;
  a.accum = accum;
  a.err_word = err_word;

  /* Few tokens: the launch streams the weights once and is bound by how many SMs pull on
   * HBM, so the feature tile is the one of 32, 48 or 64 rows that gives a CTA the least
   * to stream (6144 features: 128 tiles of 48; 4096: 128 tiles of 32).  Else 256-feature
   * tiles for the tensor pipe. */
  int bn = 256;
  if (n <= 128) {
    long long best = -1;
    for (int cand : {64, 48, 32}) {
      const long long tiles = (out_f + cand - 1) / cand;
      const long long per_cta = (tiles + facts.sm_count - 1) / facts.sm_count * cand;
      if (best < 0 || per_cta < best) { best = per_cta; bn = cand; }
    }
  }
  if (n > 128) return launch_gemm<256, 1, 128>(w, x, a, facts.sm_count);
  /* a handful of tokens (decode-side chunks, speculative verification): four slabs of K
   * per request, and only the token rows that exist are fetched */
  if (in_f % 64 == 0 && n <= 16) return launch_narrow<4, 16>(bn, w, x, a, facts.sm_count);
  if (in_f % 64 == 0 && n <= 64) return launch_narrow<4, 64>(bn, w, x, a, facts.sm_count);
  if (in_f % 64 == 0) return launch_narrow<4, 128>(bn, w, x, a, facts.sm_count);
  return launch_narrow<1, 128>(bn, w, x, a, facts.sm_count);
}

extern "C" wst_status_t wst_gemm_int4_hier(const void *qw, const void *si, const void *sb,
                                           const void *x, const void *bias, void *y,
                                           int32_t in_f, int32_t out_f, int32_t n, int32_t accum) {
  WST_CHECK_ARG(qw && si && sb && x && y, "wst_gemm_int4_hier: null pointer");
  WST_CHECK_ARG(in_f > 0 && out_f > 0, "wst_gemm_int4_hier: non-positive dimension");
  WST_CHECK_ARG(n > 0, "wst_gemm_int4_hier: n must be positive");
  WST_CHECK_ARG(in_f % 32 == 0, "wst_gemm_int4_hier: in_features must be a multiple of 32");
  WST_CHECK_ARG((reinterpret_cast<uintptr_t>(qw) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(sb) & 3) == 0 &&
                    (!bias || (reinterpret_cast<uintptr_t>(bias) & 7) == 0),
                "wst_gemm_int4_hier: buffers must be 16-byte aligned");
  DeviceFacts facts;
  if (!device_facts(&facts)) return WST_ERR_CUDA;
  if (facts.cc_major < 10)
    return fail(WST_ERR_UNSUPPORTED_ARCH, "wst_gemm_int4_hier: this library is built for sm_100a only");
  unsigned int *err_word = device_error_word();
  if (!err_word) return WST_ERR_CUDA;
  GemmArgs a{};
  a.bias = static_cast<const __half *>(bias);
  a.y = static_cast<float *>(y);
  a.in_f = in_f;
  a.out_f = out_f;
  a.n = n;
  a.accum = accum;
  a.err_word = err_word;
  a.qw = static_cast<const uint4 *>(qw);
  a.si = static_cast<const uint8_t *>(si);
  a.sb = static_cast<const __half2 *>(sb);
  /* the token count decides the feature tile as for fp16 weights: 256 rows for the tensor
   * pipe, 64 when the launch is a stream of the (four times smaller) weights */
  if (n > 128) return launch_gemm<256, 1, 128, false, true>(nullptr, x, a, facts.sm_count);
  return launch_gemm<64, 1, 128, false, true>(nullptr, x, a, facts.sm_count);
}

static wst_status_t qkv_rope_append_common(
    const char *name, const void *w, const void *qw, const void *si, const void *sb, const void *x, const void *bias, void *q_out, void *k_cache, void *v_cache,
    const void *cos_tab, const void *sin_tab, const void *seq_pos0, int32_t in_f, int32_t n_seq,
    int32_t n, int32_t n_q, int32_t n_kv, int32_t head_dim, int32_t max_seq, int32_t table_len,
    const void *q_norm_w, const void *k_norm_w, float eps) {
  WST_CHECK_ARG((w || (qw && si && sb)) && x && q_out && k_cache && v_cache && cos_tab && sin_tab &&
                    seq_pos0,
                "wst_b200_qkv_rope_append_batch: null pointer");
  WST_CHECK_ARG(in_f > 0 && n_seq > 0 && n > 0 && n_q > 0 && n_kv > 0 && max_seq > 0 &&
                    table_len > 0,
                "wst_b200_qkv_rope_append_batch: non-positive shape");
  WST_CHECK_ARG(head_dim == 64 || head_dim == 128,
                "wst_b200_qkv_rope_append_batch: head_dim must be 64 or 128");
  WST_CHECK_ARG(in_f % (qw ? 32 : 8) == 0,
                "wst_b200_qkv_rope_append_batch: in_features must be a multiple of 8 (32 for int4 weights)");
  const long long tokens = static_cast<long long>(n_seq) * n;
  const long long out_f = static_cast<long long>(n_q + 2 * n_kv) * head_dim;
  WST_CHECK_ARG(tokens <= 0x7fffffffLL && out_f <= 0x7fffffffLL,
                "wst_b200_qkv_rope_append_batch: shape overflows");
  for (const void *ptr : {w ? w : qw, x, static_cast<const void *>(q_out), static_cast<const void *>(k_cache),
                          static_cast<const void *>(v_cache), cos_tab, sin_tab})
    WST_CHECK_ARG((reinterpret_cast<uintptr_t>(ptr) & 15) == 0,
                  "wst_b200_qkv_rope_append_batch: buffers must be 16-byte aligned");
  WST_CHECK_ARG((!bias || (reinterpret_cast<uintptr_t>(bias) & 3) == 0) &&
                    (!q_norm_w || (reinterpret_cast<uintptr_t>(q_norm_w) & 3) == 0) &&
                    (!k_norm_w || (reinterpret_cast<uintptr_t>(k_norm_w) & 3) == 0),
                "wst_b200_qkv_rope_append_batch: bias and gains must be 4-byte aligned");
  DeviceFacts facts;
  if (!device_facts(&facts)) return WST_ERR_CUDA;
  if (facts.cc_major < 10)
    return fail(WST_ERR_UNSUPPORTED_ARCH, "%s: this library is built for sm_100a only", name);
  unsigned int *err_word = device_error_word();
  if (!err_word) return WST_ERR_CUDA;
  GemmArgs a{};
  a.bias = static_cast<const __half *>(bias);
  a.in_f = in_f;
  a.out_f = static_cast<int>(out_f);
  a.n = static_cast<int>(tokens);
  a.err_word = err_word;
  a.q_out = static_cast<__half *>(q_out);
  a.k_cache = static_cast<__half *>(k_cache);
  a.v_cache = static_cast<__half *>(v_cache);
  a.cos_tab = static_cast<const float *>(cos_tab);
  a.sin_tab = static_cast<const float *>(sin_tab);
  a.q_gain = static_cast<const __half *>(q_norm_w);
  a.k_gain = static_cast<const __half *>(k_norm_w);
  a.seq_pos0 = static_cast<const int32_t *>(seq_pos0);
  a.n_q = n_q;
  a.n_kv = n_kv;
  a.hd = head_dim;
  a.n_per_seq = n;
  a.max_seq = max_seq;
  a.table_len = table_len;
  a.eps = eps;
  if (qw) {
    a.qw = static_cast<const uint4 *>(qw);
    a.si = static_cast<const uint8_t *>(si);
    a.sb = static_cast<const __half2 *>(sb);
    return launch_gemm<256, 1, 128, true, true>(nullptr, x, a, facts.sm_count);
  }
  return launch_gemm<256, 1, 128, true>(w, x, a, facts.sm_count);
}

extern "C" wst_status_t wst_b200_qkv_rope_append_batch(
    const void *w, const void *x, const void *bias, void *q_out, void *k_cache, void *v_cache,
    const void *cos_tab, const void *sin_tab, const void *seq_pos0, int32_t in_f, int32_t n_seq,
    int32_t n, int32_t n_q, int32_t n_kv, int32_t head_dim, int32_t max_seq, int32_t table_len,
    const void *q_norm_w, const void *k_norm_w, float eps) {
  return qkv_rope_append_common("wst_b200_qkv_rope_append_batch", w, nullptr, nullptr, nullptr, x, bias,
                                q_out, k_cache, v_cache, cos_tab, sin_tab, seq_pos0, in_f, n_seq, n, n_q,
                                n_kv, head_dim, max_seq, table_len, q_norm_w, k_norm_w, eps);
}

/* The same with the qkv weights in the hierarchical int4 format of wst_gemm_int4_hier. */
extern "C" wst_status_t wst_b200_qkv_int4_rope_append_batch(
    const void *qw, const void *si, const void *sb, const void *x, const void *bias, void *q_out,
    void *k_cache, void *v_cache, const void *cos_tab, const void *sin_tab, const void *seq_pos0,
    int32_t in_f, int32_t n_seq, int32_t n, int32_t n_q, int32_t n_kv, int32_t head_dim,
    int32_t max_seq, int32_t table_len, const void *q_norm_w, const void *k_norm_w, float eps) {
  WST_CHECK_ARG(qw && si && sb, "wst_b200_qkv_int4_rope_append_batch: null pointer");
  return qkv_rope_append_common("wst_b200_qkv_int4_rope_append_batch", nullptr, qw, si, sb, x, bias,
                                q_out, k_cache, v_cache, cos_tab, sin_tab, seq_pos0, in_f, n_seq, n, n_q,
                                n_kv, head_dim, max_seq, table_len, q_norm_w, k_norm_w, eps);
}

/* The engine sizes its prefill chunks by this (cuda/chunk_gemm.cu:367 returns 16, the
 * widest pass of its kernels; src/chunk.rs:20, engine.rs:682-693).  A pass here takes
 * any width; 512 tokens is the chunk the prefill kernels of this library are tuned on. */
extern "C" int32_t wst_chunk_max_tokens(void) { return 512; }
