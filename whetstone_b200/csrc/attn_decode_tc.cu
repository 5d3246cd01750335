/* Decode attention over the 8-bit (e4m3) cache on the tensor-memory path.
 *
 * The row-block kernel (attn_rows.cu) spends 32 mma.sync per 64-row tile and warp on
 * the seven valid query rows of a 16-row fragment and converts every tile once per
 * consumer warp; over the e4m3 cache -- half the bytes of the fp16 cache -- that work, not
 * HBM, is its bound.  Here a tile is 128 keys, it is converted once per block, and both
 * contractions are tcgen05.mma with M = 128.
 *
 * One CTA per (KV head, slice of the sequence); a slice owns tiles split, split + n, ...
 *
 *   TMA warp        raw e4m3 tiles [128 keys][128 bytes] of K and of V into a ring of four
 *                   16 KB slots; the first four are requested before the launch ahead in
 *                   the stream has finished (see the kernel)
 *   4 + 4           e4m3 -> fp16 (exact) from the raw ring into two K and three V slots of
 *     converter     32 KB laid out as K-major UMMA operands ([2 halves][128 rows][128 B],
 *     warps         128-byte swizzle): four warps take the K tiles, four the V tiles, which
 *                   they store TRANSPOSED ([head_dim][keys], through ldmatrix and
 *                   stmatrix.trans) with the rows past the live data as zeros.
 *   MMA warp        S(j) = Q K(j)^T (Q in tensor memory) into one of two score buffers,
 *                   O += P(j-1) V(j-1)
 *   4 softmax       The GQA group's rows (at most 16) are REPLICATED in the four lane
 *     warps         quadrants of the 128-row Q tile: warp w reads the scores of its own
 *                   quadrant and handles only keys 32w .. 32w+31 of every tile, as an
 *                   independent online-softmax stream with its own maximum and sum; its
 *                   rows of P are zero outside those keys, so its rows of O accumulate
 *                   exactly its keys.  The four streams of a row are merged at the end
 *                   like the slices of a sequence.  (A thread owns a row of tensor
 *                   memory, and a warp can reach only its quadrant: without the replicas
 *                   one warp would take the exponentials of all 128 keys of the seven
 *                   rows and the other three would idle.)
 *
 * What was measured on the way (SM clocks per tile and slice, 131072 rows, 28 tiles):
 *   - Plain loads into registers instead of the raw ring: sixteen loads per thread in
 *     flight share six scoreboards, so every wait for a tile also waited for the newest
 *     request: 3400.
 *   - TMA ring, eight warps converting K and V in turn, cvt only: 2400.  The same with
 *     integer operations only: 2400.  Either way one pipe of each scheduler (the one cvt
 *     and ex2 share, or the integer one) carried about 1300 clocks of work per tile, and
 *     every warp paid its waits, loads and stores twice per tile.
 *   - Eight lanes of a 16-byte store along one fp16 row collide in pairs (the row's halves
 *     lie 16 KB apart): eight lanes down eight rows do not.  2330.
 *   - Separate K and V quartets: 1930 (with cvt for half of the pairs and integer
 *     operations for the other half: 1900 -> 1750 at 131072 rows).
 * A tile moves 192 KB through shared memory (32 in, 32 + 64 through the converters, 64 read
 * by the tensor core), 1536 clocks at 128 bytes per clock, and about 900 clocks through
 * each of the two pipes named above; HBM delivers its 32 KB in about 1300.
 *
 * Each slice leaves one (acc, m, l) row per query head in the scratch layout of the
 * row-block kernel; attn_merge_kernel finishes.  All waits are bounded (codes 0x7xx).
 */

#include "attn_rows.cuh"
#include "tensor_map.cuh"
#include "wst_common.cuh"
#include "wst_ptx.cuh"

namespace wst {
namespace {

using namespace ptx;

constexpr float kLog2eTc = 1.4426950408889634f;

struct TcCfg {
  static constexpr int HD = 128, BN = 128;
  static constexpr int HALF_BYTES = BN * 128;          /* 64 columns of 128 rows */
  static constexpr int SLOT = 2 * HALF_BYTES;          /* one K or V tile as fp16: 32 KB */
  static constexpr int NK = 2, NV = 3;                 /* converted slots: a K tile is read once, by S(j); a V
                                                          tile waits for the softmax of its tile as well */
  static constexpr int NCV = NK + NV;
  static constexpr int RAW_SLOT = BN * HD;             /* one K or V tile as e4m3: 16 KB */
  static constexpr int NRAW = 4;
  static constexpr int CONV_WARPS = 8;
  static constexpr int OFF_CONV = 0;
  static constexpr int OFF_RAW = OFF_CONV + NCV * SLOT;
  static constexpr int OFF_BAR = OFF_RAW + NRAW * RAW_SLOT;
  static constexpr int NBAR = 2 * NCV + 2 * NRAW + 2 + 2 + 1 + 1 + 1 + 1;
  static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 16 + 1024;
  static constexpr int THREADS = 32 * (6 + CONV_WARPS); /* 4 softmax warps, MMA warp, TMA warp, converters */
  static constexpr int COL_S = 0;     /* two score buffers of 128 columns */
  static constexpr int COL_O = 256;
  static constexpr int COL_P = 384;   /* fp16 P: 64 columns */
  static constexpr int COL_Q = 448;   /* fp16 Q: 64 columns */
  static constexpr int TMEM_COLS = 512;
  static constexpr int DR = HD + 4;   /* a partial row: acc | m | l | pad pad */
};
static_assert(TcCfg::SMEM_BYTES <= 232448, "shared memory of one CTA");

struct TcArgs {
  const float *q;        /* [n_q][128] fp32 */
  const uint8_t *k8, *v8; /* [n_kv][max_seq][128] e4m3 (the tensor maps describe the same bytes) */
  float *scratch;        /* [n_kv][n_splits][gqa][132] */
  const int32_t *pos;    /* device cursor */
  int n_q, n_kv, gqa, max_seq, n_splits;
  float qscale;          /* scale * log2(e) * k_scale */
  float out_scale;       /* v_scale */
  int early;             /* request the first tiles before the launch ahead has finished */
  unsigned int *err_word;
};

__device__ __forceinline__ float max3f(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

/* Four e4m3 bytes -> four fp16 values (exact: every e4m3 number is an fp16 number), the
 * low pair by cvt and the high pair by integer operations, so that the work is spread over
 * two pipes.  cvt.f16x2.e4m3x2 issues at a quarter of the full rate, on the pipe that also
 * serves the exponentials of the softmax warps; four integer operations per pair at half
 * rate cost as much on the integer pipe; with eight converter warps either pipe alone was
 * the bound of the kernel.  The integer route: a byte s.eeee.mmm in the top half of a 16-bit
 * lane, shifted right by one under its sign, is the fp16 pattern s.0eeee.mmm0000000, whose
 * exponent field counts from 15 where e4m3 counts from 7 (subnormals land on fp16
 * subnormals): 2^-8 times the value, which one half2 multiplication puts right.  (The bytes
 * 0x7f / 0xff, NaN in e4m3, read as +-480 on this route.) */
__device__ __forceinline__ void e4m3x4_to_f16(uint32_t in, uint32_t &lo, uint32_t &hi) {
  asm("{\n\t.reg .b16 a, b;\n\t"
      "mov.b32 {a, b}, %1;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, a;\n\t}"
      : "=r"(lo)
      : "r"(in));
  const uint32_t x1 = __byte_perm(in, 0u, 0x3424u); /* 00 b2 00 b3 */
  const uint32_t small = ((x1 >> 1) & 0x3F803F80u) | (x1 & 0x80008000u);
  asm("mul.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(small), "r"(0x5C005C00u)); /* times 256 */
}

__global__ void __launch_bounds__(TcCfg::THREADS, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                      const TcArgs a) {
  using C = TcCfg;
  constexpr int HD = C::HD, BN = C::BN, HALF_BYTES = C::HALF_BYTES, NCV = C::NCV, NRAW = C::NRAW;
  constexpr int NK = C::NK, NV = C::NV;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::OFF_BAR;
  auto bar = [bar0](int i) { return bar0 + 8u * i; };
  constexpr int C_FULL = 0, C_EMPTY = NCV, RAW_FULL = 2 * NCV, RAW_EMPTY = RAW_FULL + NRAW;
  constexpr int S_FULL = RAW_EMPTY + NRAW, S_FREE = S_FULL + 2, P_READY = S_FREE + 2;
  constexpr int PV_DONE = P_READY + 1, O_DONE = PV_DONE + 1, Q_READY = O_DONE + 1;
  /* item i = the K (even) or V (odd) tile of the slice's tile i / 2: its converted slot and
   * how many times that slot has been used before */
  auto conv_slot = [](int i) { return (i & 1) ? NK + (i >> 1) % NV : (i >> 1) % NK; };
  auto conv_use = [](int i) { return (i & 1) ? (i >> 1) / NV : (i >> 1) / NK; };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + C::OFF_BAR + C::NBAR * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, ns = a.n_splits;

  /* The launch right before this one in the stream -- still running under programmatic
   * dependent launch -- can only be writing the newest cache row; every older row was
   * written by launches that finished long ago.  So the slice's first tiles are requested
   * first of all, by the thread that sets up the raw ring's barriers, while the rest of the
   * block is still being set up and before the dependency resolves (without the cursor,
   * which is not known yet: tiles past the live rows are requested and never read).  The
   * newest row is read again with plain loads after the wait, by the converter threads that
   * own its pieces. */
  grid_launch_dependents();
  auto request = [&](int i) {
    mbar_arrive_expect_tx(bar(RAW_FULL + i % NRAW), C::RAW_SLOT);
    tma_load_3d(sbase + C::OFF_RAW + (i % NRAW) * C::RAW_SLOT, (i & 1) ? &vmap : &kmap, bar(RAW_FULL + i % NRAW), 0,
                (split + (i >> 1) * ns) * BN, kvh);
  };
  int n_early = 0;
  if (warp == 5 && lane == 0) {
    for (int i = 0; i < NRAW; ++i) {
      mbar_init(bar(RAW_FULL + i), 1);
      mbar_init(bar(RAW_EMPTY + i), C::CONV_WARPS / 2);
    }
    mbar_init_fence();
    if (a.early)
      while (n_early < NRAW && (split + (n_early >> 1) * ns) * BN < a.max_seq) request(n_early++);
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < NCV; ++i) {
      mbar_init(bar(C_FULL + i), C::CONV_WARPS / 2);
      mbar_init(bar(C_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(S_FREE + i), 128);
    }
    mbar_init(bar(P_READY), 128);
    mbar_init(bar(PV_DONE), 1);
    mbar_init(bar(O_DONE), 1);
    mbar_init(bar(Q_READY), 128);
    mbar_init_fence();
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
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

  int pos0 = *a.pos;
  pos0 = pos0 < 0 ? 0 : pos0;
  const int kv_end = pos0 + 1 < a.max_seq ? pos0 + 1 : a.max_seq; /* rows [0, kv_end) are live */
  const int n_tiles = (kv_end + BN - 1) / BN;
  const int T = split < n_tiles ? (n_tiles - split + ns - 1) / ns : 0; /* tiles split, split + ns, ... */

  if (warp == 5) {
    /* ------- TMA producer: item i is the K (even) or V (odd) tile of the slice's tile i / 2 */
    if (lane == 0) {
      for (int i = n_early; i < 2 * T; ++i) {
        if (i >= NRAW && !mbar_wait(bar(RAW_EMPTY + i % NRAW), ((i / NRAW) - 1) & 1, a.err_word, 0x701u)) break;
        request(i);
      }
      /* tiles requested early that turned out to lie past the live rows: let them land
       * before the block may leave */
      for (int i = 2 * T; i < n_early; ++i) mbar_wait(bar(RAW_FULL + i), 0, a.err_word, 0x704u);
    }
  } else if (warp >= 6) {
    /* ------- converters.  Warps 6..9 convert the K tiles and warps 10..13 the V tiles, a
     * whole tile per warp quartet: one round of waits, loads and stores per tile and warp,
     * and the two tiles of a step are converted side by side.  A K thread takes eight
     * 16-byte pieces; eight neighbouring lanes take the same piece of eight consecutive
     * rows: under the 128-byte swizzle those are eight different bank groups in the raw tile
     * and in the fp16 tile alike, so every 16-byte load and store of a warp is four
     * wavefronts. */
    const bool v_side = warp >= 10;
    const int cw = (warp - 6) & 3;
    const int row0 = 8 * cw + (lane & 7);  /* K piece n: row row0 + 32 (n / 2), 16-byte column lane / 8 + 4 (n % 2) */
    const int col = lane >> 3;
    const int ch = 2 * col; /* it becomes fp16 chunks ch and ch + 1 of half n % 2 */
    /* V items are stored TRANSPOSED, [head_dim rows][keys], so that P V reads a K-major
     * operand like Q K^T does.  ldmatrix hands thread t four bytes of key t / 4 (head_dim
     * 4 (t % 4) .. + 3 of a 16-byte piece); the two fp16 pairs they become go into two
     * 8 x 8 matrices that stmatrix.trans writes as rows of eight keys.  Threads with
     * t % 4 >= 2 swap their two pairs, so that the eight rows of a matrix are eight
     * different head_dim values modulo 8: eight different bank groups under the swizzle. */
    const int vm = lane >> 3, vi = lane & 7;           /* the lane addresses row vi of matrix vm */
    const bool swap_pairs = (lane & 2) != 0;
    const int hd_x = 4 * (vi >> 1) + 2 * (vi >> 2) + (vi & 1);       /* row vi of the first matrix */
    const int hd_y = 4 * (vi >> 1) + 2 * (1 - (vi >> 2)) + (vi & 1); /* and of the second */
    for (int j = 0; j < T; ++j) {
      const int i = 2 * j + (v_side ? 1 : 0);
      const int st = i % NRAW, cs = conv_slot(i), use = conv_use(i);
      if (!mbar_wait(bar(RAW_FULL + st), (i / NRAW) & 1, a.err_word, 0x702u)) break;
      const uint32_t src = sbase + C::OFF_RAW + st * C::RAW_SLOT;
      const uint32_t dst = sbase + C::OFF_CONV + cs * C::SLOT;
      if (v_side) {
        const int live = kv_end - (split + j * ns) * BN;
        uint32_t w[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { /* key block 4 cw + n / 2, 64-byte group n % 2 */
          const int kb = 4 * cw + (n >> 1);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(w[n][0]), "=r"(w[n][1]), "=r"(w[n][2]), "=r"(w[n][3])
                       : "r"(src + swz128(8 * kb + vi, 4 * (n & 1) + vm)));
          if (live <= BN && 8 * kb + (lane >> 2) == live - 1) { /* the newest row: the copy in shared memory may be stale */
            const uint8_t *rowp = a.v8 + (static_cast<long long>(kvh) * a.max_seq + kv_end - 1) * HD +
                                  64 * (n & 1) + 4 * (lane & 3);
#pragma unroll
            for (int m = 0; m < 4; ++m) w[n][m] = *reinterpret_cast<const uint32_t *>(rowp + 16 * m);
          }
          /* dead rows may hold anything, and 0 * NaN is NaN */
          if (8 * kb + (lane >> 2) >= live) w[n][0] = w[n][1] = w[n][2] = w[n][3] = 0u;
        }
        if (use > 0 && !mbar_wait(bar(C_EMPTY + cs), (use - 1) & 1, a.err_word, 0x703u)) break;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int kb = 4 * cw + (n >> 1);
          uint32_t x[4], y[4];
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            uint32_t lo, hi;
            e4m3x4_to_f16(w[n][m], lo, hi);
            x[m] = swap_pairs ? hi : lo;
            y[m] = swap_pairs ? lo : hi;
          }
          const uint32_t at = dst + (kb >> 3) * HALF_BYTES;
          const int hd0 = 16 * (4 * (n & 1) + vm);
          asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(
                           at + swz128(hd0 + hd_x, kb & 7)),
                       "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]) : "memory");
          asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(
                           at + swz128(hd0 + hd_y, kb & 7)),
                       "r"(y[0]), "r"(y[1]), "r"(y[2]), "r"(y[3]) : "memory");
        }
      } else {
        uint4 r[8];
#pragma unroll
        for (int n = 0; n < 8; ++n)
          asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(r[n].x), "=r"(r[n].y), "=r"(r[n].z), "=r"(r[n].w)
                       : "r"(src + swz128(row0 + 32 * (n >> 1), col + 4 * (n & 1))));
        const int newest = kv_end - 1 - (split + j * ns) * BN; /* the newest row, if it is in this tile */
        if (newest < BN) {
#pragma unroll
          for (int n = 0; n < 8; ++n)
            if (row0 + 32 * (n >> 1) == newest) /* the copy in shared memory may be stale */
              r[n] = *reinterpret_cast<const uint4 *>(
                  a.k8 + (static_cast<long long>(kvh) * a.max_seq + kv_end - 1) * HD + 16 * (col + 4 * (n & 1)));
        }
        if (use > 0 && !mbar_wait(bar(C_EMPTY + cs), (use - 1) & 1, a.err_word, 0x703u)) break;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int row = row0 + 32 * (n >> 1);
          const uint32_t at = dst + (n & 1) * HALF_BYTES;
          uint32_t h[8];
          e4m3x4_to_f16(r[n].x, h[0], h[1]);
          e4m3x4_to_f16(r[n].y, h[2], h[3]);
          e4m3x4_to_f16(r[n].z, h[4], h[5]);
          e4m3x4_to_f16(r[n].w, h[6], h[7]);
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at + swz128(row, ch)),
                       "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at + swz128(row, ch + 1)),
                       "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
        }
      }
      fence_async_smem(); /* the tensor core reads these tiles through the async proxy */
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(C_FULL + cs));
        mbar_arrive(bar(RAW_EMPTY + st));
      }
    }
  } else if (warp == 4) {
    /* -------------------------------------------------------- MMA issuer */
    constexpr uint32_t idesc_qk = umma_idesc(128, BN, 0);
    constexpr uint32_t idesc_pv = umma_idesc(128, HD, 0); /* V arrives transposed: K-major */
    bool ok = mbar_wait(bar(Q_READY), 0, a.err_word, 0x710u);
    tc_fence_after_sync();
    auto issue_pv = [&](int j) -> bool { /* O += P(j) V(j) */
      if (!mbar_wait(bar(P_READY), j & 1, a.err_word, 0x711u)) return false;
      tc_fence_after_sync();
      const int item = 2 * j + 1;
      if (!mbar_wait(bar(C_FULL + conv_slot(item)), conv_use(item) & 1, a.err_word, 0x714u)) return false;
      tc_fence_after_sync();
      const uint32_t v_lo = umma_desc_lo(sbase + C::OFF_CONV + conv_slot(item) * C::SLOT, 16);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4;
          umma_ts_f16_lohi(tmem + C::COL_O, tmem + C::COL_P + kk * 8, v_lo + off, kDescHi, idesc_pv,
                           (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bar(PV_DONE));
        umma_commit(bar(C_EMPTY + conv_slot(item)));
        if (j == T - 1) umma_commit(bar(O_DONE));
      }
      __syncwarp();
      return true;
    };
    for (int j = 0; ok && j < T; ++j) {
      const int item = 2 * j;
      if (!mbar_wait(bar(C_FULL + conv_slot(item)), conv_use(item) & 1, a.err_word, 0x712u)) { ok = false; break; }
      if (j >= 2 && !mbar_wait(bar(S_FREE + (j & 1)), ((j >> 1) - 1) & 1, a.err_word, 0x713u)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t k_lo = umma_desc_lo(sbase + C::OFF_CONV + conv_slot(item) * C::SLOT, 16);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          umma_ts_f16_lohi(tmem + C::COL_S + (j & 1) * BN, tmem + C::COL_Q + ks * 8, k_lo + off, kDescHi,
                           idesc_qk, ks > 0);
        }
        umma_commit(bar(S_FULL + (j & 1)));
        umma_commit(bar(C_EMPTY + conv_slot(item)));
      }
      __syncwarp();
      if (j >= 1 && !issue_pv(j - 1)) { ok = false; break; }
    }
    if (ok && T > 0) issue_pv(T - 1);
  } else {
    /* ----- softmax stream w: rows of quadrant w, keys 32w .. 32w+31 of every tile */
    const int w = warp;
    const uint32_t lane_base = static_cast<uint32_t>(w * 32) << 16;
    const bool valid = lane < a.gqa;

    /* q row `lane` of the group, replicated in every quadrant: fp16 * scale, two per column */
    {
      const float *src = a.q + static_cast<long long>(kvh * a.gqa + (valid ? lane : 0)) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD / 2; c0 += 32) {
        uint32_t qp[32];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float4 f = __ldg(reinterpret_cast<const float4 *>(src + 2 * (c0 + e)));
          qp[e] = valid ? pack_half2(f.x * a.qscale, f.y * a.qscale) : 0u;
          qp[e + 1] = valid ? pack_half2(f.z * a.qscale, f.w * a.qscale) : 0u;
        }
        tmem_st_32x32(tmem + lane_base + C::COL_Q + c0, qp);
      }
      /* this quadrant's rows of P: zero outside the stream's own keys, for good */
      uint32_t z[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) z[i] = 0u;
      tmem_st_32x32(tmem + lane_base + C::COL_P, z);
      tmem_st_32x32(tmem + lane_base + C::COL_P + 32, z);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(Q_READY));
    }

    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < T; ++j) {
      if (!mbar_wait(bar(S_FULL + (j & 1)), (j >> 1) & 1, a.err_word, 0x720u)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t sv[32];
      tmem_ld_32x32(tmem + lane_base + C::COL_S + (j & 1) * BN + 32 * w, sv);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(S_FREE + (j & 1)));
      const int key0 = (split + j * ns) * BN + 32 * w;
      if (key0 + 32 > kv_end) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (key0 + c >= kv_end) sv[c] = 0xff800000u; /* -inf */
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; c += 2) mx = max3f(mx, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
      /* the offset moves only when some row of the warp grows by more than 2^8 */
      const bool grow = mx > m_run + 8.f || (m_run == -INFINITY && mx > -INFINITY);
      const bool warp_grow = __any_sync(0xffffffffu, grow);
      const float m_new = warp_grow ? fmaxf(m_run, mx) : m_run;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      float psum = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float p0 = ex2(__uint_as_float(sv[c]) - m_use);
        const float p1 = ex2(__uint_as_float(sv[c + 1]) - m_use);
        psum += p0 + p1;
        pk[c >> 1] = pack_half2(p0, p1);
      }
      /* P(j-1) has been read and O is quiescent once PV(j-1) is done */
      if (j > 0 && !mbar_wait(bar(PV_DONE), (j - 1) & 1, a.err_word, 0x721u)) { ok = false; break; }
      tc_fence_after_sync();
      tmem_st_32x16(tmem + lane_base + C::COL_P + 16 * w, pk);
      if (warp_grow && j > 0) {
        const float factor = ex2(m_run - m_use); /* 1 for rows that did not move, 0 from -inf */
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + lane_base + C::COL_O + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
          tmem_st_32x32(tmem + lane_base + C::COL_O + c0, v);
        }
        l_run *= factor;
      }
      m_run = m_new;
      l_run += psum;
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(P_READY));
    }

    /* the four streams of a row -> one (acc, m, l) row of the slice, through shared memory
     * (the operand slots are idle by now) */
    float *dump = reinterpret_cast<float *>(smem + C::OFF_CONV);
    if (ok && T > 0) ok = mbar_wait(bar(O_DONE), 0, a.err_word, 0x722u);
    tc_fence_after_sync();
    ok = __all_sync(0xffffffffu, ok); /* the loads below are collective */
    {
      float *row = dump + static_cast<size_t>(w * 16 + (valid ? lane : 0)) * C::DR;
      if (ok && T > 0) {
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + lane_base + C::COL_O + c0, v);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4 *>(row + c0 + e) =
                  make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                              __uint_as_float(v[e + 3]));
          }
        }
        if (valid) {
          row[HD] = m_run;
          row[HD + 1] = l_run;
        }
      } else if (valid) {
        for (int e = 0; e < HD; ++e) row[e] = 0.f;
        row[HD] = -INFINITY;
        row[HD + 1] = 0.f;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    for (int idx = threadIdx.x; idx < a.gqa * (HD / 4); idx += 128) {
      const int r = idx / (HD / 4), c4 = idx % (HD / 4);
      float mw[4], M = -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        mw[k] = dump[static_cast<size_t>(k * 16 + r) * C::DR + HD];
        M = fmaxf(M, mw[k]);
      }
      const float m_use = M == -INFINITY ? 0.f : M;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float den = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float wgt = ex2(mw[k] - m_use);
        const float *cell = dump + static_cast<size_t>(k * 16 + r) * C::DR;
        const float4 v = *reinterpret_cast<const float4 *>(cell + 4 * c4);
        acc.x = fmaf(wgt, v.x, acc.x);
        acc.y = fmaf(wgt, v.y, acc.y);
        acc.z = fmaf(wgt, v.z, acc.z);
        acc.w = fmaf(wgt, v.w, acc.w);
        den = fmaf(wgt, cell[HD + 1], den);
      }
      acc.x *= a.out_scale; acc.y *= a.out_scale; acc.z *= a.out_scale; acc.w *= a.out_scale;
      float *dst = a.scratch + ((static_cast<long long>(kvh) * ns + split) * a.gqa + r) * C::DR;
      *reinterpret_cast<float4 *>(dst + 4 * c4) = acc;
      if (c4 == 0) *reinterpret_cast<float2 *>(dst + HD) = make_float2(M, den);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

}  // namespace

/* Decode over the e4m3 cache on the tensor-memory path (see the top of this file);
 * declared in attn_rows.cuh. */
wst_status_t launch_decode_fp8_tc(const RowsLaunch &L) {
  using C = TcCfg;
  DeviceFacts facts;
  if (!device_facts(&facts)) return WST_ERR_CUDA;
  const int gqa = L.n_q / L.n_kv;
  /* Slices: one CTA per SM when a slice has many tiles; with few, a tenth of the SMs is left
   * to the merge kernel and to the first blocks of the next launch, which then request their
   * tiles and set themselves up while this launch streams (33 against 37 slices per KV head
   * at 32768 rows and 4 KV heads: 14.4 against 15.2 us per layer; at 131072 rows: 40.2
   * against 37.2). */
  const int tiles = (L.max_seq + C::BN - 1) / C::BN;
  int splits = facts.sm_count / L.n_kv;
  if (splits > 1 && tiles <= 14 * splits) {
    const int fewer = (facts.sm_count - facts.sm_count / 10) / L.n_kv;
    if (fewer >= 1) splits = fewer;
  }
  if (rows_tuning().decode_splits > 0) splits = rows_tuning().decode_splits;
  if (splits > tiles) splits = tiles;
  if (splits > kRowsMaxSplits) splits = kRowsMaxSplits;
  while (splits > 1 && rows_scratch_floats(L.n_kv * gqa, splits, L.hd) > L.scratch_floats) --splits;
  if (splits < 1 || !L.scratch || rows_scratch_floats(L.n_kv * gqa, splits, L.hd) > L.scratch_floats)
    return fail(WST_ERR_INVALID_ARG, "%s: the split scratch is too small", L.name);

  TcArgs a{};
  a.q = L.q;
  a.k8 = reinterpret_cast<const uint8_t *>(L.k);
  a.v8 = reinterpret_cast<const uint8_t *>(L.v);
  a.early = decode_overlap_allowed() ? 1 : 0;
  a.scratch = L.scratch;
  a.pos = L.pos0_dev;
  a.n_q = L.n_q;
  a.n_kv = L.n_kv;
  a.gqa = gqa;
  a.max_seq = L.max_seq;
  a.n_splits = splits;
  a.qscale = L.scale * kLog2eTc * L.k_scale;
  a.out_scale = L.v_scale;
  a.err_word = device_error_word();
  if (!a.err_word) return WST_ERR_CUDA;

  CUtensorMap kmap, vmap;
  KvMapKey key{};
  key.rank = 3;
  key.d0 = static_cast<uint64_t>(L.hd / 2); /* 128 e4m3 bytes described as 64 two-byte elements */
  key.d1 = static_cast<uint64_t>(L.max_seq);
  key.d2 = static_cast<uint64_t>(L.n_kv);
  key.d3 = 1;
  key.b1 = C::BN;
  key.base = L.k;
  wst_status_t st = cached_kv_tensor_map(&kmap, key);
  if (st != WST_OK) return st;
  key.base = L.v;
  st = cached_kv_tensor_map(&vmap, key);
  if (st != WST_OK) return st;

  static thread_local int configured_dev = -1;
  int dev = 0;
  WST_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    WST_CUDA(cudaFuncSetAttribute(attn_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  C::SMEM_BYTES));
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(splits), static_cast<unsigned>(L.n_kv));
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = current_stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, attn_decode_tc_kernel, kmap, vmap, a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("wst_b200_attn_decode_fp8 (launch)", e);

  SplitMerge m;
  m.scratch = L.scratch;
  m.out = L.out;
  m.n_tok = 1;
  m.n_q = L.n_q;
  m.n_kv = L.n_kv;
  m.hd = L.hd;
  m.n_splits = splits;
  m.n_rowblk = 1;
  m.tpb = 1;
  m.rows_cap = gqa;
  m.n_units = L.n_kv;
  m.name = L.name;
  return launch_split_merge(m);
}

}  // namespace wst
