/* Kernel sets 2 and 4: split-KV attention of a small block of query rows against
 * a long stretch of one KV head's cache -- batch-1 decode (rows = the heads of
 * one GQA group), small chunks / speculative verification (rows = heads x draft
 * tokens) and the ragged, paged form of the latter.
 *
 * The path is HBM-bound: every K and V byte of the visible prefix is needed
 * exactly once.  So the design is built around that one stream:
 *
 *   - One CTA owns (sequence, KV head, row block, sequence slice) and serves ALL
 *     query rows that share the KV head, so the cache is read from DRAM once, not
 *     once per query head.
 *   - A dedicated producer warp streams 64-position K and V tiles through a
 *     multi-stage shared-memory ring with TMA (cp.async.bulk.tensor, 128-byte
 *     swizzle) and mbarriers; ~128 KB are in flight per SM.
 *   - Consumer warps each take 16 positions of a tile.  QK^T and PV are
 *     mma.sync m16n8k16 (fp16 in, fp32 accumulate) because at ~7 query heads per
 *     KV byte the CUDA cores could not keep up with HBM; the online softmax
 *     state (running max, denominator) is fp32 and reduced with warp shuffles.
 *   - The sequence is split over CTAs so that all SMs stream (slice s takes
 *     tiles s, s + n, s + 2n, ...); each slice writes an unnormalised
 *     (m, l, acc) row per query row, and a small second kernel -- launched with
 *     programmatic stream serialization, so already resident when the last
 *     slice ends -- merges them with every load in flight at once.  Nothing
 *     spins and no counters persist between launches.
 *
 * Semantics follow cuda/attention.cu:57-193 (decode) and cuda/chunk_ops.cu:187-264
 * (chunk: query j sees rows [0, pos0+j]) of the engine.
 */

#include <atomic>

#include "attn_rows.cuh"
#include "tensor_map.cuh"
#include "wst_ptx.cuh"


namespace wst {
namespace {

using namespace ptx;

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct RowsArgs {
  const float *q;
  long long q_tok_stride;
  const __half *k, *v; /* the cache itself, next to the tensor maps: the newest row is patched by plain loads */
  const int32_t *page_table;
  int max_pages, n_pool_pages;
  const int32_t *pos0_dev;
  int pos0_bias, clamp_nonneg, pos0_val;
  const int32_t *cu_tokens;
  int n_tok, tok_seq_stride;
  int n_q, n_kv, gqa, max_seq;
  float qscale; /* scale * log2(e): scores live in log2 units */
  float *scratch;
  unsigned int *err_word;
  void *out;
  int partial_out;
  int n_splits, n_rowblk, tpb, rows_cap;
  int nstage;      /* ring stages in use, 2 .. Cfg::NSTAGE */
  int early_depth; /* 0: nothing is requested before the grid dependency resolves; else the
                    * number of tiles kept in flight ahead of it */
  int via_scratch; /* a single slice still writes its row to scratch: the merge kernel
                    * follows (it carries the cross-GPU exchange) */
  float out_scale; /* fp8 cache: the values' scale, applied to the accumulated rows */
};

/* KV8: the cache holds e4m3 bytes.  A stage is then the raw K and V tiles, [BN rows][HD
 * bytes] each, and every consumer warp keeps a private fp16 copy of its own 16 positions
 * of the tile in flight (PRIV_BYTES), converted from the stage right before use. */
template <int HD, int MT, int RG, bool KV8 = false>
struct Cfg {
  static constexpr int BN = kRowsTile;
  static constexpr int NH = HD / 64;             /* 64-column (128-byte) halves */
  static constexpr int ROWS = 16 * MT * RG;
  static constexpr int CWARPS = 4 * RG;
  static constexpr int CTHREADS = CWARPS * 32;
  static constexpr int THREADS = CTHREADS + 32;
  static constexpr int HALF_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = KV8 ? 2 * BN * HD : 2 * NH * HALF_BYTES;
  static constexpr int PRIV_WARP_BYTES = 2 * NH * 16 * 128; /* K then V, [NH][16 rows][128 B] */
  static constexpr int PRIV_BYTES = KV8 ? CWARPS * PRIV_WARP_BYTES : 0;
  static constexpr int NSTAGE = (kRowsRingBytes - PRIV_BYTES) / STAGE_BYTES; /* 6 (head_dim 128), 12 (64), 5 (fp8) */
  static constexpr int Q_BYTES = NH * ROWS * 128;
  /* the warp-combine dump [RG][4][16*MT][HD+4] floats reuses the ring */
  static constexpr int DUMP_BYTES = RG * 4 * 16 * MT * (HD + 4) * 4;
  static constexpr int MIN_STAGES = (DUMP_BYTES + STAGE_BYTES - 1) / STAGE_BYTES < 2
                                        ? 2
                                        : (DUMP_BYTES + STAGE_BYTES - 1) / STAGE_BYTES;
  /* ring of `stages` stages | q tile | barriers (full, empty per stage) and the flag word */
  static constexpr int smem_bytes(int stages) {
    return stages * STAGE_BYTES + PRIV_BYTES + Q_BYTES + (2 * NSTAGE + 2) * 8 + 64 + 1024;
  }
  static_assert(MIN_STAGES <= NSTAGE, "combine buffer must fit the ring");
  static_assert(smem_bytes(NSTAGE) <= 232448, "shared memory of one CTA");
};


__device__ __forceinline__ void store_half4(__half *dst, float a, float b, float c, float d) {
  __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t *>(&lo);
  packed.y = *reinterpret_cast<uint32_t *>(&hi);
  *reinterpret_cast<uint2 *>(dst) = packed;
}

__device__ __forceinline__ void consumer_bar(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

/* four e4m3 bytes -> four fp16 values (exact: every e4m3 number is an fp16 number) */
__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t in, uint32_t &lo, uint32_t &hi) {
  asm("{\n\t.reg .b16 a, b;\n\t"
      "mov.b32 {a, b}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, a;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(in));
}

template <int HD, int MT, int RG, bool PAGED, bool KV8 = false>
__global__ void __launch_bounds__(Cfg<HD, MT, RG, KV8>::THREADS, 1)
attn_rows_kernel(const __grid_constant__ CUtensorMap kmap,
                 const __grid_constant__ CUtensorMap vmap, const RowsArgs a) {
  using C = Cfg<HD, MT, RG, KV8>;
  static_assert(!KV8 || (HD == 128 && !PAGED && MT == 1 && RG == 1), "fp8 cache: the decode shape");
  constexpr int BN = C::BN, NH = C::NH, ROWS = C::ROWS;
  constexpr int HALF_BYTES = C::HALF_BYTES, STAGE_BYTES = C::STAGE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / a.n_rowblk;
  const int rb = blockIdx.y % a.n_rowblk;
  const int s = blockIdx.z;
  const int nst = a.nstage;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t *qsm = smem + nst * STAGE_BYTES + C::PRIV_BYTES;
  const uint32_t priv_u32 = smem_u32(smem + nst * STAGE_BYTES); /* fp8 cache: the warps' fp16 copies */
  uint64_t *bars = reinterpret_cast<uint64_t *>(qsm + C::Q_BYTES);
  const uint32_t stages_u32 = smem_u32(smem);
  const uint32_t q_u32 = smem_u32(qsm);
  const uint32_t full_u32 = smem_u32(bars);
  const uint32_t empty_u32 = smem_u32(bars + C::NSTAGE);
  const uint32_t go_u32 = smem_u32(bars + 2 * C::NSTAGE); /* "dependency resolved", see below */

  if (threadIdx.x == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(full_u32 + 8 * i, 1);
      mbar_init(empty_u32 + 8 * i, C::CWARPS);
    }
    st_shared_volatile(go_u32, 0u);
    mbar_init_fence();
    tma_prefetch_desc(&kmap);
    tma_prefetch_desc(&vmap);
  }
  __syncthreads();

  /* Slice `split` owns tiles split, split + n_splits, split + 2 n_splits, ...:
   * the first tiles of a slice do not depend on the sequence length, so for a
   * single contiguous sequence the producer starts streaming them before the
   * cursor has even been read (tiles past the live rows are loaded and ignored;
   * they lie inside the cache allocation or read as zeros). */
  const int ns = a.n_splits;
  auto issue_to = [&](int tile, uint32_t full, uint32_t kdst) {
    mbar_arrive_expect_tx(full, STAGE_BYTES);
    const uint32_t vdst = kdst + (KV8 ? BN * HD : NH * HALF_BYTES);
    if constexpr (KV8) { /* a row of 128 e4m3 bytes is one 128-byte swizzle row: one box per tile */
      const int plane = s * a.n_kv + kvh;
      tma_load_3d(kdst, &kmap, full, 0, tile * BN, plane);
      tma_load_3d(vdst, &vmap, full, 0, tile * BN, plane);
    } else if constexpr (!PAGED) {
      const int plane = s * a.n_kv + kvh;
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        tma_load_3d(kdst + h * HALF_BYTES, &kmap, full, h * 64, tile * BN, plane);
        tma_load_3d(vdst + h * HALF_BYTES, &vmap, full, h * 64, tile * BN, plane);
      }
    } else {
#pragma unroll
      for (int pg = 0; pg < BN / 16; ++pg) {
        const int slot = tile * (BN / 16) + pg;
        int page = slot < a.max_pages
                       ? a.page_table[static_cast<long long>(s) * a.max_pages + slot]
                       : -1;
        /* an unmapped slot reads as zeros: coordinate just past the pool */
        if (page < 0 || page >= a.n_pool_pages) page = a.n_pool_pages;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          tma_load_4d(kdst + h * HALF_BYTES + pg * 16 * 128, &kmap, full, h * 64, 0, kvh, page);
          tma_load_4d(vdst + h * HALF_BYTES + pg * 16 * 128, &vmap, full, h * 64, 0, kvh, page);
        }
      }
    }
  };
  auto issue = [&](int i) {
    const int stage = i % nst;
    issue_to(split + i * ns, full_u32 + 8 * stage, stages_u32 + stage * STAGE_BYTES);
  };
  int spec = 0; /* tiles issued ahead of knowing the sequence length */
  if (!PAGED && a.cu_tokens == nullptr)
    while (spec < nst && static_cast<long long>(split + spec * ns) * BN < a.max_seq) ++spec;

  /* Decode (one new token): the launch just before this one in the stream --
   * still running under programmatic dependent launch -- can only be writing the
   * newest cache row; every row in a tile below that one was written by launches
   * that finished long ago.  So the slice's first tiles are requested right here,
   * before the dependency is resolved, and their latency hides behind the tail of
   * the previous kernel: `early_depth` of them at once, then one more whenever one
   * has landed (so that many stay in flight; all of the ring as soon as a consumer
   * thread reports the dependency resolved), so that the kernel ahead keeps getting
   * its own last loads out in between.  The newest row of a
   * tile requested this early is read again after the wait, with plain loads, and
   * stored over the copy in shared memory. */
  /* Let the kernels behind this one in the stream be scheduled as early as there is
   * room for them (the next launch's blocks start the moment this one's leave their
   * SM, a launch latency sooner than if they were released after the stream); what
   * they may read is ordered by their own griddepcontrol.wait, not by this. */
  grid_launch_dependents();
  const bool early = !PAGED && a.early_depth > 0;
  const int n_early = early ? spec : 0;
  if (early) {
    /* the group's q rows and the cursor towards L2 while the dependency is open: a
     * prefetch has no architectural effect, whatever the launch ahead still writes */
    if (warp == 0) {
      const char *qrow = reinterpret_cast<const char *>(a.q + static_cast<long long>(kvh) * a.gqa * HD);
      const int lines = (a.gqa * HD * 4 + 127) / 128;
      for (int l = lane; l < lines; l += 32)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(qrow + l * 128));
      if (lane == 0 && a.pos0_dev) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.pos0_dev));
    }
    if (warp == C::CWARPS) {
      if (lane == 0 && spec > 0) {
        const int window = a.early_depth < spec ? a.early_depth : spec;
        for (int i = 0; i < window; ++i) issue(i);
        for (int i = window; i < spec; ++i) { /* `window` tiles in flight at a time */
          const long long t0 = clock64();
          while (!mbar_try_wait(full_u32 + 8 * (i - window), 0) && ld_shared_volatile(go_u32) == 0u)
            if (clock64() - t0 > kWaitCycleLimit) break; /* only a hint: go on */
          issue(i);
        }
      }
      __syncwarp();
      grid_dependency_wait();
    } else {
      grid_dependency_wait();
    }
  } else {
    /* Nothing above touches global memory, so under programmatic dependent launch
     * it overlaps the tail of the previous kernel in the stream.  From here on we
     * read what that kernel may have written (cursor, q, cache rows). */
    grid_dependency_wait();
    if (warp == C::CWARPS && lane < spec) issue(lane); /* one lane per stage */
  }

  int tok_begin = s * a.tok_seq_stride, n_tok = a.n_tok;
  if (a.cu_tokens) {
    tok_begin = a.cu_tokens[s];
    n_tok = a.cu_tokens[s + 1] - tok_begin;
  }
  const int tok0 = rb * a.tpb;
  if (tok0 >= n_tok) return; /* ragged batch: this row block has no tokens (spec == 0 here) */
  const int ntok_blk = min(a.tpb, n_tok - tok0);
  const int rows_valid = ntok_blk * a.gqa;

  const int32_t pos_raw = a.pos0_dev ? a.pos0_dev[s] : 0; /* issued now, used below */

  /* q -> fp16, pre-multiplied by scale*log2(e), swizzled like the K tiles.  Done
   * before the cursor value is first used, so that the two global round trips
   * (cursor, q) overlap instead of following one another. */
  if (warp < C::CWARPS) {
    constexpr int ITEMS = ROWS * (HD / 8) / C::CTHREADS; /* exact: 1, 2 or 4 */
    static_assert(ITEMS * C::CTHREADS == ROWS * (HD / 8), "q tile must divide evenly");
    float4 lo[ITEMS], hi[ITEMS];
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) { /* every load in flight before any is used */
      const int idx = threadIdx.x + it * C::CTHREADS;
      const int row = idx / (HD / 8), ch = idx % (HD / 8);
      lo[it] = hi[it] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < rows_valid) {
        const int tok = tok_begin + tok0 + row / a.gqa;
        const int head = kvh * a.gqa + row % a.gqa;
        const float4 *src = reinterpret_cast<const float4 *>(
            a.q + static_cast<long long>(tok) * a.q_tok_stride +
            static_cast<long long>(head) * HD + ch * 8);
        lo[it] = __ldg(src);
        hi[it] = __ldg(src + 1);
      }
    }
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int idx = threadIdx.x + it * C::CTHREADS;
      const int row = idx / (HD / 8), ch = idx % (HD / 8);
      uint4 packed;
      packed.x = pack_half2(lo[it].x * a.qscale, lo[it].y * a.qscale);
      packed.y = pack_half2(lo[it].z * a.qscale, lo[it].w * a.qscale);
      packed.z = pack_half2(hi[it].x * a.qscale, hi[it].y * a.qscale);
      packed.w = pack_half2(hi[it].z * a.qscale, hi[it].w * a.qscale);
      *reinterpret_cast<uint4 *>(qsm + (ch >> 3) * (ROWS * 128) + swz128(row, ch & 7)) = packed;
    }
    /* the dependency is resolved and this thread's q rows are here: only now may the
     * producer ask for the rest of the ring at once -- released any earlier, those
     * requests (tens of KB per SM) queue ahead of the q loads and the first tile is
     * consumed 0.8 us later */
    if (threadIdx.x == 0) st_shared_volatile(go_u32, 1u);
  }

  int pos0 = a.pos0_dev ? pos_raw + a.pos0_bias : a.pos0_val;
  if (a.clamp_nonneg && pos0 < 0) pos0 = 0;
  const int max_seq = a.max_seq;
  auto limit_of = [pos0, max_seq](int tok) {
    long long l = static_cast<long long>(pos0) + tok + 1;
    l = l < 0 ? 0 : l;
    return static_cast<int>(l < max_seq ? l : max_seq);
  };
  const int kv_end = limit_of(tok0 + ntok_blk - 1); /* rows [0, kv_end) are live data */
  const int lim_min = limit_of(tok0);
  const int n_tiles = (kv_end + BN - 1) / BN;
  const int my_tiles = split < n_tiles ? (n_tiles - split + ns - 1) / ns : 0;

  /* the slice's tile that holds the newest row, if it was requested before the
   * dependency was resolved: that one row is patched from global memory */
  int patch = -1;
  if (my_tiles > 0 && my_tiles - 1 < n_early && split + (my_tiles - 1) * ns == n_tiles - 1)
    patch = my_tiles - 1;

  /* ------------------------------------------------------------ producer */
  if (warp == C::CWARPS) {
    if (lane != 0) return;
    for (int i = spec; i < my_tiles; ++i) {
      const int stage = i % nst, round = i / nst;
      if (i >= nst && !mbar_wait(empty_u32 + 8 * stage, (round - 1) & 1, a.err_word, 0x101u))
        break;
      issue(i);
    }
    return;
  }

  /* ----------------------------------------------------------- consumers */
  const int rg = warp >> 2; /* row group: rows [rg*16*MT, +16*MT) */
  const int w = warp & 3;   /* positions [16w, 16w+16) of every tile */
  const int ctid = threadIdx.x;

  /* the newest row's 16-byte chunks (K then V), one per lane, asked for now and
   * stored over the early copy when that tile is consumed (only the warp that owns
   * the row's positions; early requests are made for one row group only) */
  const int prow_new = (kv_end - 1) & (BN - 1);
  const bool patcher = patch >= 0 && w == (prow_new >> 4) && lane < 2 * NH * 8;
  uint4 patch_val = make_uint4(0u, 0u, 0u, 0u);
  if (patcher) {
    const int ch = lane % (NH * 8);
    const __half *src = (lane < NH * 8 ? a.k : a.v) +
                        (static_cast<long long>(s * a.n_kv + kvh) * a.max_seq + (kv_end - 1)) * HD +
                        ch * 8;
    patch_val = __ldcg(reinterpret_cast<const uint4 *>(src));
  }

  consumer_bar(C::CTHREADS);

  int lim[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = rg * 16 * MT + mt * 16 + (lane >> 2) + hh * 8;
      lim[mt][hh] = r < rows_valid ? limit_of(tok0 + r / a.gqa) : kv_end;
    }

  auto q_frag_addr = [&](int mt, int ks) {
    const int row = rg * 16 * MT + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int chg = 2 * ks + (lane >> 4);
    return q_u32 + (chg >> 3) * (ROWS * 128) + swz128(row, chg & 7);
  };

  uint32_t qf[MT == 1 ? HD / 16 : 1][4];
  if constexpr (MT == 1) {
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      ldsm_x4(q_frag_addr(0, ks), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  float m_run[MT][2], l_run[MT][2];
  float o[MT][HD / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[mt][nt][c] = 0.f;
  }

  int stage = 0;
  uint32_t phase = 0;
  for (int i = 0; i < my_tiles; ++i) {
    if (!mbar_wait(full_u32 + 8 * stage, phase, a.err_word, 0x102u)) break;
    const int tile = split + i * ns;
    uint32_t kb = stages_u32 + stage * STAGE_BYTES;
    uint32_t vb = kb + NH * HALF_BYTES;
    /* K / V operand addresses: row `prow` of the tile, 16-byte chunk `chg` of its HD halves */
    uint32_t row_off = 0, half_stride = HALF_BYTES;
    if constexpr (KV8) {
      /* this warp's 16 positions of the raw tile -> fp16 in its private buffer, in the
       * layout the fragment loads below expect ([NH][16 rows][128 B], swizzled): a lane
       * takes 4 of the 128 sixteen-byte chunks of K and of V; every chunk is 16 e4m3
       * values = two chunks of fp16.  Eight neighbouring lanes take the same chunk of eight
       * consecutive rows: eight different bank groups under the swizzle, in the raw tile
       * and in the copy (eight lanes along one row collide in pairs in the copy, whose
       * halves lie 2 KB apart). */
      const uint32_t kp = priv_u32 + warp * C::PRIV_WARP_BYTES, vp = kp + NH * 16 * 128;
      const uint32_t kraw = kb, vraw = kb + BN * HD;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t raw = t ? vraw : kraw, dst = t ? vp : kp;
        uint4 in[4];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int row = (lane & 7) + 8 * (c4 >> 1), ch8 = (lane >> 3) + 4 * (c4 & 1);
          asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(in[c4].x), "=r"(in[c4].y), "=r"(in[c4].z), "=r"(in[c4].w)
                       : "r"(raw + swz128(16 * w + row, ch8)));
        }
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int row = (lane & 7) + 8 * (c4 >> 1), ch8 = (lane >> 3) + 4 * (c4 & 1);
          const uint32_t words[4] = {in[c4].x, in[c4].y, in[c4].z, in[c4].w};
          uint32_t h[8];
#pragma unroll
          for (int k = 0; k < 4; ++k) e4m3x4_to_f16x4(words[k], h[2 * k], h[2 * k + 1]);
          const int ch = 2 * ch8; /* fp16 chunk index over the row's 16 chunks */
          const uint32_t at = dst + (ch >> 3) * (16 * 128);
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at + swz128(row, ch & 7)),
                       "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at + swz128(row, (ch + 1) & 7)),
                       "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
        }
      }
      __syncwarp();
      kb = kp;
      vb = vp;
      row_off = 16 * w; /* rows of the private copy count from the warp's first position */
      half_stride = 16 * 128;
    }
    if (i == patch) {
      if (patcher) {
        const int ch = lane % (NH * 8);
        const uint32_t dst = (lane < NH * 8 ? kb : vb) + (ch >> 3) * HALF_BYTES + swz128(prow_new, ch & 7);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(patch_val.x),
                     "r"(patch_val.y), "r"(patch_val.z), "r"(patch_val.w)
                     : "memory");
      }
      __syncwarp();
    }

    /* S = Q K^T for this warp's 16 positions */
    float sacc[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) sacc[mt][nt][c] = 0.f;

#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int mi = lane >> 3;
      const int prow = 16 * w + (mi >> 1) * 8 + (lane & 7);
      const int chg = 2 * ks + (mi & 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(kb + (chg >> 3) * half_stride + swz128(prow - row_off, chg & 7), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if constexpr (MT == 1) {
          mma_16816(sacc[0][0], qf[ks], b0, b1);
          mma_16816(sacc[0][1], qf[ks], b2, b3);
        } else {
          uint32_t af[4];
          ldsm_x4(q_frag_addr(mt, ks), af[0], af[1], af[2], af[3]);
          mma_16816(sacc[mt][0], af, b0, b1);
          mma_16816(sacc[mt][1], af, b2, b3);
        }
      }
    }

    /* causal / end-of-sequence mask: only tiles that reach past the smallest limit */
    if (tile * BN + BN > lim_min) {
      const int pbase = tile * BN + 16 * w + 2 * (lane & 3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int p = pbase + nt * 8 + (c & 1);
            if (p >= lim[mt][c >> 1]) sacc[mt][nt][c] = -INFINITY;
          }
    }

    /* online softmax in fp32, two rows per thread per 16-row tile */
    uint32_t pa[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float mx = fmaxf(fmaxf(sacc[mt][0][2 * hh], sacc[mt][0][2 * hh + 1]),
                         fmaxf(sacc[mt][1][2 * hh], sacc[mt][1][2 * hh + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[mt][hh], mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float corr = ex2(m_run[mt][hh] - m_use);
        m_run[mt][hh] = m_new;
        float psum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float p = ex2(sacc[mt][nt][2 * hh + c] - m_use);
            sacc[mt][nt][2 * hh + c] = p;
            psum += p;
          }
        l_run[mt][hh] = fmaf(l_run[mt][hh], corr, psum);
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
          o[mt][nt][2 * hh] *= corr;
          o[mt][nt][2 * hh + 1] *= corr;
        }
      }
      pa[mt][0] = pack_half2(sacc[mt][0][0], sacc[mt][0][1]);
      pa[mt][1] = pack_half2(sacc[mt][0][2], sacc[mt][0][3]);
      pa[mt][2] = pack_half2(sacc[mt][1][0], sacc[mt][1][1]);
      pa[mt][3] = pack_half2(sacc[mt][1][2], sacc[mt][1][3]);
    }

    /* Rows past the live data may hold anything (even NaN bit patterns), and
     * 0 * NaN is NaN: clear this warp's V rows beyond kv_end in the last tile. */
    if (tile * BN + BN > kv_end) {
      for (int idx = lane; idx < 16 * NH * 8; idx += 32) {
        const int prow = 16 * w + idx / (NH * 8);
        const int rest = idx % (NH * 8);
        if (tile * BN + prow >= kv_end) {
          asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(
                           vb + (rest >> 3) * half_stride + (prow - row_off) * 128 + (rest & 7) * 16),
                       "r"(0u)
                       : "memory");
        }
      }
      fence_async_smem();
      __syncwarp();
    }

    /* O += P V */
#pragma unroll
    for (int jj = 0; jj < HD / 16; ++jj) {
      const int mi = lane >> 3;
      const int prow = 16 * w + (mi & 1) * 8 + (lane & 7);
      const int chg = 2 * jj + (mi >> 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4_trans(vb + (chg >> 3) * half_stride + swz128(prow - row_off, chg & 7), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_16816(o[mt][2 * jj], pa[mt], b0, b1);
        mma_16816(o[mt][2 * jj + 1], pa[mt], b2, b3);
      }
    }

    __syncwarp();
    if (lane == 0) mbar_arrive(empty_u32 + 8 * stage);
    if (++stage == nst) {
      stage = 0;
      phase ^= 1u;
    }
  }

  /* Tiles that were streamed ahead but lie past this slice's share: wait for
   * them to land, nothing may still be in flight when the ring is reused. */
  for (int i = my_tiles; i < spec; ++i)
    if (!mbar_wait(full_u32 + 8 * (i % nst), (i / nst) & 1, a.err_word, 0x103u)) break;

  /* row sums live spread over the four lanes of a quad */
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float l = l_run[mt][hh];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      l_run[mt][hh] = l;
    }

  /* ---- combine the four warps of each row group through the idle ring: every
   * warp dumps its rows as [acc HD | m | l | pad pad], then each thread merges one
   * (row, 4-column) cell of the four copies and stores it, coalesced. */
  constexpr int DR = HD + 4;
  constexpr int RPG = 16 * MT; /* rows per row group */
  float *dump = reinterpret_cast<float *>(smem);
  consumer_bar(C::CTHREADS); /* every warp is done with the ring */
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float *row = dump + (static_cast<size_t>(rg * 4 + w) * RPG + mt * 16 + (lane >> 2) + hh * 8) * DR;
#pragma unroll
      for (int nt = 0; nt < HD / 8; ++nt)
        *reinterpret_cast<float2 *>(row + nt * 8 + 2 * (lane & 3)) =
            make_float2(o[mt][nt][2 * hh], o[mt][nt][2 * hh + 1]);
      if ((lane & 3) == 0) {
        row[HD] = m_run[mt][hh];
        row[HD + 1] = l_run[mt][hh];
      }
    }
  consumer_bar(C::CTHREADS);

  const int unit = (s * a.n_kv + kvh) * a.n_rowblk + rb;
  const bool direct = ns == 1 && !a.via_scratch;
  for (int idx = ctid; idx < rows_valid * (HD / 4); idx += C::CTHREADS) {
    const int r = idx / (HD / 4), c4 = idx % (HD / 4);
    const float *cell = dump + (static_cast<size_t>(r / RPG) * 4 * RPG + r % RPG) * DR;
    float mw[4], M = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mw[k] = cell[static_cast<size_t>(k) * RPG * DR + HD];
      M = fmaxf(M, mw[k]);
    }
    const float m_use = M == -INFINITY ? 0.f : M;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float wgt = ex2(mw[k] - m_use);
      const float4 v = *reinterpret_cast<const float4 *>(cell + static_cast<size_t>(k) * RPG * DR + 4 * c4);
      acc.x = fmaf(wgt, v.x, acc.x);
      acc.y = fmaf(wgt, v.y, acc.y);
      acc.z = fmaf(wgt, v.z, acc.z);
      acc.w = fmaf(wgt, v.w, acc.w);
      den = fmaf(wgt, cell[static_cast<size_t>(k) * RPG * DR + HD + 1], den);
    }
    if constexpr (KV8) { /* the stored values times their scale are the values */
      acc.x *= a.out_scale; acc.y *= a.out_scale; acc.z *= a.out_scale; acc.w *= a.out_scale;
    }
    const int head = kvh * a.gqa + r % a.gqa;
    if (direct && !a.partial_out) {
      const int tok = tok_begin + tok0 + r / a.gqa;
      const float inv = den > 0.f ? 1.f / den : 0.f;
      store_half4(static_cast<__half *>(a.out) +
                      (static_cast<long long>(tok) * a.n_q + head) * HD + 4 * c4,
                  acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    } else if (direct) { /* the caller's (m, l, acc) triple, natural-log m */
      float *dst = static_cast<float *>(a.out) + static_cast<long long>(head) * (HD + 2);
      if (c4 == 0) {
        dst[0] = M * kLn2;
        dst[1] = den;
      }
      reinterpret_cast<float2 *>(dst + 2 + 4 * c4)[0] = make_float2(acc.x, acc.y);
      reinterpret_cast<float2 *>(dst + 2 + 4 * c4)[1] = make_float2(acc.z, acc.w);
    } else { /* this slice's row for the merge kernel */
      float *dst = a.scratch +
                   ((static_cast<long long>(unit) * ns + split) * a.rows_cap + r) * DR;
      *reinterpret_cast<float4 *>(dst + 4 * c4) = acc;
      if (c4 == 0) *reinterpret_cast<float2 *>(dst + HD) = make_float2(M, den);
    }
  }
}

/* ---------------------------------------------------------- slice merge */

/* Second kernel of a split launch: one block per (unit, row).  Launched with
 * programmatic stream serialization, so its blocks are already resident when
 * the last slice finishes; each warp takes a quarter of the slices with every
 * load in flight at once (at most 16 per thread), so the merge costs about one
 * memory round trip.  Same arithmetic as cuda/attention.cu:170-193, in log2
 * units. */
struct MergeArgs {
  const float *scratch;
  void *out;
  const int32_t *cu_tokens;
  int n_tok, tok_seq_stride, n_q, n_kv, gqa;
  int n_splits, n_rowblk, tpb, rows_cap;
  const int *slice_counts; /* per unit, or null: n_splits for all */
  int partial_out;
  /* cross-GPU exchange (world > 1): one token, so a block is one query head */
  uint2 *const *mailboxes; /* [world] -> packets [2][world][n_q][hd+2] on rank g */
  unsigned int *xstate;    /* this rank: per-head call counters [n_q] */
  unsigned int *err_word;
  int rank, world;
};

/* ---- packets of the cross-GPU exchange: {value, tag} in ONE 64-bit access, so a
 * packet is valid exactly when its tag is the call's tag */
__device__ __forceinline__ unsigned long long make_packet(float value, unsigned int tag) {
  return (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(value);
}
__device__ __forceinline__ void st_packet(uint2 *p, float value, unsigned int tag) {
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(make_packet(value, tag)) : "memory");
}
__device__ __forceinline__ void st_packet2(uint2 *p, float v0, float v1, unsigned int tag) {
  asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(make_packet(v0, tag)),
               "l"(make_packet(v1, tag))
               : "memory");
}
/* two adjacent packets (16-byte aligned) in one request; each half is still a single
 * 64-bit access */
__device__ __forceinline__ void ld_packet2(const uint2 *p, unsigned long long &a,
                                           unsigned long long &b) {
  asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(128) attn_merge_kernel(const MergeArgs a) {
  constexpr int DR = HD + 4;
  constexpr int LPR = HD / 4;      /* lanes that cover one row as float4 */
  constexpr int SUB = 32 / LPR;    /* slice sub-groups inside a warp (1 or 2) */
  constexpr int GROUPS = 4 * SUB;  /* slice groups per block */
  constexpr int PER = kRowsMaxSplits / GROUPS;
  __shared__ float4 s_acc[GROUPS][LPR];
  __shared__ float s_m[GROUPS], s_l[GROUPS];

  grid_launch_dependents();
  /* the ranks' mailbox addresses never change: fetched while the dependency is open */
  uint2 *peer_box[8];
#pragma unroll
  for (int g = 0; g < 8; ++g) peer_box[g] = (a.world > 1 && g < a.world) ? a.mailboxes[g] : nullptr;
  grid_dependency_wait();

  const int row = blockIdx.x, unit = blockIdx.y;
  const int rb = unit % a.n_rowblk;
  const int kvh = (unit / a.n_rowblk) % a.n_kv;
  const int s = unit / (a.n_rowblk * a.n_kv);
  int tok_begin = s * a.tok_seq_stride, n_tok = a.n_tok;
  if (a.cu_tokens) {
    tok_begin = a.cu_tokens[s];
    n_tok = a.cu_tokens[s + 1] - tok_begin;
  }
  const int tok0 = rb * a.tpb;
  if (tok0 >= n_tok) return;
  const int ntok_blk = min(a.tpb, n_tok - tok0);
  if (row >= ntok_blk * a.gqa) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = warp * SUB + lane / LPR, c4 = lane % LPR;
  /* the head's call counter (exchange only), in flight together with the partial rows */
  const int head_x = ((unit / a.n_rowblk) % a.n_kv) * a.gqa + row % a.gqa;
  const unsigned int xcount = a.world > 1 ? __ldcg(a.xstate + head_x) : 0u;
  const int ns = a.slice_counts ? min(a.slice_counts[unit], a.n_splits) : a.n_splits;
  const float *base = a.scratch + (static_cast<long long>(unit) * a.n_splits * a.rows_cap + row) * DR;
  const long long sp_stride = static_cast<long long>(a.rows_cap) * DR;

  float4 v[PER];
  float2 ml[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int sp = group + i * GROUPS;
    if (sp < ns) {
      v[i] = __ldcg(reinterpret_cast<const float4 *>(base + sp * sp_stride) + c4);
      ml[i] = __ldcg(reinterpret_cast<const float2 *>(base + sp * sp_stride + HD));
    } else {
      v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      ml[i] = make_float2(-INFINITY, 0.f);
    }
  }
  float M = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) M = fmaxf(M, ml[i].x);
  const float m_use = M == -INFINITY ? 0.f : M;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const float wgt = ex2(ml[i].x - m_use);
    acc.x = fmaf(wgt, v[i].x, acc.x);
    acc.y = fmaf(wgt, v[i].y, acc.y);
    acc.z = fmaf(wgt, v[i].z, acc.z);
    acc.w = fmaf(wgt, v[i].w, acc.w);
    den = fmaf(wgt, ml[i].y, den);
  }
  s_acc[group][c4] = acc;
  if (c4 == 0) {
    s_m[group] = M;
    s_l[group] = den;
  }
  __syncthreads();
  if (threadIdx.x >= LPR) return;

  float big = -INFINITY;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) big = fmaxf(big, s_m[g]);
  const float big_use = big == -INFINITY ? 0.f : big;
  float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
  float dsum = 0.f;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const float wgt = ex2(s_m[g] - big_use);
    const float4 p = s_acc[g][threadIdx.x];
    tot.x = fmaf(wgt, p.x, tot.x);
    tot.y = fmaf(wgt, p.y, tot.y);
    tot.z = fmaf(wgt, p.z, tot.z);
    tot.w = fmaf(wgt, p.w, tot.w);
    dsum = fmaf(wgt, s_l[g], dsum);
  }
  const int head = kvh * a.gqa + row % a.gqa;
  const int col = 4 * threadIdx.x;

  if (a.world > 1) {
    /* The KV sequence is sharded over the GPUs of the box.  This rank's triple of the
     * head goes into every other rank's mailbox (plain peer stores over NVLink), the
     * others' are awaited in this GPU's own mailbox -- each packet for at most about a
     * second -- and folded in.  Every float travels as an 8-byte {value, tag} packet
     * written with one 64-bit store, so a packet is valid exactly when its tag is this
     * call's: no fence, no flag, no ordering between packets.  The tag is a per-head
     * call counter in device memory (graph replays advance it); mailboxes exist twice,
     * used by tag parity: a rank can publish call t+2 only after it has received
     * everybody's t+1, which they sent after reading t.  Every rank runs its own launch
     * on its own GPU; nothing here waits for another launch on the same GPU. */
    const float m_nat = big * kLn2;
    const unsigned int tag = xcount + 1u;
    const int par = static_cast<int>(tag & 1u);
    constexpr int stride = HD + 2;
    const long long my_slot = (static_cast<long long>(par) * a.world + a.rank) * a.n_q + head;
    auto publish = [&](uint2 *mailbox) {
      uint2 *dst = mailbox + my_slot * stride;
      if (threadIdx.x == 0) {
        st_packet(dst, m_nat, tag);
        st_packet(dst + 1, dsum, tag);
      }
      st_packet2(dst + 2 + col, tot.x, tot.y, tag);
      st_packet2(dst + 4 + col, tot.z, tot.w, tag);
    };
    uint2 *own_box = nullptr;
#pragma unroll
    for (int g = 0; g < 8; ++g) { /* the first eight ranks' addresses are in registers */
      if (g == a.rank) own_box = peer_box[g];
      if (g < a.world && g != a.rank) publish(peer_box[g]);
    }
    for (int g = 8; g < a.world; ++g)
      if (g != a.rank) publish(a.mailboxes[g]);
    if (a.rank >= 8) own_box = a.mailboxes[a.rank];
    const uint2 *box = own_box + (static_cast<long long>(par) * a.world * a.n_q + head) * stride;
    const long long rank_stride = static_cast<long long>(a.n_q) * stride;
    /* Fold the peers' triples in as they arrive, in any order (running maximum, like
     * the online softmax itself).  Per pass the packets of up to four pending peers are
     * requested together -- three 16-byte loads each, all in flight at once -- so a pass
     * costs one round trip to this GPU's L2, not one per packet. */
    float top = m_nat == -INFINITY ? -INFINITY : m_nat;
    float4 sum = tot;
    float lsum = dsum;
    if (m_nat == -INFINITY) {
      sum = make_float4(0.f, 0.f, 0.f, 0.f);
      lsum = 0.f;
    }
    unsigned int pending = (a.world >= 32 ? 0xffffffffu : ((1u << a.world) - 1u)) & ~(1u << a.rank);
    bool ok = true;
    const long long t0 = clock64();
    while (pending != 0u) {
      for (int base = 0; base < a.world; base += 4) {
        unsigned long long pk[4][6];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int g = base + k;
          if (g < a.world && ((pending >> g) & 1u)) {
            const uint2 *t = box + g * rank_stride;
            ld_packet2(t, pk[k][0], pk[k][1]);
            ld_packet2(t + 2 + col, pk[k][2], pk[k][3]);
            ld_packet2(t + 4 + col, pk[k][4], pk[k][5]);
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int g = base + k;
          if (g < a.world && ((pending >> g) & 1u)) {
            bool here = true;
#pragma unroll
            for (int i = 0; i < 6; ++i) here = here && static_cast<unsigned int>(pk[k][i] >> 32) == tag;
            if (!here) continue;
            pending &= ~(1u << g);
            const float m_g = __uint_as_float(static_cast<unsigned int>(pk[k][0]));
            if (m_g == -INFINITY) continue; /* an empty shard contributes nothing */
            const float top_new = fmaxf(top, m_g);
            const float f_old = top == -INFINITY ? 0.f : expf(top - top_new);
            const float f_new = expf(m_g - top_new);
            sum.x = fmaf(__uint_as_float(static_cast<unsigned int>(pk[k][2])), f_new, sum.x * f_old);
            sum.y = fmaf(__uint_as_float(static_cast<unsigned int>(pk[k][3])), f_new, sum.y * f_old);
            sum.z = fmaf(__uint_as_float(static_cast<unsigned int>(pk[k][4])), f_new, sum.z * f_old);
            sum.w = fmaf(__uint_as_float(static_cast<unsigned int>(pk[k][5])), f_new, sum.w * f_old);
            lsum = fmaf(__uint_as_float(static_cast<unsigned int>(pk[k][1])), f_new, lsum * f_old);
            top = top_new;
          }
        }
      }
      if (pending != 0u && clock64() - t0 > kWaitCycleLimit) {
        ok = false;
        break;
      }
    }
    ok = __all_sync(__activemask(), ok);
    if (ok) {
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      store_half4(static_cast<__half *>(a.out) + static_cast<long long>(head) * HD + col,
                  sum.x * inv, sum.y * inv, sum.z * inv, sum.w * inv);
    } else if (threadIdx.x == 0) {
      atomicCAS(a.err_word, 0u, 0x401u);
    }
    __syncwarp(); /* every lane has read the counter and is done with the call */
    if (threadIdx.x == 0) a.xstate[head] = tag;
    return;
  }

  if (a.partial_out) {
    float *dst = static_cast<float *>(a.out) + static_cast<long long>(head) * (HD + 2);
    if (threadIdx.x == 0) {
      dst[0] = big * kLn2;
      dst[1] = dsum;
    }
    reinterpret_cast<float2 *>(dst + 2 + col)[0] = make_float2(tot.x, tot.y);
    reinterpret_cast<float2 *>(dst + 2 + col)[1] = make_float2(tot.z, tot.w);
  } else {
    const int tok = tok_begin + tok0 + row / a.gqa;
    const float inv = dsum > 0.f ? 1.f / dsum : 0.f;
    store_half4(static_cast<__half *>(a.out) + (static_cast<long long>(tok) * a.n_q + head) * HD +
                    col,
                tot.x * inv, tot.y * inv, tot.z * inv, tot.w * inv);
  }
}

/* The slice merge for launches with few slices per unit and many rows (the ragged
 * verify: at most a handful of slices, tens of query rows per unit): one WARP per
 * (unit, row) instead of one block, eight rows per block, lane = four output columns,
 * up to eight slices' rows in flight per lane at once, folded with a running maximum.
 * An eighth as many blocks as attn_merge_kernel would launch, all resident in one wave. */
template <int HD>
__global__ void __launch_bounds__(256) attn_merge_rows_kernel(const MergeArgs a) {
  constexpr int DR = HD + 4;
  constexpr int LPR = HD / 4;
  grid_launch_dependents();
  grid_dependency_wait();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp, unit = blockIdx.y;
  const int rb = unit % a.n_rowblk;
  const int kvh = (unit / a.n_rowblk) % a.n_kv;
  const int s = unit / (a.n_rowblk * a.n_kv);
  int tok_begin = s * a.tok_seq_stride, n_tok = a.n_tok;
  if (a.cu_tokens) {
    tok_begin = a.cu_tokens[s];
    n_tok = a.cu_tokens[s + 1] - tok_begin;
  }
  const int tok0 = rb * a.tpb;
  if (tok0 >= n_tok) return;
  const int ntok_blk = min(a.tpb, n_tok - tok0);
  if (row >= ntok_blk * a.gqa || lane >= LPR) return;

  const int ns = a.slice_counts ? min(a.slice_counts[unit], a.n_splits) : a.n_splits;
  const float *base = a.scratch + (static_cast<long long>(unit) * a.n_splits * a.rows_cap + row) * DR;
  const long long sp_stride = static_cast<long long>(a.rows_cap) * DR;
  float M = -INFINITY, den = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sp0 = 0; sp0 < ns; sp0 += 8) {
    float4 v[8];
    float2 ml[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (sp0 + i < ns) {
        v[i] = __ldcg(reinterpret_cast<const float4 *>(base + (sp0 + i) * sp_stride) + lane);
        ml[i] = __ldcg(reinterpret_cast<const float2 *>(base + (sp0 + i) * sp_stride + HD));
      } else {
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        ml[i] = make_float2(-INFINITY, 0.f);
      }
    }
    float top = M;
#pragma unroll
    for (int i = 0; i < 8; ++i) top = fmaxf(top, ml[i].x);
    const float use = top == -INFINITY ? 0.f : top;
    const float keep = ex2(M - use); /* 0 while nothing has been folded in yet */
    acc.x *= keep;
    acc.y *= keep;
    acc.z *= keep;
    acc.w *= keep;
    den *= keep;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float wgt = ex2(ml[i].x - use);
      acc.x = fmaf(wgt, v[i].x, acc.x);
      acc.y = fmaf(wgt, v[i].y, acc.y);
      acc.z = fmaf(wgt, v[i].z, acc.z);
      acc.w = fmaf(wgt, v[i].w, acc.w);
      den = fmaf(wgt, ml[i].y, den);
    }
    M = top;
  }
  const int head = kvh * a.gqa + row % a.gqa;
  const int tok = tok_begin + tok0 + row / a.gqa;
  const float inv = den > 0.f ? 1.f / den : 0.f;
  store_half4(static_cast<__half *>(a.out) + (static_cast<long long>(tok) * a.n_q + head) * HD +
                  4 * lane,
              acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

/* ------------------------------------------------- portable fallback kernel */

/* One warp per (token, query head); eight lanes share a cache position, each
 * holding an hd/8 slice of q and of the accumulator, so a warp sweeps four
 * positions at a time.  CUDA cores only; natural-log softmax with expf. */
struct SimpleArgs {
  const float *q;
  long long q_tok_stride;
  const __half *k, *v;
  int n_q, gqa, hd, max_seq, n_tok;
  const int32_t *pos0_dev;
  int pos0_bias, clamp_nonneg, pos0_val;
  float scale;
  void *out;
  int partial_out;
};

template <int EPL> /* elements per lane = hd / 8, multiple of 4, <= 32 */
__global__ void __launch_bounds__(128) attn_simple_kernel(const SimpleArgs a) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= a.n_tok * a.n_q) return;
  const int tok = row / a.n_q, head = row % a.n_q;
  const int kvh = head / a.gqa;
  const int grp = lane >> 3, sub = lane & 7;

  int pos0 = a.pos0_dev ? *a.pos0_dev + a.pos0_bias : a.pos0_val;
  if (a.clamp_nonneg && pos0 < 0) pos0 = 0;
  long long lim_ll = static_cast<long long>(pos0) + tok + 1;
  lim_ll = lim_ll < 0 ? 0 : lim_ll;
  const int limit = static_cast<int>(lim_ll < a.max_seq ? lim_ll : a.max_seq);

  const int hd = a.hd;
  const float *qp = a.q + static_cast<long long>(tok) * a.q_tok_stride +
                    static_cast<long long>(head) * hd + sub * EPL;
  float qv[EPL], acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    qv[e] = qp[e] * a.scale;
    acc[e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const __half *kb = a.k + static_cast<long long>(kvh) * a.max_seq * hd + sub * EPL;
  const __half *vb = a.v + static_cast<long long>(kvh) * a.max_seq * hd + sub * EPL;

  for (int p0 = 0; p0 < limit; p0 += 4) {
    const int p = p0 + grp;
    const bool live = p < limit;
    float part = 0.f;
    if (live) {
      const __half2 *kr = reinterpret_cast<const __half2 *>(kb + static_cast<long long>(p) * hd);
#pragma unroll
      for (int e = 0; e < EPL / 2; ++e) {
        const float2 kk = __half22float2(kr[e]);
        part = fmaf(qv[2 * e], kk.x, part);
        part = fmaf(qv[2 * e + 1], kk.y, part);
      }
    }
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    if (live) {
      const float m_new = fmaxf(m, part);
      const float corr = expf(m - m_new);
      const float pw = expf(part - m_new);
      l = l * corr + pw;
      m = m_new;
      const __half2 *vr = reinterpret_cast<const __half2 *>(vb + static_cast<long long>(p) * hd);
#pragma unroll
      for (int e = 0; e < EPL / 2; ++e) {
        const float2 vv = __half22float2(vr[e]);
        acc[2 * e] = fmaf(pw, vv.x, acc[2 * e] * corr);
        acc[2 * e + 1] = fmaf(pw, vv.y, acc[2 * e + 1] * corr);
      }
    }
  }

  /* fold the four position groups together */
#pragma unroll
  for (int off = 8; off <= 16; off <<= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, off);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, off);
    const float m_new = fmaxf(m, m_o);
    const float c_me = m == -INFINITY ? 0.f : expf(m - m_new);
    const float c_ot = m_o == -INFINITY ? 0.f : expf(m_o - m_new);
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float a_o = __shfl_xor_sync(0xffffffffu, acc[e], off);
      acc[e] = acc[e] * c_me + a_o * c_ot;
    }
    l = l * c_me + l_o * c_ot;
    m = m_new;
  }
  if (grp != 0) return;
  if (a.partial_out) {
    float *dst = static_cast<float *>(a.out) + static_cast<long long>(head) * (hd + 2);
    if (sub == 0) {
      dst[0] = m;
      dst[1] = l;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[2 + sub * EPL + e] = acc[e];
  } else {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __half *dst = static_cast<__half *>(a.out) +
                  (static_cast<long long>(tok) * a.n_q + head) * hd + sub * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[e] = __float2half_rn(acc[e] * inv);
  }
}

/* ------------------------------------------------------------ host side */

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

/* Launch with programmatic stream serialization: the kernel may become resident
 * while its predecessor in the stream drains; it orders itself with
 * griddepcontrol.wait. */
template <typename Kern, typename... Args>
cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = current_stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  return e == cudaSuccess ? cudaGetLastError() : e;
}

template <int HD, int MT, int RG, bool PAGED, bool KV8 = false>
wst_status_t launch_cfg(const RowsLaunch &L, const RowsArgs &args, const CUtensorMap &kmap,
                        const CUtensorMap &vmap, dim3 grid) {
  using C = Cfg<HD, MT, RG, KV8>;
  auto kern = attn_rows_kernel<HD, MT, RG, PAGED, KV8>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  WST_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    WST_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  C::smem_bytes(C::NSTAGE)));
    configured_dev = dev;
  }
  /* the ring depth in use sizes the block's shared memory: at half the ring two blocks
   * (of consecutive launches) share an SM */
  RowsArgs sized = args;
  if (sized.nstage < C::MIN_STAGES) sized.nstage = C::MIN_STAGES;
  if (sized.nstage > C::NSTAGE) sized.nstage = C::NSTAGE;
  if (sized.early_depth > sized.nstage) sized.early_depth = sized.nstage;
  cudaError_t e = launch_pdl(kern, grid, dim3(C::THREADS), C::smem_bytes(sized.nstage), kmap, vmap,
                             sized);
  if (e != cudaSuccess)
    return fail(WST_ERR_CUDA, "%s (launch): %s (%s)", L.name, cudaGetErrorString(e),
                cudaGetErrorName(e));
  return WST_OK;
}

template <int HD, bool PAGED>
wst_status_t launch_shape(const RowsLaunch &L, const RowsArgs &args, const CUtensorMap &kmap,
                          const CUtensorMap &vmap, dim3 grid, int rows) {
  if (rows == 16) return launch_cfg<HD, 1, 1, PAGED>(L, args, kmap, vmap, grid);
  if (rows == 32) return launch_cfg<HD, 2, 1, PAGED>(L, args, kmap, vmap, grid);
  return launch_cfg<HD, 2, 2, PAGED>(L, args, kmap, vmap, grid);
}

/* Rows a block carries for `n_tok` tokens of a GQA group of `gqa` heads. */
int rows_for(int gqa, int n_tok) {
  const long long want = static_cast<long long>(gqa) * n_tok;
  if (want <= 16) return 16;
  if (want <= 32) return 32;
  return 64;
}

}  // namespace

bool rows_kernel_supports(int n_q, int n_kv, int hd, const void *k, const void *v) {
  if (hd != 64 && hd != 128) return false;
  if (n_kv <= 0 || n_q % n_kv != 0 || n_q / n_kv > 64) return false;
  return aligned16(k) && aligned16(v);
}

int rows_pick_splits(int n_units, int max_len, int sm_count) {
  /* Few units (decode): one slice per SM.  Many units of uneven length (a
   * ragged batch): slices of about 2048 positions, more blocks than SMs, and
   * the block scheduler evens out the lengths. */
  int splits = sm_count / (n_units > 0 ? n_units : 1);
  const int by_len = (max_len + 2047) / 2048;
  if (splits < by_len) splits = by_len;
  const int tiles = (max_len + kRowsTile - 1) / kRowsTile;
  if (splits > tiles) splits = tiles;
  if (splits > kRowsMaxSplits) splits = kRowsMaxSplits;
  if (splits < 1) splits = 1;
  return splits;
}

long long rows_scratch_floats(int n_units_times_rows, int splits, int hd) {
  return static_cast<long long>(n_units_times_rows) * splits * (hd + 4);
}

RowsTuning &rows_tuning() {
  static RowsTuning t;
  return t;
}

static std::atomic<int> g_decode_overlap{1};
bool decode_overlap_allowed() { return g_decode_overlap.load() != 0; }
void set_decode_overlap(bool on) { g_decode_overlap.store(on ? 1 : 0); }

/* tiles a decode launch requests at once ahead of its grid dependency, and the ring
 * depth of a decode launch at head_dim 128 (twice as many half-size stages at 64) */
constexpr int kDefaultEarlyDepth = 2;
constexpr int kDecodeStages = 6;

wst_status_t launch_rows(const RowsLaunch &L) {
  DeviceFacts facts;
  if (!device_facts(&facts)) return WST_ERR_CUDA;
  if (facts.cc_major < 10)
    return fail(WST_ERR_UNSUPPORTED_ARCH, "%s: this library is built for sm_100a only", L.name);
  const RowsTuning &tune = rows_tuning();

  const int gqa = L.n_q / L.n_kv;
  const int rows = rows_for(gqa, L.n_tok);
  int tpb = rows / gqa; /* tokens per row block */
  if (tpb > L.n_tok) tpb = L.n_tok;
  const int n_rowblk = (L.n_tok + tpb - 1) / tpb;
  const int n_units = L.n_seq * L.n_kv * n_rowblk;
  const int rows_cap = tpb * gqa;
  const bool decode_shape = !L.paged && !L.cu_tokens && L.n_tok == 1 && L.n_seq == 1;

  int splits = L.want_splits > 0 ? L.want_splits : rows_pick_splits(n_units, L.max_len, facts.sm_count);
  if (decode_shape && L.want_splits <= 0) {
    /* Decode leaves an eighth of the SMs without a slice.  The slices are a static,
     * equal partition, so one launch is as slow as its slowest SM; and the free SMs take
     * the merge kernel's blocks and the first blocks of the NEXT launch, which fill
     * their rings and wait, so consecutive launches overlap like a software pipeline.
     * Measured at 28/4/128: 13.1 us per layer at context 32768 with 32 slices per KV
     * head against 14.2 with 37 (all 148 SMs), 33.4 against 40.6 at context 100000. */
    int cap = facts.sm_count * 7 / 8 / (n_units > 0 ? n_units : 1);
    if (cap < 1) cap = 1;
    if (tune.decode_splits > 0) cap = tune.decode_splits;
    const int tiles = (L.max_len + kRowsTile - 1) / kRowsTile;
    if (cap > tiles) cap = tiles;
    if (splits > cap || tune.decode_splits > 0) splits = cap;
  }
  if (splits > kRowsMaxSplits) splits = kRowsMaxSplits;
  /* the slices must fit the caller's scratch */
  if (!aligned16(L.scratch)) splits = 1; /* the merge reads scratch rows as float4 */
  while (splits > 1 &&
         (!L.scratch || rows_scratch_floats(n_units * rows_cap, splits, L.hd) > L.scratch_floats))
    --splits;

  /* The cross-GPU exchange rides in the merge kernel (one block per query head). */
  const bool exchange = L.world > 1;
  if (exchange && !(decode_shape && L.mailboxes && L.xstate && L.scratch && aligned16(L.scratch) &&
                    rows_scratch_floats(n_units * rows_cap, splits, L.hd) <= L.scratch_floats))
    return fail(WST_ERR_SHAPE,
                "%s: the in-kernel exchange takes one token of one contiguous sequence with a "
                "split scratch (head_dim 64 or 128)", L.name);

  if (L.kv8 && !(L.hd == 128 && !L.paged && rows == 16))
    return fail(WST_ERR_SHAPE,
                "%s: the fp8 cache takes head_dim 128, a contiguous cache and at most 16 query "
                "rows per KV head", L.name);

  RowsArgs a{};
  a.q = L.q;
  a.q_tok_stride = L.q_tok_stride;
  a.k = L.k;
  a.v = L.v;
  a.page_table = L.page_table;
  a.max_pages = L.max_pages;
  a.n_pool_pages = L.n_pool_pages;
  a.pos0_dev = L.pos0_dev;
  a.pos0_bias = L.pos0_bias;
  a.clamp_nonneg = L.clamp_pos0_nonneg ? 1 : 0;
  a.pos0_val = L.pos0_val;
  a.cu_tokens = L.cu_tokens;
  a.n_tok = L.n_tok;
  a.tok_seq_stride = L.tok_seq_stride;
  a.n_q = L.n_q;
  a.n_kv = L.n_kv;
  a.gqa = gqa;
  a.max_seq = L.max_seq;
  a.qscale = L.scale * kLog2e * (L.kv8 ? L.k_scale : 1.f); /* keys = stored bytes * k_scale */
  a.out_scale = L.kv8 ? L.v_scale : 1.f;
  a.scratch = L.scratch;
  a.out = L.out;
  a.partial_out = L.partial_out ? 1 : 0;
  a.n_splits = splits;
  a.n_rowblk = n_rowblk;
  a.tpb = tpb;
  a.rows_cap = rows_cap;
  a.via_scratch = exchange ? 1 : 0;
  const int max_stages = kRowsRingBytes / (L.hd == 128 ? 32768 : 16384);
  a.nstage = max_stages;
  if (decode_shape) a.nstage = L.hd == 128 ? kDecodeStages : 2 * kDecodeStages;
  if (tune.ring_stages >= 2 && tune.ring_stages <= max_stages) a.nstage = tune.ring_stages;
  if (L.kv8) a.nstage = Cfg<128, 1, 1, true>::NSTAGE;
  /* requests ahead of the grid dependency: decode only (the launch ahead writes at
   * most the newest row), one row group (the patch of that row is a warp's job) */
  a.early_depth = 0;
  if (L.newest_row_only && decode_shape && rows <= 32 && decode_overlap_allowed() && !L.kv8) {
    a.early_depth = tune.early_depth >= 0 ? tune.early_depth : kDefaultEarlyDepth;
    if (a.early_depth > a.nstage) a.early_depth = a.nstage;
  }
  a.err_word = device_error_word();
  if (!a.err_word) return WST_ERR_CUDA;
  CUtensorMap kmap, vmap;
  KvMapKey key{};
  key.d0 = static_cast<uint64_t>(L.kv8 ? L.hd / 2 : L.hd); /* fp8 rows described as 64 two-byte elements */
  if (L.paged) {
    key.d1 = 16; key.d2 = static_cast<uint64_t>(L.n_kv); key.d3 = static_cast<uint64_t>(L.n_pool_pages);
    key.b1 = 16; key.rank = 4;
  } else {
    key.d1 = static_cast<uint64_t>(L.max_seq);
    key.d2 = static_cast<uint64_t>(L.n_kv) * L.n_seq; key.d3 = 1;
    key.b1 = kRowsTile; key.rank = 3;
  }
  key.base = L.k;
  wst_status_t st = cached_kv_tensor_map(&kmap, key);
  if (st != WST_OK) return st;
  key.base = L.v;
  st = cached_kv_tensor_map(&vmap, key);
  if (st != WST_OK) return st;

  const dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(L.n_kv * n_rowblk),
                  static_cast<unsigned>(L.n_seq));
  if (L.kv8) {
    st = launch_cfg<128, 1, 1, false, true>(L, a, kmap, vmap, grid);
  } else if (L.hd == 128) {
    st = L.paged ? launch_shape<128, true>(L, a, kmap, vmap, grid, rows)
                 : launch_shape<128, false>(L, a, kmap, vmap, grid, rows);
  } else {
    st = L.paged ? launch_shape<64, true>(L, a, kmap, vmap, grid, rows)
                 : launch_shape<64, false>(L, a, kmap, vmap, grid, rows);
  }
  if (st != WST_OK || (splits == 1 && !exchange)) return st;

  SplitMerge m;
  m.scratch = L.scratch;
  m.out = L.out;
  m.cu_tokens = L.cu_tokens;
  m.n_tok = L.n_tok;
  m.tok_seq_stride = L.tok_seq_stride;
  m.n_q = L.n_q;
  m.n_kv = L.n_kv;
  m.hd = L.hd;
  m.n_splits = splits;
  m.n_rowblk = n_rowblk;
  m.tpb = tpb;
  m.rows_cap = rows_cap;
  m.n_units = n_units;
  m.partial_out = L.partial_out;
  m.mailboxes = L.mailboxes;
  m.xstate = L.xstate;
  m.rank = L.rank;
  m.world = exchange ? L.world : 1;
  m.name = L.name;
  return launch_split_merge(m);
}

wst_status_t launch_split_merge(const SplitMerge &S) {
  MergeArgs m{};
  m.scratch = S.scratch;
  m.out = S.out;
  m.cu_tokens = S.cu_tokens;
  m.n_tok = S.n_tok;
  m.tok_seq_stride = S.tok_seq_stride;
  m.n_q = S.n_q;
  m.n_kv = S.n_kv;
  m.gqa = S.n_q / S.n_kv;
  m.n_splits = S.n_splits;
  m.n_rowblk = S.n_rowblk;
  m.tpb = S.tpb;
  m.rows_cap = S.rows_cap;
  m.partial_out = S.partial_out ? 1 : 0;
  m.slice_counts = S.slice_counts;
  m.mailboxes = static_cast<uint2 *const *>(S.mailboxes);
  m.xstate = static_cast<unsigned int *>(S.xstate);
  m.rank = S.rank;
  m.world = S.world;
  m.err_word = device_error_word();
  if (!m.err_word) return WST_ERR_CUDA;
  cudaError_t e;
  if ((S.slice_counts || (S.n_splits <= 16 && S.rows_cap >= 16)) && !S.partial_out && S.world <= 1) {
    /* few slices, many rows (ragged verify, a sliced chunk): a warp per row */
    const dim3 rgrid(static_cast<unsigned>((S.rows_cap + 7) / 8), static_cast<unsigned>(S.n_units));
    e = S.hd == 128 ? launch_pdl(attn_merge_rows_kernel<128>, rgrid, dim3(256), 0, m)
                    : launch_pdl(attn_merge_rows_kernel<64>, rgrid, dim3(256), 0, m);
  } else {
    const dim3 mgrid(static_cast<unsigned>(S.rows_cap), static_cast<unsigned>(S.n_units));
    e = S.hd == 128 ? launch_pdl(attn_merge_kernel<128>, mgrid, dim3(128), 0, m)
                    : launch_pdl(attn_merge_kernel<64>, mgrid, dim3(128), 0, m);
  }
  if (e != cudaSuccess)
    return fail(WST_ERR_CUDA, "%s (merge launch): %s (%s)", S.name, cudaGetErrorString(e),
                cudaGetErrorName(e));
  return WST_OK;
}

wst_status_t launch_simple(const RowsLaunch &L) {
  if (L.paged || L.n_seq != 1 || L.cu_tokens)
    return fail(WST_ERR_SHAPE, "%s: the portable kernel takes one contiguous sequence", L.name);
  if (L.hd % 32 != 0 || L.hd > 256 || L.hd <= 0)
    return fail(WST_ERR_INVALID_ARG, "%s: head_dim must be a multiple of 32, at most 256", L.name);
  SimpleArgs a{};
  a.q = L.q;
  a.q_tok_stride = L.q_tok_stride;
  a.k = L.k;
  a.v = L.v;
  a.n_q = L.n_q;
  a.gqa = L.n_q / L.n_kv;
  a.hd = L.hd;
  a.max_seq = L.max_seq;
  a.n_tok = L.n_tok;
  a.pos0_dev = L.pos0_dev;
  a.pos0_bias = L.pos0_bias;
  a.clamp_nonneg = L.clamp_pos0_nonneg ? 1 : 0;
  a.pos0_val = L.pos0_val;
  a.scale = L.scale;
  a.out = L.out;
  a.partial_out = L.partial_out ? 1 : 0;
  const long long rows = static_cast<long long>(L.n_tok) * L.n_q;
  const dim3 grid(static_cast<unsigned>((rows + 3) / 4)), block(128);
  cudaStream_t st = current_stream();
  switch (L.hd / 8) {
    case 4: attn_simple_kernel<4><<<grid, block, 0, st>>>(a); break;
    case 8: attn_simple_kernel<8><<<grid, block, 0, st>>>(a); break;
    case 12: attn_simple_kernel<12><<<grid, block, 0, st>>>(a); break;
    case 16: attn_simple_kernel<16><<<grid, block, 0, st>>>(a); break;
    case 20: attn_simple_kernel<20><<<grid, block, 0, st>>>(a); break;
    case 24: attn_simple_kernel<24><<<grid, block, 0, st>>>(a); break;
    case 28: attn_simple_kernel<28><<<grid, block, 0, st>>>(a); break;
    default: attn_simple_kernel<32><<<grid, block, 0, st>>>(a); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(WST_ERR_CUDA, "%s (launch): %s (%s)", L.name, cudaGetErrorString(e),
                cudaGetErrorName(e));
  return WST_OK;
}

}  // namespace wst
