// Grouped expert matrix products on the 5th-generation tensor cores (tcgen05), bfloat16.
//
// Both products are computed transposed ("swap-AB"): the weight tile is the M side of the MMA
// (128 output features per tile, always full), the expert's token rows are the N side (BN = 16 to
// 256), so a decode step with a handful of rows per expert still issues full-width MMAs and the
// kernel's time is the time to stream the weights from HBM once.
//
//   D^T[feature, token] = sum_k W[e][feature][k] * X[row(token)][k]
//
//   A (weights)      : TMA tiles of bf16, K-major, 128-byte swizzle, from a 3-D tensor map over
//                      [E, rows, K].  gemm2 takes 128 consecutive rows in one box.  gemm1 interleaves, per
//                      TMEM lane quadrant, 16 gate rows with the 16 matching up rows, so one accumulator
//                      holds both halves and a warp finds gate and up of a feature 16 lanes apart; the
//                      interleave is done by the tensor map itself (a 5-D view [E, I/16, 2, 16, K] of the
//                      weights), so it is still one TMA instruction per stage.
//   B (activations)  : TMA tile [BN rows x 64 k] from a 2-D map over the expert-sorted rows [R, K]; or,
//                      for gemm1 given the tokens in their own order and the sorted routes, gathered by
//                      two more warps with 16-byte cp.async copies straight into the swizzled tile (a
//                      token's row is read where the norm wrote it: no copy of the rows into expert
//                      order, no launch for it).
//   D (accumulator)  : TMEM, 128 lanes x BN float32 columns, two buffers so the epilogue of one tile
//                      overlaps the main loop of the next.
//
// One CTA = 8 warps: warp 0 issues TMA loads, warp 1 allocates TMEM and issues tcgen05.mma, warps 2-5
// read the accumulator (tcgen05.ld, one TMEM lane quadrant each), apply the epilogue and store, warps
// 6-7 gather token rows (gemm1 from unsorted tokens only; otherwise they leave at once).
//   gemm1 epilogue: gate and up are rounded to bfloat16 (where the reference stores them), the two
//                   half-warps swap what the other needs by a warp shuffle (one takes tokens 0-7 of a
//                   chunk, the other tokens 8-15), act(g, u) is stored.
//   gemm2 epilogue: accumulator x route weight (float32), stored as bfloat16; a tile's route weights
//                   (token -> route -> weight, two loads one after the other) are fetched a tile ahead.
//   Both epilogues read the accumulator 16 columns at a time, the next chunk's load under this chunk's
//   arithmetic, turn the (feature x token) chunk round in a warp-private piece of shared memory and
//   store 16 bytes per thread.
// CTAs are persistent: tile t -> (expert, token tile, feature tile) is derived from the device-side
// expert offsets, so ragged row counts need no padding and no host round trip.
//
// Token tiles of 128 and 256 rows with many tiles (long steps) run on PAIRS of CTAs, clusters of two
// (template argument PAIR, see Smem): one tile of 256 weight rows per pair, tcgen05.mma.cta_group::2 issued
// by the leading CTA, each CTA loading its own weight rows and half of the tokens; the partner's TMA loads
// are counted at the leading CTA's barrier, tcgen05.commit with cluster multicast arrives at both CTAs'
// barriers.  No TMA load is multicast: every CTA loads its own tiles.  Every wait on an mbarrier is
// bounded; on a timeout the CTA records a status code, lets copies in flight land, frees its TMEM and
// returns, and the host reports the code (ftk_read_status).
//
// Stands for the reference's Triton grouped GEMM, its per-route decode GEMV and the activation kernel
// (python/freetoken/kernel/triton/fused_moe.py:156-302, python/freetoken/kernel/triton/decode_moe.py:5-75,
// python/freetoken/kernel/triton/activation.py:67-112).
#include "tc_common.cuh"

namespace ftk {

__device__ int g_status[4];  // [0] first error code, [1] block, [2] detail; 0 = fine

constexpr int kThreads = 256;
constexpr int kGatherThreads = 64;  // warps 6 and 7
constexpr int kBK = 64;          // k elements per stage (128 bytes: one swizzle row)
constexpr int kTileM = 128;      // accumulator rows (TMEM lanes)
constexpr int kABytes = kTileM * kBK * 2;
constexpr int kMaxExperts = 1024;

struct TcParams {
  const int32_t* offsets;        // [E + 1]
  int n_experts;
  int K;                         // reduction length
  int n_out;                     // output features per row (I for gemm1, H for gemm2)
  int m_tiles;                   // feature tiles per expert
  int up_row_offset;             // gemm1: I (row of the up half that matches gate row 0)
  const int32_t* sorted_routes;  // gemm2; gemm1 when it gathers
  const float* route_weights;    // gemm2
  // gemm1 gathering its rows: the tokens' rows [gather_rows, K] in their own order; sorted row r is the row
  // of token sorted_routes[r] / gather_div
  const __nv_bfloat16* gather_src;
  int gather_div;
  int gather_rows;
  int n_routes;
  int act;
  float alpha, limit;
  __nv_bfloat16* out;
};

// DEEP: one CTA per SM (many tiles: each SM streams on its own, with a longer pipeline for the large
// token tiles); otherwise two CTAs per SM (few tiles: more of them run at once).
// PAIR: two CTAs (a cluster) work on one tile of 256 weight rows x BN tokens with cta_group::2: each CTA
// loads and multiplies its own 128 weight rows (its own feature tile) and half of the tile's tokens, the
// tensor cores read the other half from the partner's shared memory.  A token tile then enters an SM once per
// 256 weight rows instead of once per 128, which is what binds these sizes (measured: 9.0-9.4 TB/s from L2
// into the SMs at 4,096, 8,192 and 16,384 tokens, whatever the pipeline's depth and the boxes' size).
template <int BN, bool DEEP, bool PAIR = false>
struct Smem {
  // 64-element pieces of k per stage.  Two of them make every row of a weight tile a 256-byte read,
  // which the memory serves faster than twice 128 bytes (measured: 6.7 against 6.1 TB/s).
  static constexpr int kAtoms = DEEP ? 2 : 1;
  static constexpr int kStages = PAIR ? (BN <= 128 ? 4 : 3)
                                 : DEEP ? (BN <= 16 ? 5 : (BN <= 32 ? 4 : (BN <= 64 ? 4 : (BN <= 128 ? 3 : 2))))
                                        : (BN <= 16 ? 5 : (BN <= 128 ? 4 : 3));
  // loads kept in flight while every CTA streams (measured for the small token tiles: 144 KB per SM
  // is the best; more of them from all SMs at once slow the memory down)
  static constexpr int kDepth = (DEEP && BN <= 16) ? 4 : kStages;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;  // token rows of a tile in this CTA's shared memory
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kBBoxRows = BN < 32 ? BN : 32;  // token rows per TMA box: only boxes with rows are loaded
  static constexpr int kStageBytes = kAtoms * (kABytes + kBBytes);
  static constexpr int kAccCols = BN;                  // TMEM columns of one accumulator buffer
  static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
  static constexpr int kDynamic = kStages * kStageBytes + 1024;
};

template <int BN, bool GATED, bool DEEP, bool PAIR = false>
__global__ void __launch_bounds__(kThreads) moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b,
                                                               TcParams p) {
  // The expert offsets are read before pdl_wait(): whoever writes them (the routing kernels) never lets
  // the next kernel in early, so they are complete when any block of this kernel runs.  The weight
  // tiles of the first loads go out before the wait too; what the kernel before wrote (the activations)
  // is read after it, and nothing is stored before it.
  pdl_trigger();
  using S = Smem<BN, DEEP, PAIR>;
  extern __shared__ unsigned char dyn_smem[];
  __shared__ uint64_t full_bar[S::kStages], empty_bar[S::kStages], acc_full[2], acc_empty[2];
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // CTA 0 of a pair leads: it issues the products
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int tile_prefix[kMaxExperts + 1];  // token tiles of experts 0..e-1
  __shared__ float turn[4][16][33];             // per epilogue warp: a 16-token chunk turned round
  __shared__ float tile_w[GATED ? 1 : 2][GATED ? 1 : 4][GATED ? 1 : BN];  // per epilogue warp: the route weights of this tile's tokens and the next's

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles_base = (smem_addr(dyn_smem) + 1023u) & ~1023u;
  unsigned char* tiles = dyn_smem + (tiles_base - smem_addr(dyn_smem));

  const bool gathers = GATED && p.gather_src != nullptr;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(&full_bar[s], gathers ? 1 + kGatherThreads : 1);  // the TMA thread, and every gathering thread
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], PAIR ? 8 : 4);  // the epilogue warps (of both CTAs)
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair(&tmem_slot, S::kTmemCols); else tmem_alloc(&tmem_slot, S::kTmemCols);
  }
  // token tiles per expert, prefix-summed by warp 0
  if (warp == 0) {
    const int E = p.n_experts;
    const int per = (E + 31) / 32;
    int local = 0;
    for (int i = 0; i < per; ++i) {
      const int e = lane * per + i;
      if (e < E) local += (p.offsets[e + 1] - p.offsets[e] + BN - 1) / BN;
    }
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - local;
    for (int i = 0; i < per; ++i) {
      const int e = lane * per + i;
      if (e < E) {
        tile_prefix[e] = run;
        run += (p.offsets[e + 1] - p.offsets[e] + BN - 1) / BN;
      }
    }
    if (lane == 31) tile_prefix[E] = incl;
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the partner's barriers are set up before anything arrives at them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int m_units = PAIR ? (p.m_tiles + 1) / 2 : p.m_tiles;  // feature tiles, or pairs of them
  const int total_tiles = tile_prefix[p.n_experts] * m_units;
  // Tiles are dealt out in turns.  A last turn with a tile for only a few CTAs costs about two thirds of
  // a whole turn (a lone SM streams a tile at about 70 GB/s, not much faster than its share when all
  // SMs stream).  Where that costs more than it, only as many CTAs take part as fill every turn: with
  // 1,344 tiles on 148 SMs, 135 CTAs take ten tiles each instead of 148 taking nine and twelve of them
  // a tenth.  The others leave at once.  Costs are counted in tile times of a full turn.
  const int all = PAIR ? (int)gridDim.x / 2 : (int)gridDim.x;           // CTAs, or pairs of them
  const int me = PAIR ? (int)blockIdx.x / 2 : (int)blockIdx.x;
  const int turns = (total_tiles + all - 1) / all;
  const int even = turns > 0 ? (total_tiles + turns - 1) / turns : 1;
  const int rest = total_tiles % all;
  const int cost_all = total_tiles - rest + (rest ? max(rest, 2 * all / 3) : 0);
  // (one CTA per SM and the small token tiles only: that is where it was measured)
  const int G = (DEEP && BN <= 32 && turns * even < cost_all) ? even : all;
  const int t_first = me < G ? me : total_tiles;
  const int k_blocks = (p.K + S::kAtoms * kBK - 1) / (S::kAtoms * kBK);  // k past the end reads as zero
  volatile int* abortp = &abort_flag;

  constexpr int kFeat = GATED ? 64 : 128;  // output features of one feature tile
  // tile -> expert, token tile, first feature
  auto locate = [&](int t, int& e, int& row0, int& rows, int& m0) {
    const int g = t / m_units;
    m0 = PAIR ? ((t % m_units) * 2 + (int)rank) * kFeat : (t % m_units) * kFeat;
    int lo = 0, hi = p.n_experts - 1;  // last e with tile_prefix[e] <= g
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (tile_prefix[mid] <= g) lo = mid; else hi = mid - 1;
    }
    e = lo;
    const int start = p.offsets[e], end = p.offsets[e + 1];
    row0 = start + (g - tile_prefix[e]) * BN;
    rows = min(BN, end - row0);
  };
  // the token rows this CTA loads for a tile: first row and number of boxes.  A pair computes a multiple of 64
  // columns, half of them from each CTA's shared memory.
  auto token_part = [&](int row0, int rows, int& b0, int& nb) {
    if (PAIR) {
      const int half = min(BN, (rows + 63) & ~63) / 2;
      b0 = row0 + (int)rank * half;
      nb = half / S::kBBoxRows;
    } else {
      b0 = row0;
      nb = (rows + S::kBBoxRows - 1) / S::kBBoxRows;
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // Load i goes to stage i % kStages.  While every CTA streams, a CTA keeps only `depth` loads in
      // flight (more of them from all SMs at once slow the memory down); in the last, partly filled
      // wave of tiles the few CTAs that still work use every stage, since each of them is then bound
      // by the latency of its own loads.
      int i = 0;
      bool ok = true;
      const int full_waves = total_tiles / G * G;
      const bool thin_tail = 2 * (total_tiles - full_waves) <= G;
      const int depth_main = S::kDepth;
      auto stage_bytes = [&](int rows) {
        int b0, nb;
        token_part(0, rows, b0, nb);
        if (gathers) nb = 0;
        // (the leading CTA of a pair counts the partner's bytes too: both load the same amount)
        return (uint32_t)((PAIR ? 2 : 1) * S::kAtoms * (kABytes + nb * S::kBBoxRows * kBK * 2));
      };
      // the barrier a stage's loads are counted at: this CTA's, of a pair the leading CTA's
      auto full_of = [&](int s) { return PAIR ? cluster_address_of(&full_bar[s], 0) : smem_addr(&full_bar[s]); };
      auto load_a = [&](int s, int kb, int m0, int e) {
        unsigned char* a = tiles + s * S::kStageBytes;
#pragma unroll
        for (int h = 0; h < S::kAtoms; ++h) {
          const int k0 = (kb * S::kAtoms + h) * kBK;
          unsigned char* dst = a + h * kABytes;  // weight rows past the expert's last read as zero
          if (GATED) {  // (k, row in group, gate|up, group of 16 features, expert)
            if (PAIR) tma_load_5d_pair(dst, &map_a, full_of(s), k0, 0, 0, m0 >> 4, e);
            else tma_load_5d(dst, &map_a, &full_bar[s], k0, 0, 0, m0 >> 4, e);
          } else {
            if (PAIR) tma_load_3d_pair(dst, &map_a, full_of(s), k0, m0, e);
            else tma_load_3d(dst, &map_a, &full_bar[s], k0, m0, e);
          }
        }
      };
      auto load_b = [&](int s, int kb, int row0, int rows) {
        if (gathers) return;  // warps 6 and 7 bring the rows
        unsigned char* b = tiles + s * S::kStageBytes + S::kAtoms * kABytes;
        int b0, nb;
        token_part(row0, rows, b0, nb);
#pragma unroll
        for (int h = 0; h < S::kAtoms; ++h)
          for (int jb = 0; jb < nb; ++jb) {
            unsigned char* dst = b + h * S::kBBytes + jb * S::kBBoxRows * kBK * 2;
            if (PAIR) tma_load_2d_pair(dst, &map_b, full_of(s), (kb * S::kAtoms + h) * kBK, b0 + jb * S::kBBoxRows);
            else tma_load_2d(dst, &map_b, &full_bar[s], (kb * S::kAtoms + h) * kBK, b0 + jb * S::kBBoxRows);
          }
      };
      // the weights of the first loads, while the kernel before this one may still be running
      int ahead = 0;
      if (t_first < total_tiles) {
        int e, row0, rows, m0;
        locate(t_first, e, row0, rows, m0);
        ahead = min(depth_main, k_blocks);
        for (int kb = 0; kb < ahead; ++kb) {
          if (rank == 0) mbar_expect_tx(&full_bar[kb], stage_bytes(rows));
          load_a(kb, kb, m0, e);
        }
        pdl_wait();
        for (int kb = 0; kb < ahead; ++kb) load_b(kb, kb, row0, rows);
      } else {
        pdl_wait();
      }
      for (int t = t_first; t < total_tiles && ok; t += G) {
        int e, row0, rows, m0;
        locate(t, e, row0, rows, m0);
        const int depth = (t >= full_waves && thin_tail) ? S::kStages : depth_main;
        for (int kb = 0; kb < k_blocks; ++kb, ++i) {
          if (t == t_first && kb < ahead) continue;  // already on its way
          const int j = i - depth;  // the load whose stage must have been read before load i goes out
          if (j >= 0 && !mbar_wait(&empty_bar[j % S::kStages], (uint32_t)(j / S::kStages) & 1u, abortp)) {
            ok = false;
            atomicCAS(&g_status[0], 0, 101);
            abort_flag = 1;
            break;
          }
          const int s = i % S::kStages;
          if (rank == 0) mbar_expect_tx(&full_bar[s], stage_bytes(rows));
          load_a(s, kb, m0, e);
          load_b(s, kb, row0, rows);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (of a pair: the leading CTA's)
    if (lane == 0 && rank == 0) {
      int s = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;  // bit a: phase of accumulator buffer a
      int acc = 0;
      bool ok = true;
      for (int t = t_first; t < total_tiles && ok; t += G) {
        if (!(PAIR ? mbar_wait_cluster(&acc_empty[acc], ((acc_phase >> acc) & 1u) ^ 1u, abortp)
                   : mbar_wait(&acc_empty[acc], ((acc_phase >> acc) & 1u) ^ 1u, abortp))) {
          atomicCAS(&g_status[0], 0, 102);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        int e, row0, rows, m0;
        locate(t, e, row0, rows, m0);
        // only the columns of tokens that exist are computed (and only their boxes were loaded)
        const uint32_t idesc = PAIR ? instr_desc_pair(min(BN, (rows + 63) & ~63)) : instr_desc(min(BN, (rows + 15) & ~15));
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * S::kAccCols);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[s], phase, abortp)) {  // (of a pair: both CTAs' loads are counted here)
            ok = false;
            atomicCAS(&g_status[0], 0, 103);
            abort_flag = 1;
            break;
          }
          if (gathers) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // rows written by cp.async
          tc_fence_after();
          const uint32_t a_addr = tiles_base + s * S::kStageBytes;
#pragma unroll
          for (int h = 0; h < S::kAtoms; ++h) {
            const uint64_t b_desc = smem_desc(a_addr + S::kAtoms * kABytes + h * S::kBBytes);
            const uint64_t a_desc = smem_desc(a_addr + h * kABytes);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {  // 16 k elements = 32 bytes = 2 descriptor units
              if (PAIR) tc_mma_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | h | k) != 0);
              else tc_mma(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | h | k) != 0);
            }
          }
          // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if (PAIR) tc_commit_pair(&empty_bar[s]); else tc_commit(&empty_bar[s]);
          if (++s == S::kStages) {
            s = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (PAIR) tc_commit_pair(&acc_full[acc]); else tc_commit(&acc_full[acc]);
        acc_phase ^= 1u << acc;
        acc ^= 1;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ gather (warps 6 and 7, gemm1 from unsorted tokens)
    // Thread g copies 16-byte chunk g % 8 of the 128-byte row pieces of rows g / 8, g / 8 + 8, ... of the
    // token tile, into the place the 128-byte swizzle gives it; a row without a token is filled with zeros.
    if (gathers) {
      const int g = (warp - 6) * 32 + lane, c = g & 7, rbase = g >> 3;
      constexpr int kPer = BN / 8;  // rows of a tile per thread
      pdl_wait();
      int i = 0;
      bool ok = true;
      for (int t = t_first; t < total_tiles && ok; t += G) {
        int e, row0, rows, m0;
        locate(t, e, row0, rows, m0);
        const int r_end = min(BN, (rows + 15) & ~15);  // the columns the MMAs compute
        int tok[kPer];
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
          const int r = rbase + 8 * q;
          int tk = -1;
          if (r < rows) {
            const int route = p.sorted_routes[row0 + r];
            tk = route >= 0 ? route / p.gather_div : -1;
            if (tk >= p.gather_rows) tk = -1;
          }
          tok[q] = tk;
        }
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++i) {
          const int s = i % S::kStages;
          if (i >= S::kStages && !mbar_wait(&empty_bar[s], (uint32_t)(i / S::kStages - 1) & 1u, abortp)) {
            ok = false;
            atomicCAS(&g_status[0], 0, 105);
            abort_flag = 1;
            break;
          }
          const uint32_t b_addr = tiles_base + s * S::kStageBytes + S::kAtoms * kABytes;
#pragma unroll
          for (int h = 0; h < S::kAtoms; ++h) {
            const int k0 = (kb * S::kAtoms + h) * kBK + c * 8;
#pragma unroll
            for (int q = 0; q < kPer; ++q) {
              const int r = rbase + 8 * q;
              if (r < r_end) {
                const bool there = tok[q] >= 0 && k0 < p.K;  // (K is a multiple of 8: a chunk is inside or outside)
                const __nv_bfloat16* src = p.gather_src + (there ? (size_t)tok[q] * p.K + k0 : 0);
                const uint32_t dst = b_addr + h * S::kBBytes + r * 128 + ((c ^ (r & 7)) << 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(there ? 16 : 0) : "memory");
              }
            }
          }
          // this thread's arrival at the stage's barrier happens when its copies have landed
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&full_bar[s])) : "memory");
        }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;               // TMEM lanes [32 quad, 32 quad + 32)
    uint32_t acc_phase = 0;
    int acc = 0;
    pdl_wait();  // nothing is stored while the kernel before this one runs; a block without tiles waits too
    // The route weights of a tile's tokens (down product) are two loads, one after the other: token -> route ->
    // weight.  They are fetched a tile ahead, the routes before this tile's accumulator is waited for, the
    // weights in the middle of its chunks, so that neither holds the epilogue up.
    constexpr int kWPer = (BN + 31) / 32;
    int wbuf = 0;
    int next_route[kWPer];
    auto fetch_routes = [&](int t2) {
      int e2, row02, rows2, m02;
      if (t2 < total_tiles) locate(t2, e2, row02, rows2, m02); else rows2 = 0;
#pragma unroll
      for (int j = 0; j < kWPer; ++j) {
        const int n = lane + 32 * j;
        next_route[j] = (n < rows2) ? p.sorted_routes[row02 + n] : -1;
      }
    };
    auto fetch_weights = [&](int buf) {
      float wv[kWPer];
#pragma unroll
      for (int j = 0; j < kWPer; ++j)
        wv[j] = (next_route[j] >= 0 && next_route[j] < p.n_routes) ? p.route_weights[next_route[j]] : 0.f;
#pragma unroll
      for (int j = 0; j < kWPer; ++j)
        if (lane + 32 * j < BN) tile_w[buf][quad][lane + 32 * j] = wv[j];
      __syncwarp();
    };
    if (!GATED) {
      fetch_routes(t_first);
      fetch_weights(0);
    }
    for (int t = t_first; t < total_tiles; t += G) {
      int e, row0, rows, m0;
      locate(t, e, row0, rows, m0);
      if (!GATED) fetch_routes(t + G);
      // the whole warp takes one decision: the loads below need all 32 lanes
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[acc], (acc_phase >> acc) & 1u, abortp))) {
        if (lane == 0) atomicCAS(&g_status[0], 0, 104);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int c_end = min(BN, (rows + 15) & ~15);
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * S::kAccCols);
      float (*tb)[33] = turn[quad];
      // One chunk of 16 tokens (columns c..c+15 of this warp's 32 accumulator rows), turned round through
      // shared memory so that a thread stores 8 consecutive features of one token.
      auto chunk = [&](const uint32_t (&r)[16], int c) {
        if (GATED) {
          // lanes 0-15 of a quadrant hold gate, lanes 16-31 the up values of the same 16 features.  Both halves
          // work: a lane of the first takes tokens 0-7 of its feature (and gets their up values from its
          // partner), a lane of the second tokens 8-15 (and gets their gate values).
          const bool first = lane < 16;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float mine = __uint_as_float(first ? r[i] : r[8 + i]);
            const float theirs = __shfl_xor_sync(0xffffffffu, __uint_as_float(first ? r[8 + i] : r[i]), 16);
            const float g = to_float(__float2bfloat16_rn(first ? mine : theirs));
            const float u = to_float(__float2bfloat16_rn(first ? theirs : mine));
            tb[first ? i : 8 + i][lane & 15] = gated_act_fast(g, u, p.act, p.alpha, p.limit);
          }
          __syncwarp();
          // 16 tokens x 16 features: one 16-byte store (8 features of one token) per thread
          const int n = c + (lane >> 1), f0 = m0 + quad * 16 + (lane & 1) * 8;
          if (n < rows && f0 < p.n_out) {
            const float* src = &tb[lane >> 1][(lane & 1) * 8];
            __nv_bfloat16* dst = p.out + (size_t)(row0 + n) * p.n_out + f0;
            if (f0 + 8 <= p.n_out) {
              uint4 pk;
              pk.x = pack2(src[0], src[1]); pk.y = pack2(src[2], src[3]);
              pk.z = pack2(src[4], src[5]); pk.w = pack2(src[6], src[7]);
              *reinterpret_cast<uint4*>(dst) = pk;
            } else {
              for (int e2 = 0; f0 + e2 < p.n_out; ++e2) dst[e2] = __float2bfloat16_rn(src[e2]);
            }
          }
          __syncwarp();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) tb[i][lane] = __uint_as_float(r[i]) * tile_w[wbuf][quad][c + i];
          __syncwarp();
          // 16 tokens x 32 features: two 16-byte stores per thread
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int tk = (lane >> 2) + 8 * j;
            const int n = c + tk, f0 = m0 + quad * 32 + (lane & 3) * 8;
            if (n < rows && f0 < p.n_out) {
              const float* src = &tb[tk][(lane & 3) * 8];
              __nv_bfloat16* dst = p.out + (size_t)(row0 + n) * p.n_out + f0;
              if (f0 + 8 <= p.n_out) {
                uint4 pk;
                pk.x = pack2(src[0], src[1]); pk.y = pack2(src[2], src[3]);
                pk.z = pack2(src[4], src[5]); pk.w = pack2(src[6], src[7]);
                *reinterpret_cast<uint4*>(dst) = pk;
              } else {
                for (int e2 = 0; f0 + e2 < p.n_out; ++e2) dst[e2] = __float2bfloat16_rn(src[e2]);
              }
            }
          }
          __syncwarp();
        }
      };
      // after the last read of this accumulator buffer it goes back to the MMA warp
      auto release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR && rank == 1) mbar_arrive_remote(&acc_empty[acc], 0); else mbar_arrive(&acc_empty[acc]);
        }
      };
      // the next chunk's load runs under this chunk's arithmetic and stores
      uint32_t ra[16], rb[16];
      tmem_ld16_start(t_addr, ra);
      bool weights_fetched = GATED;
#pragma unroll 1
      for (int c = 0; c < c_end; c += 32) {
        if (!weights_fetched && 2 * c >= c_end) {  // (the other buffer: this tile still reads its own)
          fetch_weights(wbuf ^ 1);
          weights_fetched = true;
        }
        tmem_ld16_finish(ra);
        const bool more = c + 16 < c_end;
        if (more) tmem_ld16_start(t_addr + c + 16, rb); else release();
        chunk(ra, c);
        if (more) {
          tmem_ld16_finish(rb);
          if (c + 32 < c_end) tmem_ld16_start(t_addr + c + 32, ra); else release();
          chunk(rb, c + 16);
        }
      }
      if (!weights_fetched) fetch_weights(wbuf ^ 1);
      wbuf ^= 1;
      acc_phase ^= 1u << acc;
      acc ^= 1;
    }
  }
  // ---------------------------------------------------------------- teardown
  if (abort_flag) {
    if (threadIdx.x == 0) g_status[1] = blockIdx.x;
    for (int i = 0; i < 2000; ++i) __nanosleep(100);  // let copies in flight land before the CTA leaves
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // nothing of the partner's is still on its way to this CTA
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, S::kTmemCols); else tmem_dealloc(tmem_base, S::kTmemCols);
  }
}

// ---------------------------------------------------------------- host side
static int pick_bn(int n_routes, int n_experts) {
  const int want = (int)(1.5 * n_routes / n_experts) + 8;
  for (int bn : {16, 32, 64, 128}) if (want <= bn) return bn;
  return 256;
}

template <int BN, bool GATED, bool DEEP>
static int launch_tc_impl(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int max_tiles, cudaStream_t s) {
  using S = Smem<BN, DEEP>;
  auto kern = moe_gemm_tc_kernel<BN, GATED, DEEP>;
  static int ctas_per_sm = 0, sms = 0;
  if (!ctas_per_sm) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic) != cudaSuccess) return 2;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int n = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, S::kDynamic);
    // the query can answer for the current carve-out rather than the largest one: also count by hand
    cudaFuncAttributes fa;
    int smem_sm = 0;
    cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    if (cudaFuncGetAttributes(&fa, kern) == cudaSuccess && smem_sm > 0) {
      const int per_cta = S::kDynamic + (int)fa.sharedSizeBytes + 1024;
      const int by_hand = smem_sm / per_cta;
      if (by_hand > n) n = by_hand;
    }
    const int by_tmem = 512 / S::kTmemCols;
    ctas_per_sm = n < 1 ? 1 : (n > by_tmem ? by_tmem : n);
    if (ctas_per_sm > 2) ctas_per_sm = 2;
    if (DEEP) ctas_per_sm = 1;
  }
  {
    static const char* const names[2][2][5] = {
        {{"expert down product: tcgen05, 16 tokens a tile", "expert down product: tcgen05, 32 tokens a tile",
          "expert down product: tcgen05, 64 tokens a tile", "expert down product: tcgen05, 128 tokens a tile",
          "expert down product: tcgen05, 256 tokens a tile"},
         {"expert down product: tcgen05, 16 tokens a tile, deep pipeline", "expert down product: tcgen05, 32 tokens a tile, deep pipeline",
          "expert down product: tcgen05, 64 tokens a tile, deep pipeline", "expert down product: tcgen05, 128 tokens a tile, deep pipeline",
          "expert down product: tcgen05, 256 tokens a tile, deep pipeline"}},
        {{"expert gate/up product: tcgen05, 16 tokens a tile", "expert gate/up product: tcgen05, 32 tokens a tile",
          "expert gate/up product: tcgen05, 64 tokens a tile", "expert gate/up product: tcgen05, 128 tokens a tile",
          "expert gate/up product: tcgen05, 256 tokens a tile"},
         {"expert gate/up product: tcgen05, 16 tokens a tile, deep pipeline", "expert gate/up product: tcgen05, 32 tokens a tile, deep pipeline",
          "expert gate/up product: tcgen05, 64 tokens a tile, deep pipeline", "expert gate/up product: tcgen05, 128 tokens a tile, deep pipeline",
          "expert gate/up product: tcgen05, 256 tokens a tile, deep pipeline"}}};
    note_variant(names[GATED ? 1 : 0][DEEP ? 1 : 0][BN == 16 ? 0 : BN == 32 ? 1 : BN == 64 ? 2 : BN == 128 ? 3 : 4]);
  }
  int grid = sms * ctas_per_sm;
  if (grid > max_tiles) grid = max_tiles;
  if (grid < 1) grid = 1;
  FTK_LAUNCH(kern, grid, kThreads, S::kDynamic, s, ma, mb, p);
  return 0;
}

static int g_pairs_enabled = 1;

// Token tiles of 256 rows, many tiles: pairs of CTAs on tiles of 256 weight rows.  -1 when the device
// cannot hold a cluster of two such CTAs (the caller then launches the one-CTA form).
template <int BN, bool GATED>
static int launch_tc_pairs(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int max_token_tiles, cudaStream_t s) {
  using S = Smem<BN, true, true>;
  auto kern = moe_gemm_tc_kernel<BN, GATED, true, true>;
  static int clusters = -1;
  if (clusters < 0) {
    clusters = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamic) != cudaSuccess) return -1;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = S::kDynamic;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) clusters = n < sms / 2 ? n : sms / 2;
    cudaGetLastError();
  }
  if (clusters < 1) return -1;
  note_variant(BN == 256 ? (GATED ? "expert gate/up product: tcgen05, 256 tokens a tile, pairs of CTAs"
                                  : "expert down product: tcgen05, 256 tokens a tile, pairs of CTAs")
                         : (GATED ? "expert gate/up product: tcgen05, 128 tokens a tile, pairs of CTAs"
                                  : "expert down product: tcgen05, 128 tokens a tile, pairs of CTAs"));
  const long long pair_tiles = (long long)max_token_tiles * ((p.m_tiles + 1) / 2);
  const int pairs = (int)(pair_tiles < clusters ? (pair_tiles < 1 ? 1 : pair_tiles) : clusters);
  launch_kernel_clusters(kern, 2, dim3((unsigned)(2 * pairs)), dim3(kThreads), (size_t)S::kDynamic, s, ma, mb, p);
  return 0;
}

// Few tiles: shallow pipelines, two CTAs per SM.  More than two tiles per SM: one deep pipeline per SM.
template <int BN, bool GATED>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int max_tiles, int likely_tiles,
                     cudaStream_t s) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // measured: 192 tiles (one token) are faster two CTAs to an SM, 384 (two tokens) already one deep pipeline per SM
  if (likely_tiles > 2 * sms) return launch_tc_impl<BN, GATED, true>(ma, mb, p, max_tiles, s);
  return launch_tc_impl<BN, GATED, false>(ma, mb, p, max_tiles, s);
}

template <bool GATED>
static int run_tc(const void* x, int x_cols, const void* w, int w_rows, const TcParams& p, cudaStream_t s,
                  const char* name) {
  // TMA needs 16-byte row strides; the epilogue stores 8 features at a time; the gate/up interleave
  // works on groups of 16 features
  if (x_cols % 8 != 0 || p.n_out % 8 != 0 || p.n_experts > kMaxExperts) return -1;
  if (GATED && p.n_out % 16 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -1;
  const int bn = pick_bn(p.n_routes, p.n_experts);
  CUtensorMap ma, mb;
  const uint64_t K = (uint64_t)x_cols;
  if (GATED) {
    // [E][2][I/16][16][K] seen as (K, 16, 2, I/16, E): a box of (64, 16, 2, 4, 1) lands in shared memory as
    // 4 groups of [16 gate rows, 16 up rows]
    const uint64_t I = (uint64_t)p.n_out;
    const uint64_t dims[5] = {K, 16, 2, I / 16, (uint64_t)p.n_experts};
    const uint64_t strides[4] = {K * 2, I * K * 2, 16 * K * 2, 2 * I * K * 2};
    const uint32_t box[5] = {kBK, 16, 2, 4, 1};
    if (!make_map(&ma, w, 5, dims, strides, box)) {
      set_error("%s: cuTensorMapEncodeTiled refused the weight map", name);
      return 4;
    }
  } else {
    const uint64_t dims[3] = {K, (uint64_t)w_rows, (uint64_t)p.n_experts};
    const uint64_t strides[2] = {K * 2, (uint64_t)w_rows * K * 2};
    const uint32_t box[3] = {kBK, 128, 1};
    if (!make_map(&ma, w, 3, dims, strides, box)) {
      set_error("%s: cuTensorMapEncodeTiled refused the weight map", name);
      return 4;
    }
  }
  {
    const uint64_t dims[2] = {K, (uint64_t)(p.gather_src ? p.gather_rows : p.n_routes)};  // (not read when the kernel gathers)
    const uint64_t strides[1] = {K * 2};
    const uint32_t box[2] = {kBK, (uint32_t)(bn < 32 ? bn : 32)};  // Smem::kBBoxRows
    if (!make_map(&mb, x, 2, dims, strides, box)) {
      set_error("%s: cuTensorMapEncodeTiled refused the activation map", name);
      return 4;
    }
  }
  const int max_tiles = ((p.n_routes + bn - 1) / bn + p.n_experts) * p.m_tiles;
  // token tiles when the routes spread evenly: experts that got rows, each with its share of tiles
  const int busy = p.n_routes < p.n_experts ? p.n_routes : p.n_experts;
  const int per_expert = (p.n_routes / (busy > 0 ? busy : 1) + bn - 1) / bn;
  const int likely_tiles = busy * (per_expert > 0 ? per_expert : 1) * p.m_tiles;
  int rc;
  switch (bn) {
    case 16: rc = launch_tc<16, GATED>(ma, mb, p, max_tiles, likely_tiles, s); break;
    case 32: rc = launch_tc<32, GATED>(ma, mb, p, max_tiles, likely_tiles, s); break;
    case 64: rc = launch_tc<64, GATED>(ma, mb, p, max_tiles, likely_tiles, s); break;
    case 128: {
      int dev = 0, sms = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      rc = -1;
      if (g_pairs_enabled && likely_tiles > 2 * sms && p.m_tiles >= 2 && !p.gather_src)
        rc = launch_tc_pairs<128, GATED>(ma, mb, p, (p.n_routes + bn - 1) / bn + p.n_experts, s);
      if (rc < 0) rc = launch_tc<128, GATED>(ma, mb, p, max_tiles, likely_tiles, s);
      break;
    }
    default: {
      int dev = 0, sms = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      rc = -1;
      if (g_pairs_enabled && likely_tiles > 2 * sms && p.m_tiles >= 2 && !p.gather_src)
        rc = launch_tc_pairs<256, GATED>(ma, mb, p, (p.n_routes + bn - 1) / bn + p.n_experts, s);
      if (rc < 0) rc = launch_tc<256, GATED>(ma, mb, p, max_tiles, likely_tiles, s);
      break;
    }
  }
  if (rc) {
    set_error("%s: cannot configure the tensor-core kernel", name);
    return rc;
  }
  FTK_LAUNCH_CHECK(name);
  return 0;
}

}  // namespace ftk

using namespace ftk;

static int g_tc_enabled = 1;

// 0 sends bfloat16 grouped products to the CUDA-core kernels (for comparisons); default 1.
extern "C" int ftk_set_moe_tensor_cores(int enabled) {
  g_tc_enabled = enabled ? 1 : 0;
  return 0;
}

// 0 keeps token tiles of 128 and 256 rows on the one-CTA form (for comparisons); default 1: pairs of CTAs where they fit.
extern "C" int ftk_set_moe_pairs(int enabled) {
  g_pairs_enabled = enabled ? 1 : 0;
  return 0;
}

// `sorted_routes` given: x holds the tokens' rows [n_tokens, hidden] in their own order and the kernel
// gathers (row r of expert order is the row of token sorted_routes[r] / top_k); nullptr: x holds the
// n_routes rows in expert order.
int ftk_moe_gemm1_act_tc(const void* x, const void* w1, const int32_t* expert_offsets, int n_experts,
                         int n_routes, int hidden, int inter, int act, float alpha, float limit, void* out,
                         const int32_t* sorted_routes, int top_k, int n_tokens, cudaStream_t stream) {
  if (!g_tc_enabled) return -1;
  TcParams p{};
  p.offsets = expert_offsets; p.n_experts = n_experts; p.K = hidden; p.n_out = inter;
  p.m_tiles = (inter + 63) / 64; p.up_row_offset = inter; p.n_routes = n_routes;
  p.act = act; p.alpha = alpha; p.limit = limit; p.out = (__nv_bfloat16*)out;
  if (sorted_routes) {
    if (top_k < 1 || n_tokens < 1 || pick_bn(n_routes, n_experts) > 32) return -1;
    p.sorted_routes = sorted_routes;
    p.gather_src = (const __nv_bfloat16*)x;
    p.gather_div = top_k;
    p.gather_rows = n_tokens;
  }
  return run_tc<true>(x, hidden, w1, 2 * inter, p, stream,
                      sorted_routes ? "moe_gemm1_act (tcgen05, gathering)" : "moe_gemm1_act (tcgen05)");
}

// Whether ftk_moe_gemm1_act_gather will take these sizes on the tensor cores (bfloat16 only).  Token tiles of
// up to 32 rows only: the two gathering warps keep up with those (measured at 256 experts of 3072 x 1536:
// as fast as from copied rows up to 512 tokens x 8 routes; with 64-row tiles, 1,024 tokens, 0.82 ms against
// 0.72, with 128-row tiles, 2,048 tokens, 1.67 against 0.77), so longer steps copy their rows first.
extern "C" int ftk_moe_gemm1_gather_fits(int hidden, int inter, int n_experts, int n_routes) {
  return g_tc_enabled && hidden % 8 == 0 && inter % 16 == 0 && n_experts <= kMaxExperts && n_routes >= 1 &&
         pick_bn(n_routes, n_experts) <= 32;
}

int ftk_moe_gemm2_tc(const void* a, const void* w2, const int32_t* expert_offsets, const int32_t* sorted_routes,
                     const float* topk_weights, int n_experts, int n_routes, int hidden, int inter, void* out,
                     cudaStream_t stream) {
  if (!g_tc_enabled) return -1;
  TcParams p{};
  p.offsets = expert_offsets; p.n_experts = n_experts; p.K = inter; p.n_out = hidden;
  p.m_tiles = (hidden + 127) / 128; p.sorted_routes = sorted_routes; p.route_weights = topk_weights;
  p.n_routes = n_routes; p.out = (__nv_bfloat16*)out;
  return run_tc<false>(a, inter, w2, hidden, p, stream, "moe_gemm2 (tcgen05)");
}

// Status of the bounded waits: out[0] = first code recorded since the last call (0 = none),
// out[1] = block, then cleared.  Synchronises with the device.
int ftk_attention_tc_status(int* out);       // attention.cu
int ftk_attention_tc_set_status(int code);  // attention.cu

// Writes a code into a status word from the host, as a kernel whose wait ran out would: unit 0 = the
// grouped GEMM's word, 1 = the attention kernel's.  It exists so that the path from a status word to the
// caller's error can be exercised without making any wait on the device run out.
extern "C" int ftk_debug_set_status(int unit, int code) {
  if (unit == 1) {
    if (ftk_attention_tc_set_status(code) != 0) {
      set_error("debug_set_status: cannot write the attention status word");
      return 2;
    }
    return 0;
  }
  if (unit != 0) {
    set_error("debug_set_status: unit must be 0 (grouped GEMM) or 1 (attention), got %d", unit);
    return 1;
  }
  int host[4] = {code, -1, 0, 0};
  if (cudaMemcpyToSymbol(g_status, host, sizeof(host)) != cudaSuccess) {
    set_error("debug_set_status: cannot write the status words");
    return 2;
  }
  return 0;
}

extern "C" int ftk_read_status(int* out) {
  int attn[2] = {0, 0};
  if (ftk_attention_tc_status(attn) == 0 && attn[0]) {
    out[0] = attn[0];
    out[1] = attn[1];
    return 0;
  }
  int host[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(host, g_status, sizeof(host)) != cudaSuccess) {
    set_error("read_status: cannot read the status words");
    return 2;
  }
  out[0] = host[0];
  out[1] = host[1];
  if (host[0]) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  }
  return 0;
}
