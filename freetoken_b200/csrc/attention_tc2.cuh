// The tcgen05 attention kernel for long steps with two query tiles per CTA.  Included by attention.cu
// after attention_tc.cuh, whose helpers, sizes and status words it uses.
//
// A piece of work is 256 query rows of one KV head: two tiles A and B of 128 rows (the `group` heads of
// 128 / group consecutive tokens each), which read the same keys and values.  Each tile has its own
// four softmax warps, its own scores S and output O in TMEM (4 x 128 columns), and writes its
// probabilities as bfloat16 over the first 64 columns of its own S.  One warp issues the products in
// the order
//     S_A(0) S_B(0) | O_A+=P_A(0)V(0)  S_A(1)  O_B+=P_B(0)V(0)  S_B(1) | O_A+=P_A(1)V(1) ...
// so the tensor pipe works on one tile's products while the other tile's softmax runs: with one tile
// per CTA the chain scores -> softmax -> probabilities -> product left the pipe idle two thirds of the time.
// The pipe executes a thread's products in the order of issue, which is what allows S_X(j + 1) to
// overwrite S_X(j) / P_X(j) right after the product that read P_X(j) was issued.
//
// Everything else is as in the one-tile kernel: keys and values come from the pages by TMA in tiles
// of 128 keys (two stages), value rows past the end of the request are zeroed before the product,
// one CTA per SM works through its share of the work list, every wait is bounded.
#pragma once
#include "attention_tc.cuh"

namespace ftk {

// The softmax warps take the registers that the loading and issuing warps do not need (a warpgroup = four
// consecutive warps changes its share together).
template <int N> __device__ __forceinline__ void regs_give() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void regs_take() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

constexpr int kTc2Stages = 2;                                    // key and value tiles in flight
constexpr int kTc2Threads = 384;                                  // a warpgroup of 2 loaders + 1 MMA (+ 1 idle), 2 x 4 softmax warps
constexpr int kTc2RegsFew = 72, kTc2RegsMany = 216;                // of 384 x 168: what 128 threads give, 256 take
constexpr int kTc2Smem = (2 + 2 * kTc2Stages) * kTcTile + 1024;    // Q_A, Q_B, K and V stages

__global__ void __launch_bounds__(kTc2Threads, 1)
attention_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ unsigned char dyn_smem[];
  __shared__ uint64_t q_full, q_empty, o_free[2], k_full[kTc2Stages], k_empty[kTc2Stages], v_full[kTc2Stages],
      v_empty[kTc2Stages], s_full[2], p_full[2], pv_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_work = p.n_items * p.Hkv;
  const int n_rounds = (n_work + (int)gridDim.x - 1) / (int)gridDim.x;
  auto piece = [&](int i) {  // rounds run to and fro over the CTAs: the list is sorted by length
    return i * (int)gridDim.x + ((i & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };
  const uint32_t base = (smem_addr(dyn_smem) + 1023u) & ~1023u;
  unsigned char* tiles = dyn_smem + (base - smem_addr(dyn_smem));
  const uint32_t q_s = base, k_s = base + 2 * kTcTile, v_s = base + (2 + kTc2Stages) * kTcTile;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    mbar_init(&q_empty, 1);
    for (int s = 0; s < kTc2Stages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&s_full[x], 1); mbar_init(&p_full[x], 4);
      mbar_init(&pv_done[x], 1); mbar_init(&o_free[x], 4);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();  // set up while the kernel before this one still runs; what it wrote is read from here on
  pdl_trigger();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;
  const int G = p.G;
  const int tpt = kTcRows / G;  // tokens of one tile
  auto tiles_of = [](const Item& it) { return it.ok ? (it.ke - it.kb + kTcKeys - 1) / kTcKeys : 0; };
  auto fail = [&](int code) {
    atomicCAS(&g_attn_status[0], 0, code);
    abort_flag = 1;
  };

  if (warp < 4) {
  regs_give<kTc2RegsFew>();  // (warp 3 only fills the warpgroup)
  if (warp == 0 || warp == 2) {
    // ------------------------------------------------------------ TMA producers: warp 0 keys (and queries), warp 2 values
    if (lane < 16) {
      const int kv = warp == 2, box = lane >> 1, h = lane & 1;
      const CUtensorMap* map = kv ? &map_v : &map_k;
      uint64_t* full = kv ? v_full : k_full;
      uint64_t* empty = kv ? v_empty : k_empty;
      unsigned char* stage0 = tiles + (kv ? 2 + kTc2Stages : 2) * kTcTile + h * kTcHalf + box * 2048;
      bool ok = true;
      int g = 0;   // key tiles of all pieces so far
      int qi = 0;  // pieces with tiles so far
      for (int i_round = 0; i_round < n_rounds && ok; ++i_round) {
        const int w = piece(i_round);
        if (w >= n_work) continue;
        const Item it = load_item(p, p.n_items - 1 - w / p.Hkv);
        const int kvh = w % p.Hkv;
        const int n_tiles = tiles_of(it);
        if (n_tiles == 0) continue;
        if (!kv) {  // the queries, once the products of the piece before have read theirs
          if (!__all_sync(0x0000ffffu, mbar_wait(&q_empty, (uint32_t)(qi & 1) ^ 1u, abortp))) {
            if (lane == 0) fail(310);
            ok = false;
            break;
          }
          if (lane == 0) {
            const int n_q = it.ntok > tpt ? 2 : 1;  // tile B only when the piece has tokens for it
            mbar_expect_tx(&q_full, (uint32_t)(n_q * 2 * 128 * G * tpt));
            for (int x = 0; x < n_q; ++x)
              for (int hh = 0; hh < 2; ++hh)  // (d, head, token): rows land as token-major, head-minor
                tma_load_3d(tiles + x * kTcTile + hh * kTcHalf, &map_q, &q_full, hh * 64, kvh * G,
                            it.q_start + it.tok0 + x * tpt);
          }
        }
        ++qi;
        const int32_t* bt = p.block_table + (size_t)it.bt_row * p.bt_stride;
        for (int j = 0; j < n_tiles && ok; ++j, ++g) {
          const int st = g % kTc2Stages;
          const uint32_t par = ((g / kTc2Stages) & 1) ^ 1;
          const int key0 = it.kb + j * kTcKeys;
          const int n_box = min(8, (it.ke - key0 + 15) >> 4);  // boxes of 16 keys that hold keys of the request
          const int key = key0 + 16 * box;
          int page = 0;
          if (box < n_box) {
            const int slot = key / p.P;
            page = slot < p.bt_stride ? bt[slot] : 0;
            if (page < 0 || page >= p.num_pages) page = 0;
          }
          const int row = (page * p.Hkv + kvh) * p.P + key % p.P;
          if (!__all_sync(0x0000ffffu, mbar_wait(&empty[st], par, abortp))) {
            if (lane == 0) fail(301 + kv);
            ok = false;
            break;
          }
          if (lane == 0) mbar_expect_tx(&full[st], (uint32_t)n_box * 2 * 2048);
          __syncwarp(0x0000ffffu);
          if (box < n_box) tma_load_2d(stage0 + st * kTcTile, map, &full[st], h * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (lane 0); the warp zeroes value rows past the end
    constexpr uint32_t idesc_qk = instr_desc(kTcKeys);
    constexpr uint32_t idesc_pv = instr_desc(kTcD) | (1u << 16);  // B (values) MN-major
    bool ok = true;
    int g0 = 0;  // key tiles of the pieces before this one
    int qi = 0;  // pieces with tiles before this one
    int gx[2] = {0, 0};  // key tiles that query tile x has worked through, pieces it took part in
    int px[2] = {0, 0};
    for (int i_round = 0; i_round < n_rounds && ok; ++i_round) {
      const int w = piece(i_round);
      if (w >= n_work) continue;
      const Item it = load_item(p, p.n_items - 1 - w / p.Hkv);
      const int n_tiles = tiles_of(it);
      if (n_tiles == 0) continue;
      const int n_q = it.ntok > tpt ? 2 : 1;
      if (!mbar_wait(&q_full, (uint32_t)(qi & 1), abortp)) {
        if (lane == 0) fail(303);
        ok = false;
        break;
      }
      // S_x(j) = Q_x K(j)^T; after the last tile's scores of the last query tile the key stage and, at the end of
      // the piece, the queries are given back
      auto scores = [&](int x, int j) -> bool {
        const int g = g0 + j, ks = g % kTc2Stages;
        if (x == 0 && !mbar_wait(&k_full[ks], (uint32_t)(g / kTc2Stages) & 1u, abortp)) return false;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t d = tmem + (uint32_t)(x * kTcKeys);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {  // 16 elements of the head dimension per MMA
            const uint64_t a = smem_desc(q_s + x * kTcTile + (kk >> 2) * kTcHalf) + 2 * (kk & 3);
            const uint64_t b = smem_desc(k_s + ks * kTcTile + (kk >> 2) * kTcHalf) + 2 * (kk & 3);
            tc_mma(d, a, b, idesc_qk, kk != 0);
          }
          tc_commit(&s_full[x]);
          if (x == n_q - 1) {
            tc_commit(&k_empty[ks]);
            if (j == n_tiles - 1) tc_commit(&q_empty);
          }
        }
        __syncwarp();
        return true;
      };
      // O_x += P_x(j) V(j); the first of a piece waits until the piece before has read its output
      auto product = [&](int x, int j) -> bool {
        const int g = g0 + j, vs = g % kTc2Stages;
        if (!mbar_wait(&p_full[x], (uint32_t)((gx[x] + j) & 1), abortp)) return false;
        if (x == 0) {
          if (!mbar_wait(&v_full[vs], (uint32_t)(g / kTc2Stages) & 1u, abortp)) return false;
          const int live = it.ke - (it.kb + j * kTcKeys);  // keys of the request in this tile
          if (live < kTcKeys) {
            // the value rows past the end of the request: zero, whatever the page holds there and
            // whatever the stage held before
            for (int z = lane; z < (kTcKeys - live) * 16; z += 32) {
              const int r = live + z / 16, h = (z / 8) & 1, c = z & 7;
              *reinterpret_cast<uint4*>(tiles + (2 + kTc2Stages + vs) * kTcTile + h * kTcHalf + r * 128 + c * 16) =
                  make_uint4(0u, 0u, 0u, 0u);
            }
            fence_async_smem();
          }
        }
        if (j == 0 && !mbar_wait(&o_free[x], (uint32_t)(px[x] & 1) ^ 1u, abortp)) return false;
        __syncwarp();
        tc_fence_after();
        if (lane == 0) {
          const uint32_t d = tmem + (uint32_t)((2 + x) * kTcKeys);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {  // 16 keys per MMA
            const uint32_t a = tmem + (uint32_t)(x * kTcKeys + kk * 8);
            const uint64_t b = smem_desc_mn(v_s + vs * kTcTile + kk * 2048, kTcHalf);
            tc_mma_ts(d, a, b, idesc_pv, (j | kk) != 0);
          }
          tc_commit(&pv_done[x]);
          if (x == n_q - 1) tc_commit(&v_empty[vs]);
        }
        __syncwarp();
        return true;
      };
      for (int x = 0; x < n_q && ok; ++x) ok = scores(x, 0);
      for (int j = 0; j < n_tiles && ok; ++j)
        for (int x = 0; x < n_q && ok; ++x) {
          ok = product(x, j);
          if (ok && j + 1 < n_tiles) ok = scores(x, j + 1);
        }
      if (!ok) {
        if (lane == 0) fail(304);
        break;
      }
      g0 += n_tiles;
      ++qi;
      for (int x = 0; x < n_q; ++x) {
        gx[x] += n_tiles;
        ++px[x];
      }
    }
  }
  } else {
    regs_take<kTc2RegsMany>();
    // ------------------------------------------------------------ softmax and epilogue: warps 4..7 tile A, warps 8..11 tile B
    const int X = warp < 8 ? 0 : 1;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;           // row of the tile = TMEM lane
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + (uint32_t)(X * kTcKeys);        // scores, then probabilities over their first half
    const uint32_t o_addr = lane_addr + (uint32_t)((2 + X) * kTcKeys);  // output
    bool ok = true;
    int gx = 0;  // key tiles this query tile has worked through
    for (int i_round = 0; i_round < n_rounds && ok; ++i_round) {
      const int w = piece(i_round);
      if (w >= n_work) continue;
      const Item it = load_item(p, p.n_items - 1 - w / p.Hkv);
      const int kvh = w % p.Hkv;
      const int n_tiles = tiles_of(it);
      const int ntok = it.ok ? min(tpt, it.ntok - X * tpt) : 0;  // tokens of this query tile
      if (ntok <= 0) continue;
      const int R = ntok * G;
      const int pos_base = it.kv_len - it.q_len + it.tok0 + X * tpt;
      const int qpos = r < R ? pos_base + r / G : -1;
      // last key this row may read; rows past the tile's last are never stored and must not hold the others up
      const int hi = r < R ? min(it.ke - 1, qpos) : 0x7fffffff;
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int g = gx + j;
        if (!__all_sync(0xffffffffu, mbar_wait(&s_full[X], (uint32_t)(g & 1), abortp))) {
          if (lane == 0) fail(306);
          ok = false;
          break;
        }
        tc_fence_after();
        const int key0 = it.kb + j * kTcKeys;
        // the row's 128 scores, in registers for both passes (the largest, then the probabilities)
        float v[128];
        tmem_ld32_start(s_addr, v);
        tmem_ld32_start(s_addr + 32, v + 32);
        tmem_ld32_start(s_addr + 64, v + 64);
        tmem_ld32_start(s_addr + 96, v + 96);
        tmem_ld_wait();
        // a tile that every row of the warp reads in full needs no mask (most tiles of a long prompt)
        const bool interior = __all_sync(0xffffffffu, key0 + kTcKeys - 1 <= hi);
        if (!interior) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (key0 + i > hi) v[i] = -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
          mx4[0] = fmaxf(mx4[0], v[i]);
          mx4[1] = fmaxf(mx4[1], v[i + 1]);
          mx4[2] = fmaxf(mx4[2], v[i + 2]);
          mx4[3] = fmaxf(mx4[3], v[i + 3]);
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        mx *= sl2;  // the scale is positive: the largest score stays the largest
        // move the running maximum only when it grew by more than 8 (or is not set yet)
        float alpha = 1.f;
        if (mx > m_used + 8.f || (m_used == -INFINITY && mx > -INFINITY)) {
          alpha = m_used == -INFINITY ? 0.f : tc_exp2(m_used - mx);
          m_used = mx;
        }
        l *= alpha;
        if (__any_sync(0xffffffffu, alpha != 1.f) && j > 0) {  // O must hold every product so far before it is scaled
          if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[X], (uint32_t)((g - 1) & 1), abortp))) {
            if (lane == 0) fail(309);
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float o[32];
            tmem_ld32(o_addr + c * 32, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32(o_addr + c * 32, o);
          }
        }
        const float mb = m_used == -INFINITY ? 0.f : m_used;
        float sum = 0.f;
        // probabilities as bfloat16 over the first 64 columns of the scores (which are all in registers by now)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = tc_exp2(fmaf(v[c * 32 + i], sl2, -mb));  // exp2(-inf) = 0 for masked keys
            const float p1 = tc_exp2(fmaf(v[c * 32 + i + 1], sl2, -mb));
            sum += p0 + p1;
            pk[i >> 1] = tc_pack(p0, p1);
          }
          tmem_st16u(s_addr + (uint32_t)(c * 16), pk);
        }
        l += sum;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[X]);
      }
      // ---- epilogue
      if (ok && n_tiles > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[X], (uint32_t)((gx + n_tiles - 1) & 1), abortp))) {
          if (lane == 0) fail(308);
          ok = false;
        }
        tc_fence_after();
      }
      if (ok) {
        const bool live = n_tiles > 0;
        const int tok = it.q_start + it.tok0 + X * tpt + r / G;
        if (it.nsplit == 1) {
          const float inv = l > 0.f ? 1.f / l : 0.f;
          __nv_bfloat16* dst = (__nv_bfloat16*)p.out + ((size_t)tok * p.Hq + kvh * G + r % G) * kTcD;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float o[32];
            if (live) tmem_ld32(o_addr + c * 32, o);
            if (r < R) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                uint4 pk;
                pk.x = tc_pack(live ? o[8 * q4] * inv : 0.f, live ? o[8 * q4 + 1] * inv : 0.f);
                pk.y = tc_pack(live ? o[8 * q4 + 2] * inv : 0.f, live ? o[8 * q4 + 3] * inv : 0.f);
                pk.z = tc_pack(live ? o[8 * q4 + 4] * inv : 0.f, live ? o[8 * q4 + 5] * inv : 0.f);
                pk.w = tc_pack(live ? o[8 * q4 + 6] * inv : 0.f, live ? o[8 * q4 + 7] * inv : 0.f);
                *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = pk;
              }
            }
          }
        } else {
          // the rows of tile B follow those of tile A in the piece's slot of partial sums
          const size_t slot = ((size_t)(it.base + it.split) * p.Hkv + kvh) * p.tile_rows + X * tpt * G + r;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float o[32];
            if (live) tmem_ld32(o_addr + c * 32, o);
            if (r < R) {
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4)
                *reinterpret_cast<float4*>(p.part_o + slot * kTcD + c * 32 + q4 * 4) =
                    live ? make_float4(o[4 * q4], o[4 * q4 + 1], o[4 * q4 + 2], o[4 * q4 + 3]) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
          if (r < R) {
            p.part_ml[slot * 2] = m_used == -INFINITY ? -INFINITY : m_used * 0.6931471805599453f;
            p.part_ml[slot * 2 + 1] = l;
          }
        }
      }
      if (n_tiles > 0) {  // the output accumulator has been read: the next piece's first product may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_free[X]);
      }
      gx += n_tiles;
    }
  }
  // ---------------------------------------------------------------- teardown
  if (abort_flag) {
    if (threadIdx.x == 0) g_attn_status[1] = blockIdx.x;
    for (int i = 0; i < 2000; ++i) __nanosleep(100);  // let copies in flight land before the CTA leaves
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// 256 query rows per piece of work; otherwise what the one-tile kernel takes.
inline int launch_attention_tc2(const AttnParams& p, int n_tokens, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTc2Smem) != cudaSuccess)
      return 2;
    configured = true;
  }
  CUtensorMap mq, mk, mv;
  {
    // queries [T, Hq, D] seen as (d, head, token); a box is (64, group, tokens per tile)
    const uint64_t dims[3] = {(uint64_t)kTcD, (uint64_t)p.Hq, (uint64_t)n_tokens};
    const uint64_t strides[2] = {(uint64_t)kTcD * 2, (uint64_t)p.Hq * kTcD * 2};
    const uint32_t box[3] = {64, (uint32_t)p.G, (uint32_t)(kTcRows / p.G)};
    if (!make_map(&mq, p.q, 3, dims, strides, box)) return 4;
  }
  {
    // a slab [pages, Hkv, P, D] seen as rows of D; a box is 16 rows of one page x 64 elements
    const uint64_t dims[2] = {(uint64_t)kTcD, (uint64_t)p.num_pages * p.Hkv * p.P};
    const uint64_t strides[1] = {(uint64_t)kTcD * 2};
    const uint32_t box[2] = {64, 16};
    if (!make_map(&mk, p.k, 2, dims, strides, box) || !make_map(&mv, p.v, 2, dims, strides, box)) return 4;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 1;
  }
  const long long n_work = (long long)p.n_items * p.Hkv;
  const int grid = (int)(n_work < sms ? n_work : sms);
  FTK_LAUNCH(attention_tc2_kernel, grid, kTc2Threads, kTc2Smem, s, mq, mk, mv, p);
  return 0;
}

}  // namespace ftk
