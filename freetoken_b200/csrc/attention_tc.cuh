// Paged causal attention on the 5th-generation tensor cores (tcgen05), bfloat16, head size 128: long
// steps and decode steps.  Included by attention.cu after AttnParams / Item / load_item.
//
// A tile is 128 query rows: the `group` query heads of one KV head for 128 / group consecutive tokens
// of one segment, so a key/value tile is read once for all the heads that share it (a decode step
// fills only the first `group` rows).  Keys come in tiles of 128.  Per key tile:
//   S = Q K^T        tcgen05.mma, Q [128 x 128] and K [128 keys x 128] K-major in shared memory
//                    (TMA, 128-byte swizzle; K straight from the pages, 16 keys per box), S in TMEM
//                    (two buffers, so the next tile's product runs under this tile's softmax);
//   softmax          one thread per row (its TMEM lane): scale, mask, running maximum, exp2, sum; the
//                    probabilities go back to TMEM as bfloat16 (two buffers of 64 columns).  The
//                    running maximum is only moved when it grew by more than 8 (a factor 256), so the
//                    accumulator is rescaled a few times per row, not once per tile;
//   O += P V         tcgen05.mma with P as the A operand in TMEM and V as the MN-major B operand (the
//                    page rows as they are, three stages like the keys), O in TMEM.
// One CTA per SM = 7 warps: warps 0 and 6 issue the TMA loads of keys and values, warp 1 the MMAs, warps
// 2-5 are the softmax (and the epilogue: O / l to the output, or the partial sums of a split tile for
// the merge kernel).  A CTA works through its share of the work list; the three roles run through it on
// their own, so the loads and the first product of a piece run under the end of the piece before.
// Decode steps (FEW = true) have at most 16 live rows in a tile: `group` query heads of one or a few
// tokens.  A row per thread would leave one thread per live row with 128 exponentials a key tile, which
// then sets the pace (1.5 us a tile, 45 GB/s per SM).  There, ONE warp takes rows 0-15 with the
// 16-lane shapes of tcgen05.ld / st, which spread a row's columns over four threads (the layout of an
// mma.sync accumulator fragment); the other three softmax warps have nothing to do.
// Every wait is bounded; a timeout records a code in g_attn_status, lets copies land, frees TMEM, returns.
// Value rows past the end of the request are never multiplied as they lie in memory (they may hold
// anything): whole 16-key boxes past the end are not loaded, and all rows of the stage past the end
// are zeroed in shared memory before the product.
//
// The reference's prefill attention is a Triton kernel (python/freetoken/kernel/triton/attention.py:469-880).
#pragma once
#include "tc_common.cuh"

namespace ftk {

__device__ int g_attn_status[4];  // [0] first error code, [1] block; 0 = fine

constexpr int kTcRows = 128;
constexpr int kTcKeys = 128;
constexpr int kTcD = 128;
constexpr int kTcThreads = 224;
constexpr int kTcHalf = 128 * 64 * 2;       // bytes of a [128 rows x 64 elements] swizzle-atom column
constexpr int kTcTile = 2 * kTcHalf;        // a [128 x 128] bfloat16 tile
constexpr int kTcStages = 3;                // key and value tiles in flight
constexpr int kTcSmem = (1 + 2 * kTcStages) * kTcTile + 1024;  // Q, K and V stages
constexpr int kTcPCol = 3 * kTcKeys;        // tensor memory: S x2 (128 columns each), O (128), P x2 (64 each)

__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 consecutive columns of this thread's row in one load; completed by tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_start(uint32_t addr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr) : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// sixteen 32-bit words of this thread's row into columns [addr, addr + 16); completed by tmem_st_wait()
__device__ __forceinline__ void tmem_st16u(uint32_t addr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
// Rows 0-15 of the warp's quadrant, 32 columns from `addr`: thread t gets rows t / 4 and t / 4 + 8; of the
// i-th group of 8 columns it holds columns 8 i + 2 (t % 4) and the next one: r[4 i], r[4 i + 1] of its
// first row and r[4 i + 2], r[4 i + 3] of its second.  Completed by tmem_ld_wait().
__device__ __forceinline__ void tmem_ld_16rows_32cols(uint32_t addr, float* r) {
  uint32_t u[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
        "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(addr) : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_16rows_32cols(uint32_t addr, const float* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(addr), "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])),
        "r"(__float_as_uint(r[3])), "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])),
        "r"(__float_as_uint(r[7])), "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])),
        "r"(__float_as_uint(r[11])), "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])),
        "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15]))
      : "memory");
}
// The same rows, sixteen 32-bit columns from `addr` (the probabilities as bfloat16 pairs): of the i-th
// group of 4 columns thread t holds column 4 i + t % 4: w[2 i] of its first row, w[2 i + 1] of its second.
__device__ __forceinline__ void tmem_st_16rows_16words(uint32_t addr, const uint32_t* w) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory descriptor of an MN-major operand with 128-byte swizzle: 64 elements of the MN side
// are contiguous (128 bytes), eight k rows make a 1024-byte group (stride byte offset), the next 64
// MN elements lie `lbo` bytes further (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo >> 4) & 0x3fff) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ float tc_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t tc_pack(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// Softmax and epilogue of a tile's rows 0..15 by one warp (the warp of TMEM lanes 0..31), for tiles
// that have no more rows: thread t has rows t / 4 and t / 4 + 8 and a quarter of their columns.
__device__ __forceinline__ void attention_tc_few_rows(const AttnParams& p, uint32_t tmem, int lane, int n_work, int n_rounds,
                                                      uint64_t* s_full, uint64_t* s_empty, uint64_t* p_full,
                                                      uint64_t* pv_done, uint64_t* o_free, volatile int* abortp,
                                                      int* abort_flag) {
  const int G = p.G;
  const float sl2 = p.scale * 1.4426950408889634f;
  const int ra = lane >> 2, rb = ra + 8, cq = lane & 3;
  auto fail = [&](int code) {
    atomicCAS(&g_attn_status[0], 0, code);
    *abort_flag = 1;
  };
  bool ok = true;
  int g0 = 0;  // tiles of the pieces before this one
  for (int i_round = 0; i_round < n_rounds && ok; ++i_round) {
    const int w = i_round * (int)gridDim.x + ((i_round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
    if (w >= n_work) continue;
    const Item it = load_item(p, p.n_items - 1 - w / p.Hkv);
    const int kvh = w % p.Hkv;
    const int n_tiles = it.ok ? (it.ke - it.kb + kTcKeys - 1) / kTcKeys : 0;
    const int R = it.ok ? it.ntok * G : 0;
    const int pos_base = it.kv_len - it.q_len + it.tok0;
    // last key a row may read; rows that the tile does not have are never stored and need no mask
    const int hi_a = ra < R ? min(it.ke - 1, pos_base + ra / G) : 0x7fffffff;
    const int hi_b = rb < R ? min(it.ke - 1, pos_base + rb / G) : 0x7fffffff;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int g = g0 + j, sb = g & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (uint32_t)((g >> 1) & 1), abortp))) {
        if (lane == 0) fail(206);
        ok = false;
        break;
      }
      tc_fence_after();
      float v[64];
#pragma unroll
      for (int k = 0; k < 4; ++k) tmem_ld_16rows_32cols(tmem + (uint32_t)(sb * kTcKeys + 32 * k), v + 16 * k);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);  // the next product may overwrite this buffer
      const int key0 = it.kb + j * kTcKeys;
      const bool interior = __all_sync(0xffffffffu, key0 + kTcKeys - 1 <= min(hi_a, hi_b));
      if (!interior) {
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const int c = key0 + 8 * q + 2 * cq;
          if (c > hi_a) v[4 * q] = -INFINITY;
          if (c + 1 > hi_a) v[4 * q + 1] = -INFINITY;
          if (c > hi_b) v[4 * q + 2] = -INFINITY;
          if (c + 1 > hi_b) v[4 * q + 3] = -INFINITY;
        }
      }
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        mx_a = fmaxf(mx_a, fmaxf(v[4 * q], v[4 * q + 1]));
        mx_b = fmaxf(mx_b, fmaxf(v[4 * q + 2], v[4 * q + 3]));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2)) * sl2;  // the scale is positive
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2)) * sl2;
      // move a row's running maximum only when it grew by more than 8 (or is not set yet)
      float al_a = 1.f, al_b = 1.f;
      if (mx_a > m_a + 8.f || (m_a == -INFINITY && mx_a > -INFINITY)) {
        al_a = m_a == -INFINITY ? 0.f : tc_exp2(m_a - mx_a);
        m_a = mx_a;
      }
      if (mx_b > m_b + 8.f || (m_b == -INFINITY && mx_b > -INFINITY)) {
        al_b = m_b == -INFINITY ? 0.f : tc_exp2(m_b - mx_b);
        m_b = mx_b;
      }
      l_a *= al_a;
      l_b *= al_b;
      const bool rescale = __any_sync(0xffffffffu, al_a != 1.f || al_b != 1.f) && j > 0;
      if (g >= 2) {  // the product two tiles back has read the P buffer this tile writes
        if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[sb], (uint32_t)(((g - 2) >> 1) & 1), abortp))) {
          if (lane == 0) fail(207);
          ok = false;
          break;
        }
      }
      if (rescale) {  // O must hold every product so far before it is scaled
        if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[sb ^ 1], (uint32_t)(((g - 1) >> 1) & 1), abortp))) {
          if (lane == 0) fail(209);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int k = 0; k < 4; ++k) {
          float o[16];
          tmem_ld_16rows_32cols(tmem + (uint32_t)(2 * kTcKeys + 32 * k), o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            o[4 * i] *= al_a; o[4 * i + 1] *= al_a;
            o[4 * i + 2] *= al_b; o[4 * i + 3] *= al_b;
          }
          tmem_st_16rows_32cols(tmem + (uint32_t)(2 * kTcKeys + 32 * k), o);
        }
        tmem_st_wait();
      }
      const float mb_a = m_a == -INFINITY ? 0.f : m_a, mb_b = m_b == -INFINITY ? 0.f : m_b;
      float sum_a = 0.f, sum_b = 0.f;
      // probabilities as bfloat16 pairs into rows 0..15 of the A operand in tensor memory
      const uint32_t p_addr = tmem + (uint32_t)(kTcPCol + sb * (kTcKeys / 2));
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint32_t wds[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int x = 16 * k + 4 * i;
          const float a0 = tc_exp2(fmaf(v[x], sl2, -mb_a)), a1 = tc_exp2(fmaf(v[x + 1], sl2, -mb_a));  // exp2(-inf) = 0
          const float b0 = tc_exp2(fmaf(v[x + 2], sl2, -mb_b)), b1 = tc_exp2(fmaf(v[x + 3], sl2, -mb_b));
          sum_a += a0 + a1;
          sum_b += b0 + b1;
          wds[2 * i] = tc_pack(a0, a1);
          wds[2 * i + 1] = tc_pack(b0, b1);
        }
        tmem_st_16rows_16words(p_addr + (uint32_t)(16 * k), wds);
      }
      l_a += sum_a;
      l_b += sum_b;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
    }
    if (!ok) break;
    // ---- epilogue
    if (n_tiles > 0) {
      const int gl = g0 + n_tiles - 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[gl & 1], (uint32_t)((gl >> 1) & 1), abortp))) {
        if (lane == 0) fail(208);
        ok = false;
        break;
      }
      tc_fence_after();
    }
    // a row's sum: over the four threads that share it
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (it.ok) {
      const bool live = n_tiles > 0;
      const float inv_a = live && l_a > 0.f ? 1.f / l_a : 0.f, inv_b = live && l_b > 0.f ? 1.f / l_b : 0.f;
      const int tok_a = it.q_start + it.tok0 + ra / G, tok_b = it.q_start + it.tok0 + rb / G;
      __nv_bfloat16* dst_a = (__nv_bfloat16*)p.out + ((size_t)tok_a * p.Hq + kvh * G + ra % G) * kTcD;
      __nv_bfloat16* dst_b = (__nv_bfloat16*)p.out + ((size_t)tok_b * p.Hq + kvh * G + rb % G) * kTcD;
      const size_t slot0 = ((size_t)(it.base + it.split) * p.Hkv + kvh) * p.tile_rows;
#pragma unroll 1
      for (int k = 0; k < 4; ++k) {
        float o[16];
        if (live) {
          tmem_ld_16rows_32cols(tmem + (uint32_t)(2 * kTcKeys + 32 * k), o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = 32 * k + 8 * i + 2 * cq;
          if (it.nsplit == 1) {
            if (ra < R) *reinterpret_cast<uint32_t*>(dst_a + col) = tc_pack(o[4 * i] * inv_a, o[4 * i + 1] * inv_a);
            if (rb < R) *reinterpret_cast<uint32_t*>(dst_b + col) = tc_pack(o[4 * i + 2] * inv_b, o[4 * i + 3] * inv_b);
          } else {
            if (ra < R) *reinterpret_cast<float2*>(p.part_o + (slot0 + ra) * kTcD + col) = make_float2(o[4 * i], o[4 * i + 1]);
            if (rb < R) *reinterpret_cast<float2*>(p.part_o + (slot0 + rb) * kTcD + col) = make_float2(o[4 * i + 2], o[4 * i + 3]);
          }
        }
      }
      if (it.nsplit > 1 && cq == 0) {
        if (ra < R) {
          p.part_ml[(slot0 + ra) * 2] = m_a == -INFINITY ? -INFINITY : m_a * 0.6931471805599453f;
          p.part_ml[(slot0 + ra) * 2 + 1] = live ? l_a : 0.f;
        }
        if (rb < R) {
          p.part_ml[(slot0 + rb) * 2] = m_b == -INFINITY ? -INFINITY : m_b * 0.6931471805599453f;
          p.part_ml[(slot0 + rb) * 2 + 1] = live ? l_b : 0.f;
        }
      }
    }
    if (n_tiles > 0) {  // the output accumulator has been read: the next piece's first product may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
    }
    g0 += n_tiles;
  }
}

template <bool FEW>
__global__ void __launch_bounds__(kTcThreads)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ unsigned char dyn_smem[];
  __shared__ uint64_t q_full, q_empty, o_free, k_full[kTcStages], k_empty[kTcStages], v_full[kTcStages], v_empty[kTcStages], s_full[2], s_empty[2],
      p_full[2], pv_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A CTA works through one piece of work of every round of gridDim.x pieces: piece w is the tile
  // (or part of a tile) n_items - 1 - w / Hkv (long tiles first: they grow with the token index) for
  // KV head w % Hkv.  The three roles below run through the same pieces on their own, held together
  // only by the barriers, so the loads and the first product of a piece run under the end of the one before.
  // Rounds run to and fro over the CTAs (the work is sorted by length, so the CTA that gets the longest
  // piece of one round gets the shortest of the next).
  const int n_work = p.n_items * p.Hkv;
  const int n_rounds = (n_work + (int)gridDim.x - 1) / (int)gridDim.x;
  auto piece = [&](int i) {
    return i * (int)gridDim.x + ((i & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };
  const uint32_t base = (smem_addr(dyn_smem) + 1023u) & ~1023u;
  unsigned char* tiles = dyn_smem + (base - smem_addr(dyn_smem));
  const uint32_t q_s = base, k_s = base + kTcTile, v_s = base + (1 + kTcStages) * kTcTile;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    mbar_init(&q_empty, 1);
    mbar_init(&o_free, FEW ? 1 : 4);
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], FEW ? 1 : 4);
      mbar_init(&p_full[s], FEW ? 1 : 4); mbar_init(&pv_done[s], 1);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (FEW) {  // query rows that no load writes must not hold whatever the kernel before left there
    for (int i = threadIdx.x; i < kTcTile / 16; i += kTcThreads) reinterpret_cast<uint4*>(tiles)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Barriers and TMEM are set up while the kernel before this one still runs; what it wrote (queries,
  // the new keys and values) is read after pdl_wait().  In the form for decode steps the loader warps do
  // not wait there: the work list, the block tables and the keys and values of earlier steps were
  // written by kernels that had ended before this one could start (every kernel of a step waits for the
  // one before it before it lets the next one in, or ends), so they wait only before the queries and
  // before a key tile that holds positions of this step.
  if (!FEW || (warp != 0 && warp != 6)) pdl_wait();
  if (!FEW || warp == 1) pdl_trigger();  // (after a wait: the kernel after this one may count on the one before being over)
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;
  const int G = p.G;
  auto tiles_of = [](const Item& it) { return it.ok ? (it.ke - it.kb + kTcKeys - 1) / kTcKeys : 0; };
  auto fail = [&](int code) {
    atomicCAS(&g_attn_status[0], 0, code);
    abort_flag = 1;
  };

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------ TMA producers: warp 0 keys, warp 6 values
    // One lane per box: lane = 2 * (16-key box of the tile) + (half of the head dimension), so one
    // warp instruction issues a whole tile and every lane looks its own page up.  (One thread issuing
    // the boxes of a tile one after the other took longer than the tile's products; keys and values in
    // one warp made the keys wait for the value stage.)
    if (lane < 16) {
      const int kv = warp == 6, box = lane >> 1, h = lane & 1;
      const CUtensorMap* map = kv ? &map_v : &map_k;
      uint64_t* full = kv ? v_full : k_full;
      uint64_t* empty = kv ? v_empty : k_empty;
      unsigned char* stage0 = tiles + (kv ? 1 + kTcStages : 1) * kTcTile + h * kTcHalf + box * 2048;
      bool ok = true;
      bool waited = false;  // for the kernel before this one (decode steps)
      int g = 0;   // tiles of all pieces so far: stage g & 1
      int qi = 0;  // pieces with tiles so far
      for (int i_round = 0; i_round < n_rounds && ok; ++i_round) {
      const int w = piece(i_round);
      if (w >= n_work) continue;
        const Item it = load_item(p, p.n_items - 1 - w / p.Hkv);
        const int kvh = w % p.Hkv;
        const int n_tiles = tiles_of(it);
        if (n_tiles == 0) continue;
        // the queries go out once the products of the piece before have read theirs: before the first key
        // tile, or (decode steps) after the key tiles that may go out before the kernel before this one is over
        auto load_queries = [&]() -> bool {
          if (!__all_sync(0x0000ffffu, mbar_wait(&q_empty, (uint32_t)(qi & 1) ^ 1u, abortp))) {
            if (lane == 0) fail(210);
            return false;
          }
          if (lane == 0) {
            mbar_expect_tx(&q_full, (uint32_t)(2 * 128 * G * (p.tile_rows / G)));  // two boxes of (64, group, tokens per tile)
            for (int hh = 0; hh < 2; ++hh)  // (d, head, token): rows land as token-major, head-minor
              tma_load_3d(tiles + hh * kTcHalf, &map_q, &q_full, hh * 64, kvh * G, it.q_start + it.tok0);
          }
          return true;
        };
        const int q_at = FEW ? min(n_tiles - 1, 1) : 0;
        const int fresh_from = it.kv_len - it.q_len;  // first position that this step wrote
        const int32_t* bt = p.block_table + (size_t)it.bt_row * p.bt_stride;
        // this lane's page of tile j: looked up one tile ahead, so that the answer is there when the stage is free
        auto page_of = [&](int j) {
          const int key = it.kb + j * kTcKeys + 16 * box;
          int page = 0;
          if (j < n_tiles && key < it.ke) {
            const int slot = key / p.P;
            page = slot < p.bt_stride ? bt[slot] : 0;
            if (page < 0 || page >= p.num_pages) page = 0;
          }
          return page;
        };
        int page_next = page_of(0);
        for (int j = 0; j < n_tiles && ok; ++j, ++g) {
          const int st = g % kTcStages;
          const uint32_t par = ((g / kTcStages) & 1) ^ 1;
          const int key0 = it.kb + j * kTcKeys;
          const int n_box = min(8, (it.ke - key0 + 15) >> 4);  // boxes of 16 keys that hold keys of the request
          const int key = key0 + 16 * box;
          const int page = page_next;
          page_next = page_of(j + 1);
          const int row = (page * p.Hkv + kvh) * p.P + key % p.P;
          if (FEW && !waited && (key0 + kTcKeys > fresh_from || (!kv && j == q_at))) {
            pdl_wait();
            waited = true;
          }
          if (!kv && j == q_at && !load_queries()) {
            ok = false;
            break;
          }
          if (!__all_sync(0x0000ffffu, mbar_wait(&empty[st], par, abortp))) {
            if (lane == 0) fail(201 + kv);
            ok = false;
            break;
          }
          if (lane == 0) mbar_expect_tx(&full[st], (uint32_t)n_box * 2 * 2048);
          __syncwarp(0x0000ffffu);
          if (box < n_box) tma_load_2d(stage0 + st * kTcTile, map, &full[st], h * 64, row);
        }
        ++qi;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (lane 0); the warp zeroes value rows past the end
    constexpr uint32_t idesc_qk = instr_desc(kTcKeys);
    constexpr uint32_t idesc_pv = instr_desc(kTcD) | (1u << 16);  // B (values) MN-major
    bool ok = true;
    int g0 = 0;  // tiles of the pieces before this one
    int qi = 0;  // pieces with tiles before this one
    for (int i_round = 0; i_round < n_rounds && ok; ++i_round) {
      const int w = piece(i_round);
      if (w >= n_work) continue;
      const Item it = load_item(p, p.n_items - 1 - w / p.Hkv);
      const int n_tiles = tiles_of(it);
      if (n_tiles == 0) continue;
      if (!mbar_wait(&q_full, (uint32_t)(qi & 1), abortp)) {
        if (lane == 0) fail(203);
        ok = false;
        break;
      }
      for (int j = 0; j <= n_tiles && ok; ++j) {
        if (j < n_tiles) {
          const int g = g0 + j, st = g & 1, ks = g % kTcStages;  // score buffer, key stage
          const uint32_t par = (g >> 1) & 1;
          if (!mbar_wait2(&k_full[ks], (uint32_t)(g / kTcStages) & 1u, &s_empty[st], par ^ 1, abortp)) {
            if (lane == 0) fail(204);
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t d = tmem + (uint32_t)(st * kTcKeys);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // 16 elements of the head dimension per MMA
              const uint64_t a = smem_desc(q_s + (kk >> 2) * kTcHalf) + 2 * (kk & 3);
              const uint64_t b = smem_desc(k_s + ks * kTcTile + (kk >> 2) * kTcHalf) + 2 * (kk & 3);
              tc_mma(d, a, b, idesc_qk, kk != 0);
            }
            tc_commit(&k_empty[ks]);
            tc_commit(&s_full[st]);
            if (j == n_tiles - 1) tc_commit(&q_empty);  // the next piece's queries may come
          }
          __syncwarp();
        }
        if (j >= 1) {
          const int i = j - 1, g = g0 + i, st = g & 1, vs = g % kTcStages;  // probability buffer, value stage
          const uint32_t par = (g >> 1) & 1;
          if (!mbar_wait2(&p_full[st], par, &v_full[vs], (uint32_t)(g / kTcStages) & 1u, abortp) ||
              (i == 0 && !mbar_wait(&o_free, (uint32_t)(qi & 1) ^ 1u, abortp))) {  // the piece before has read its output
            if (lane == 0) fail(205);
            ok = false;
            break;
          }
          const int key0 = it.kb + i * kTcKeys;
          const int live = it.ke - key0;  // keys of the request in this tile
          if (live < kTcKeys) {
            // the value rows past the end of the request: zero, whatever the page holds there (the rest of
            // the last loaded box) and whatever the stage held before (boxes that were not loaded)
            for (int x = lane; x < (kTcKeys - live) * 16; x += 32) {
              const int r = live + x / 16, h = (x / 8) & 1, c = x & 7;
              *reinterpret_cast<uint4*>(tiles + (1 + kTcStages + vs) * kTcTile + h * kTcHalf + r * 128 + c * 16) =
                  make_uint4(0u, 0u, 0u, 0u);
            }
            fence_async_smem();
          }
          __syncwarp();
          tc_fence_after();
          if (lane == 0) {
            const uint32_t d = tmem + 2 * kTcKeys;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // 16 keys per MMA
              const uint32_t a = tmem + (uint32_t)(kTcPCol + st * (kTcKeys / 2) + kk * 8);
              const uint64_t b = smem_desc_mn(v_s + vs * kTcTile + kk * 2048, kTcHalf);
              tc_mma_ts(d, a, b, idesc_pv, (i | kk) != 0);
            }
            tc_commit(&v_empty[vs]);
            tc_commit(&pv_done[st]);
          }
          __syncwarp();
        }
      }
      g0 += n_tiles;
      ++qi;
    }
  } else if (FEW) {
    // ------------------------------------------------------------ softmax and epilogue of rows 0..15 by one warp
    if ((warp & 3) == 0) {
      attention_tc_few_rows(p, tmem, lane, n_work, n_rounds, s_full, s_empty, p_full, pv_done, &o_free, abortp, &abort_flag);
    }
  } else {
    // ------------------------------------------------------------ softmax and epilogue (warps 2..5), one row per thread
    const int quad = warp & 3;
    const int r = quad * 32 + lane;           // row of the tile = TMEM lane
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    bool ok = true;
    int g0 = 0;  // tiles of the pieces before this one
    for (int i_round = 0; i_round < n_rounds && ok; ++i_round) {
      const int w = piece(i_round);
      if (w >= n_work) continue;
    const Item it = load_item(p, p.n_items - 1 - w / p.Hkv);
    const int kvh = w % p.Hkv;
    const int n_tiles = tiles_of(it);
    const int R = it.ok ? it.ntok * G : 0;
    const int pos_base = it.kv_len - it.q_len + it.tok0;
    const int qpos = r < R ? pos_base + r / G : -1;
    // last key this row may read; rows past the tile's last are never stored and must not hold the others up
    const int hi = r < R ? min(it.ke - 1, qpos) : 0x7fffffff;
    float m_used = -INFINITY, l = 0.f;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int g = g0 + j, sb = g & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (uint32_t)((g >> 1) & 1), abortp))) {
        if (lane == 0) fail(206);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t s_addr = lane_addr + (uint32_t)(sb * kTcKeys);
      const int key0 = it.kb + j * kTcKeys;
      // the row's 128 scores, in registers for both passes
      float v0[32], v1[32], v2[32], v3[32];
      tmem_ld32_start(s_addr, v0);
      tmem_ld32_start(s_addr + 32, v1);
      tmem_ld32_start(s_addr + 64, v2);
      tmem_ld32_start(s_addr + 96, v3);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);  // the next product may overwrite this buffer
      // a tile that every row of the warp reads in full needs no mask (most tiles of a long prompt)
      const bool interior = __all_sync(0xffffffffu, key0 + kTcKeys - 1 <= hi);
      if (!interior) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (key0 + i > hi) v0[i] = -INFINITY;
          if (key0 + 32 + i > hi) v1[i] = -INFINITY;
          if (key0 + 64 + i > hi) v2[i] = -INFINITY;
          if (key0 + 96 + i > hi) v3[i] = -INFINITY;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(fmaxf(mx, v0[i]), fmaxf(v1[i], fmaxf(v2[i], v3[i])));
      mx *= sl2;  // the scale is positive: the largest score stays the largest
      // move the running maximum only when it grew by more than 8 (or is not set yet)
      float alpha = 1.f;
      if (mx > m_used + 8.f || (m_used == -INFINITY && mx > -INFINITY)) {
        alpha = m_used == -INFINITY ? 0.f : tc_exp2(m_used - mx);
        m_used = mx;
      }
      l *= alpha;
      const bool rescale = __any_sync(0xffffffffu, alpha != 1.f) && j > 0;
      if (g >= 2) {  // the product two tiles back has read the P buffer this tile writes
        if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[sb], (uint32_t)(((g - 2) >> 1) & 1), abortp))) {
          if (lane == 0) fail(207);
          ok = false;
          break;
        }
      }
      if (rescale) {  // O must hold every product so far before it is scaled
        if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[sb ^ 1], (uint32_t)(((g - 1) >> 1) & 1), abortp))) {
          if (lane == 0) fail(209);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float o[32];
          tmem_ld32(lane_addr + 2 * kTcKeys + c * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(lane_addr + 2 * kTcKeys + c * 32, o);
        }
      }
      const float mb = m_used == -INFINITY ? 0.f : m_used;
      float sum = 0.f;
      // probabilities as bfloat16 into this row of the A operand in tensor memory: two keys per 32-bit
      // column, 64 columns per buffer behind the output accumulator
      const uint32_t p_addr = lane_addr + (uint32_t)(kTcPCol + sb * (kTcKeys / 2));
      auto emit = [&](float (&v)[32], int c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = tc_exp2(fmaf(v[i], sl2, -mb));      // exp2(-inf) = 0 for masked keys
          const float p1 = tc_exp2(fmaf(v[i + 1], sl2, -mb));
          sum += p0 + p1;
          pk[i >> 1] = tc_pack(p0, p1);
        }
        tmem_st16u(p_addr + (uint32_t)(c * 16), pk);
      };
      emit(v0, 0);
      emit(v1, 1);
      emit(v2, 2);
      emit(v3, 3);
      l += sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
    }
    // ---- epilogue
    if (ok && n_tiles > 0) {
      const int gl = g0 + n_tiles - 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[gl & 1], (uint32_t)((gl >> 1) & 1), abortp))) {
        if (lane == 0) fail(208);
        ok = false;
      }
      tc_fence_after();
    }
    if (ok && it.ok) {
      const bool live = n_tiles > 0;
      const int tok = it.q_start + it.tok0 + r / G;
      if (it.nsplit == 1) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + ((size_t)tok * p.Hq + kvh * G + r % G) * kTcD;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float o[32];
          if (live) tmem_ld32(lane_addr + 2 * kTcKeys + c * 32, o);
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
        const size_t slot = ((size_t)(it.base + it.split) * p.Hkv + kvh) * p.tile_rows + r;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float o[32];
          if (live) tmem_ld32(lane_addr + 2 * kTcKeys + c * 32, o);
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
      if (lane == 0) mbar_arrive(&o_free);
    }
    g0 += n_tiles;
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

// What the kernel takes: bfloat16 heads of 128, pages of a multiple of 16 tokens, at most 128 query
// heads per KV head, no block selection.
inline bool attention_tc_fits(int head_dim, int page_size, int group) {
  return head_dim == kTcD && page_size >= 16 && page_size % 16 == 0 && group >= 1 && group <= kTcRows;
}

// Tiles of at most 16 rows (decode steps) on the same kernel with one softmax warp: the same sizes, at most
// 16 query heads per KV head.
constexpr int kTcFewRows = 16;
inline bool attention_tc_few_fits(int head_dim, int page_size, int group) {
  return attention_tc_fits(head_dim, page_size, group) && group <= kTcFewRows;
}

// `p.tile_rows` is 128, or 16 for the few-rows form.
inline int launch_attention_tc(const AttnParams& p, int n_tokens, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess ||
        cudaFuncSetAttribute(attention_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess)
      return 2;
    configured = true;
  }
  if (p.tile_rows != kTcRows && p.tile_rows != kTcFewRows) return 5;
  CUtensorMap mq, mk, mv;
  {
    // queries [T, Hq, D] seen as (d, head, token); a box is (64, group, tokens per tile)
    const uint64_t dims[3] = {(uint64_t)kTcD, (uint64_t)p.Hq, (uint64_t)n_tokens};
    const uint64_t strides[2] = {(uint64_t)kTcD * 2, (uint64_t)p.Hq * kTcD * 2};
    const uint32_t box[3] = {64, (uint32_t)p.G, (uint32_t)(p.tile_rows / p.G)};
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
  const long long n_work = (long long)p.n_items * p.Hkv;  // one CTA per SM, each takes every sms-th piece of work
  const int grid = (int)(n_work < sms ? n_work : sms);
  if (p.tile_rows == kTcFewRows) {
    FTK_LAUNCH(attention_tc_kernel<true>, grid, kTcThreads, kTcSmem, s, mq, mk, mv, p);
  } else {
    FTK_LAUNCH(attention_tc_kernel<false>, grid, kTcThreads, kTcSmem, s, mq, mk, mv, p);
  }
  return 0;
}

}  // namespace ftk
