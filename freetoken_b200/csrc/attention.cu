// Causal softmax attention of a step's queries over paged keys and values.
//
// One interface serves prompt portions and single decoded tokens side by side: the host cuts the
// step's queries into tiles of whole tokens (a tile = `group` query heads of one KV head for a few
// consecutive tokens of one segment) and, where that leaves SMs idle, splits a tile's key range;
// each work item is 8 int32 (see engine/attention_plan.py).  grid = (items, KV heads).  A split tile
// writes (max, sum, unnormalised output) per row to scratch and merge_kernel combines the splits in
// split order.  The reference has three kernels for this: tiled extend
// (python/freetoken/kernel/triton/attention.py:469-880), split-KV decode (:147-466) and a scalar
// fallback for float32 (:45-144).
//
// Two implementations share the indexing code below:
//   * attention_f32_kernel: the true 32-bit path.  One warp per query row, keys in chunks of 32
//     staged in shared memory, IEEE expf, float32 everywhere.
//   * attention_bf16_kernel: 64 query rows per CTA on mma.sync m16n8k16 (bf16 in, float32
//     accumulate), K/V tiles of 64 keys brought in by cp.async through the block table, online
//     softmax in float32 with exp2; probabilities are rounded to bfloat16 before P.V, as in the
//     reference (attention.py:252,573).
//   * attention_decode_bf16_kernel: the same arithmetic for tiles of at most 16 query rows (steps of
//     single decoded tokens): the four warps split each key tile between them and a three-stage
//     pipeline keeps two key/value tiles in flight.
// Keys that a tile may not read (beyond its range) are never loaded: fresh pages may hold anything.
#include <mma.h>

#include "common.cuh"

namespace ftk {

struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  const int32_t* block_table;
  int bt_stride;
  const int32_t* seg_info;
  int n_segs;
  const int32_t* items;
  int n_items;
  float* part_o;
  float* part_ml;
  int n_slots;
  int Hq, Hkv, G, D, P, num_pages, tile_rows;
  float scale;
  int window;
  // block-sparse layers: per (token, KV head) the chosen key blocks, ascending, -1 padded; the work
  // items' key ranges then count *chosen* keys (block 0 of the list first) instead of positions
  const int32_t* sel;
  int sel_stride;
  int block_size;
  // decode tiles: one counter per (split tile, KV head), zero between launches; the last of a tile's
  // splits to arrive merges them, so no merge kernel follows.  nullptr: the merge kernel does it.
  unsigned int* arrivals;
};

constexpr int kAttnArrivalSlots = 1 << 16;
__device__ unsigned int g_attn_arrivals[kAttnArrivalSlots];

constexpr int kMaxMergeSplits = 64;  // most splits of one tile that the merge step takes

struct Item {
  int seg, tok0, ntok, kb, ke, nsplit, split, base;
  int q_start, q_len, kv_len, bt_row;
  bool ok;
};

__device__ __forceinline__ Item load_item(const AttnParams& p, int idx) {
  Item it;
  const int32_t* w = p.items + (size_t)idx * 8;
  it.seg = w[0]; it.tok0 = w[1]; it.ntok = w[2]; it.kb = w[3]; it.ke = w[4];
  it.nsplit = w[5]; it.split = w[6]; it.base = w[7];
  it.ok = it.seg >= 0 && it.seg < p.n_segs && it.ntok > 0 && it.ntok * p.G <= p.tile_rows;
  if (it.ok) {
    const int32_t* s = p.seg_info + (size_t)it.seg * 4;
    it.q_start = s[0]; it.q_len = s[1]; it.kv_len = s[2]; it.bt_row = s[3];
    const int key_limit = p.sel ? p.sel_stride * p.block_size : it.kv_len;
    it.ok = it.tok0 >= 0 && it.tok0 + it.ntok <= it.q_len && it.kb >= 0 && it.ke <= key_limit &&
            (!p.sel || it.ntok == 1) &&
            it.q_len <= it.kv_len && it.bt_row >= 0 &&
            (it.nsplit == 1 || (it.nsplit <= kMaxMergeSplits && it.base >= 0 &&
                                it.base + it.nsplit <= p.n_slots && p.part_o != nullptr));
  }
  return it;
}

// Address of key/value row `pos` of the request (element offset into a [pages, Hkv, P, D] slab),
// or -1 when the block table names a page outside the pool.
// Position in the sequence of key number `v` of the tile's range: `v` itself, or, in a block-sparse
// layer, the v-th key of the chosen blocks of the tile's (single) token; -1 when there is none.
__device__ __forceinline__ int key_position(const AttnParams& p, const Item& it, int kvh, int v) {
  if (!p.sel) return v;
  const int32_t* chosen = p.sel + ((size_t)(it.q_start + it.tok0) * p.Hkv + kvh) * p.sel_stride;
  const int slot = v / p.block_size;
  if (slot >= p.sel_stride) return -1;
  const int b = chosen[slot];
  if (b < 0) return -1;
  const int pos = b * p.block_size + v % p.block_size;
  return pos < it.kv_len ? pos : -1;
}

__device__ __forceinline__ long long kv_row_offset(const AttnParams& p, const Item& it, int kvh, int v) {
  const int pos = key_position(p, it, kvh, v);
  if (pos < 0) return -1;
  const int page = p.block_table[(size_t)it.bt_row * p.bt_stride + pos / p.P];
  if (page < 0 || page >= p.num_pages) return -1;
  return (((long long)page * p.Hkv + kvh) * p.P + pos % p.P) * p.D;
}

// ================================================================= float32 path
constexpr int kF32Rows = 16;   // warps per block = query rows per tile
constexpr int kF32Chunk = 32;  // keys per chunk

template <typename T>
__global__ void __launch_bounds__(kF32Rows * 32) attention_f32_kernel(AttnParams p) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float smem[];
  const Item it = load_item(p, blockIdx.x);
  if (!it.ok) return;
  const int kvh = blockIdx.y;
  const int D = p.D, G = p.G;
  const int ldk = D + 1;
  float* sq = smem;                       // [rows][D]
  float* sk = sq + kF32Rows * D;          // [chunk][D + 1]
  float* sv = sk + kF32Chunk * ldk;       // [chunk][D]
  __shared__ int spos[kF32Chunk];         // position in the sequence of each key of the chunk (-1: none)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = it.ntok * G;
  const T* q = (const T*)p.q;
  const T* kbase = (const T*)p.k;
  const T* vbase = (const T*)p.v;

  for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    const int tok = it.q_start + it.tok0 + r / G;
    sq[i] = to_float(q[((size_t)tok * p.Hq + kvh * G + r % G) * D + d]);
  }
  const bool active = warp < R;
  const int q_pos = it.kv_len - it.q_len + it.tok0 + warp / G;
  const int lo_row = p.window > 0 ? q_pos - p.window + 1 : 0;
  constexpr int kPer = 8;  // D <= 256
  float acc[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int c0 = it.kb; c0 < it.ke; c0 += kF32Chunk) {
    __syncthreads();
    const int nk = min(kF32Chunk, it.ke - c0);
    for (int i = threadIdx.x; i < kF32Chunk * D; i += blockDim.x) {
      const int j = i / D, d = i % D;
      float kval = 0.f, vval = 0.f;
      if (j < nk) {
        const long long off = kv_row_offset(p, it, kvh, c0 + j);
        if (off >= 0) {
          kval = to_float(kbase[off + d]);
          vval = to_float(vbase[off + d]);
        }
        if (d == 0) spos[j] = off >= 0 ? key_position(p, it, kvh, c0 + j) : -1;
      }
      sk[j * ldk + d] = kval;
      sv[j * D + d] = vval;
    }
    __syncthreads();
    if (!active) continue;
    const int key = lane < nk ? spos[lane] : -1;
    const bool vis = key >= 0 && key <= q_pos && key >= lo_row;
    float s = -INFINITY;
    if (vis) {
      const float* qr = sq + warp * D;
      const float* kr = sk + lane * ldk;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(qr[d], kr[d], dot);
      s = dot * p.scale;
    }
    const float cm = warp_max(s);
    if (cm == -INFINITY) continue;  // nothing visible in this chunk
    const float m_new = fmaxf(m, cm);
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    const float pj = vis ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kPer; ++i) acc[i] *= corr;
    for (int j = 0; j < nk; ++j) {
      const float pb = __shfl_sync(0xffffffffu, pj, j);
      if (pb != 0.f) {
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] = fmaf(pb, sv[j * D + d], acc[i]);
        }
      }
    }
  }
  if (!active) return;
  const int tok = it.q_start + it.tok0 + warp / G;
  if (it.nsplit == 1) {
    T* o = (T*)p.out + ((size_t)tok * p.Hq + kvh * G + warp % G) * D;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int d = lane + 32 * i;
      if (d < D) o[d] = from_float<T>(acc[i] * inv);
    }
  } else {
    const size_t slot = ((size_t)(it.base + it.split) * p.Hkv + kvh) * p.tile_rows + warp;
    float* po = p.part_o + slot * D;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int d = lane + 32 * i;
      if (d < D) po[d] = acc[i];
    }
    if (lane == 0) {
      p.part_ml[slot * 2] = m;
      p.part_ml[slot * 2 + 1] = l;
    }
  }
}

// ================================================================= merge of split tiles
// out = sum_i acc_i e^(m_i - M) / sum_i l_i e^(m_i - M), splits taken in order.  The CTA of split s
// merges the tile's rows s, s + n_splits, ...: a warp takes a row, a lane four output columns, and the
// splits' values are fetched eight at a time, so a row costs a few memory round trips however many
// splits there are.
template <typename T>
__global__ void __launch_bounds__(512) attention_merge_kernel(AttnParams p) {
  const Item it = load_item(p, blockIdx.x);  // the work list was made on the host before the step
  pdl_wait();
  pdl_trigger();
  if (!it.ok || it.nsplit <= 1) return;
  const int kvh = blockIdx.y;
  const int D = p.D, G = p.G;
  const int R = it.ntok * G;
  const int lane = threadIdx.x & 31;
  const size_t slot_step = (size_t)p.Hkv * p.tile_rows;
  // a row per warp at a time (the rows of a block are independent, and each is three dependent trips
  // to memory), four output elements per lane
  const int warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int r = it.split + warp * it.nsplit; r < R; r += it.nsplit * n_warps) {
    const size_t slot0 = ((size_t)it.base * p.Hkv + kvh) * p.tile_rows + r;
    // the first eight splits' values of the row's first 128 columns: asked for together with the weights
    // (they do not depend on them), so that a row is two trips to memory one after the other, not three.  A
    // piece without keys has weight 0 and a slot that nobody wrote: its values are dropped below.
    auto fetch = [&](int d, int i0, float4 (&x)[8]) {
#pragma unroll
      for (int u = 0; u < 8; ++u)
        x[u] = (i0 + u < it.nsplit && d < D)
                   ? *reinterpret_cast<const float4*>(p.part_o + (slot0 + (i0 + u) * slot_step) * D + d)
                   : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    float4 first[8];
    fetch(4 * lane, 0, first);
    // weights of the splits, spread over the lanes
    float wgt[kMaxMergeSplits / 32];
    float lsum[kMaxMergeSplits / 32];
    float M = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxMergeSplits / 32; ++j) {
      const int i = lane + 32 * j;
      const float2 ml = i < it.nsplit ? *reinterpret_cast<const float2*>(p.part_ml + (slot0 + i * slot_step) * 2)
                                      : make_float2(-INFINITY, 0.f);
      wgt[j] = ml.x;
      lsum[j] = ml.y;
      M = fmaxf(M, ml.x);
    }
    M = warp_max(M);
    float L = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxMergeSplits / 32; ++j) {
      const float w = wgt[j] != -INFINITY ? expf(wgt[j] - M) : 0.f;
      wgt[j] = w;
      L += lsum[j] * w;
    }
    L = warp_sum(L);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int tok = it.q_start + it.tok0 + r / G;
    T* o = (T*)p.out + ((size_t)tok * p.Hq + kvh * G + r % G) * D;
    for (int d0 = 0; d0 < D; d0 += 128) {
      const int d = d0 + 4 * lane;  // D is a multiple of 16: a lane's four elements exist together or not at all
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int i0 = 0; i0 < it.nsplit; i0 += 8) {  // eight loads in flight before the first use
        float4 x[8];
        float w[8];
        if (d0 == 0 && i0 == 0) {
#pragma unroll
          for (int u = 0; u < 8; ++u) x[u] = first[u];
        } else {
          fetch(d, i0, x);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u;
          const float wsrc = (i >> 5) ? wgt[1] : wgt[0];
          w[u] = __shfl_sync(0xffffffffu, wsrc, i & 31);
          if (w[u] == 0.f) x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          acc.x += x[u].x * w[u];
          acc.y += x[u].y * w[u];
          acc.z += x[u].z * w[u];
          acc.w += x[u].w * w[u];
        }
      }
      if (d < D) {
        o[d] = from_float<T>(acc.x * inv);
        o[d + 1] = from_float<T>(acc.y * inv);
        o[d + 2] = from_float<T>(acc.z * inv);
        o[d + 3] = from_float<T>(acc.w * inv);
      }
    }
  }
}

// ================================================================= bfloat16 path (mma.sync)
constexpr int kBM = 64;  // query rows per CTA (4 warps x 16)
constexpr int kBN = 64;  // keys per iteration

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Element offsets of key rows [c0, c0 + 64) of the request (-1 for rows outside [.., ke)), one row per
// thread of the first 64.  Computed one tile ahead of the copy that uses them, so that the block-table
// lookups are off the copy's critical path.
__device__ __forceinline__ long long fetch_row_offset(const AttnParams& p, const Item& it, int kvh, int c0) {
  const int pos = c0 + (int)threadIdx.x;
  return (threadIdx.x < kBN && pos < it.ke) ? kv_row_offset(p, it, kvh, pos) : -1;
}
__device__ __forceinline__ void publish_row_offset(long long* row_off, long long v) {
  if (threadIdx.x < kBN) row_off[threadIdx.x] = v;
}
// block-sparse layers: the sequence position of key c0 + thread of the tile (for the mask)
__device__ __forceinline__ void publish_row_position(const AttnParams& p, const Item& it, int kvh, int c0, int* row_pos,
                                                     long long off) {
  if (p.sel && threadIdx.x < kBN) row_pos[threadIdx.x] = off >= 0 ? key_position(p, it, kvh, c0 + (int)threadIdx.x) : -1;
}
__device__ __forceinline__ void tile_row_offsets(const AttnParams& p, const Item& it, int kvh, int c0, long long* row_off) {
  publish_row_offset(row_off, fetch_row_offset(p, it, kvh, c0));
}

// Bring keys/values of one tile into [64][ld] buffers; consecutive threads copy consecutive 16-byte
// pieces of a row, rows without an offset are zero-filled.  When the pieces per row divide the 128
// threads, a thread keeps its column and only steps through rows (no division in the loop).
__device__ __forceinline__ void load_kv_tile(const AttnParams& p, const long long* row_off,
                                             __nv_bfloat16* sk, __nv_bfloat16* sv, int ld) {
  const int chunks = p.D >> 3;
  const __nv_bfloat16* kb = (const __nv_bfloat16*)p.k;
  const __nv_bfloat16* vb = (const __nv_bfloat16*)p.v;
  if ((chunks & (chunks - 1)) == 0) {  // 2, 4, 8, 16 or 32 pieces per row
    const int c = threadIdx.x & (chunks - 1);
    const int step = 128 / chunks;
    for (int j = threadIdx.x / chunks; j < kBN; j += step) {
      const long long off = row_off[j];
      const bool valid = off >= 0;
      const long long o = valid ? off + c * 8 : 0;
      cp_async16(sk + j * ld + c * 8, kb + o, valid);
      cp_async16(sv + j * ld + c * 8, vb + o, valid);
    }
  } else {
    for (int i = threadIdx.x; i < kBN * chunks; i += blockDim.x) {
      const int j = i / chunks, c = i - j * chunks;
      const long long off = row_off[j];
      const bool valid = off >= 0;
      const long long o = valid ? off + c * 8 : 0;
      cp_async16(sk + j * ld + c * 8, kb + o, valid);
      cp_async16(sv + j * ld + c * 8, vb + o, valid);
    }
  }
}

template <int DMAX>
__global__ void __launch_bounds__(128) attention_bf16_kernel(AttnParams p) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const Item it = load_item(p, blockIdx.x);
  if (!it.ok) return;
  const int kvh = blockIdx.y;
  const int D = p.D, G = p.G;
  const int ld = D + 8;  // 16 bytes of padding keep ldmatrix free of bank conflicts for every D
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sk0 = sq + kBM * ld;
  __nv_bfloat16* sv0 = sk0 + 2 * kBN * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = it.ntok * G;
  const int chunks = D >> 3;
  const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;

  // queries of the tile (rows beyond R are zero)
  for (int i = threadIdx.x; i < kBM * chunks; i += blockDim.x) {
    const int r = i / chunks, c = i % chunks;
    const bool valid = r < R;
    const int tok = it.q_start + it.tok0 + (valid ? r / G : 0);
    const size_t off = ((size_t)tok * p.Hq + kvh * G + (valid ? r % G : 0)) * D + c * 8;
    cp_async16(sq + r * ld + c * 8, q + off, valid);
  }
  const int n_iter = (it.ke - it.kb + kBN - 1) / kBN;
  __shared__ long long row_off[3][kBN];  // offsets of tile t live in row_off[t % 3]
  tile_row_offsets(p, it, kvh, it.kb, row_off[0]);
  tile_row_offsets(p, it, kvh, it.kb + kBN, row_off[1]);
  __syncthreads();
  if (n_iter > 0) load_kv_tile(p, row_off[0], sk0, sv0, ld);
  cp_async_commit();

  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
  const int pos_base = it.kv_len - it.q_len + it.tok0;
  const int qp0 = r0 < R ? pos_base + r0 / G : -1;
  const int qp1 = r1 < R ? pos_base + r1 / G : -1;
  const int lo0 = p.window > 0 ? qp0 - p.window + 1 : 0;
  const int lo1 = p.window > 0 ? qp1 - p.window + 1 : 0;
  const float sl2 = p.scale * 1.4426950408889634f;

  float o[DMAX / 8][4];
#pragma unroll
  for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int iter = 0; iter < n_iter; ++iter) {
    const int buf = iter & 1;
    __nv_bfloat16* sk = sk0 + buf * kBN * ld;
    __nv_bfloat16* sv = sv0 + buf * kBN * ld;
    if (iter + 1 < n_iter)
      load_kv_tile(p, row_off[(iter + 1) % 3], sk0 + (buf ^ 1) * kBN * ld, sv0 + (buf ^ 1) * kBN * ld, ld);
    cp_async_commit();
    // the block-table lookup for the tile after next travels while this tile is computed
    const long long next_off = fetch_row_offset(p, it, kvh, it.kb + (iter + 2) * kBN);
    cp_async_wait<1>();
    __syncthreads();

    // S = Q K^T  (16 rows x 64 keys per warp)
    float s[kBN / 8][4];
#pragma unroll
    for (int n = 0; n < kBN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DMAX / 16; ++kk) {
      if (kk * 16 < D) {
        uint32_t a[4];
        ldsm_x4(a, sq + (warp * 16 + (lane & 15)) * ld + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n2 = 0; n2 < kBN / 16; ++n2) {
          uint32_t b[4];
          ldsm_x4(b, sk + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * ld + kk * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * n2], a, b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
        }
      }
    }
    // mask, running max
    const int c0 = it.kb + iter * kBN;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < kBN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = c0 + n * 8 + (lane & 3) * 2 + e;
        const bool in = key < it.ke;
        const bool v0 = in && key <= qp0 && key >= lo0;
        const bool v1 = in && key <= qp1 && key >= lo1;
        s[n][e] = v0 ? s[n][e] * sl2 : -INFINITY;
        s[n][2 + e] = v1 ? s[n][2 + e] * sl2 : -INFINITY;
        mx0 = fmaxf(mx0, s[n][e]);
        mx1 = fmaxf(mx1, s[n][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
    const float cr0 = m0 == -INFINITY ? 0.f : fast_exp2(m0 - base0);
    const float cr1 = m1 == -INFINITY ? 0.f : fast_exp2(m1 - base1);
    m0 = mn0; m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int n = 0; n < kBN / 8; ++n) {
      s[n][0] = fast_exp2(s[n][0] - base0); s[n][1] = fast_exp2(s[n][1] - base0);
      s[n][2] = fast_exp2(s[n][2] - base1); s[n][3] = fast_exp2(s[n][3] - base1);
      sum0 += s[n][0] + s[n][1];
      sum1 += s[n][2] + s[n][3];
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * cr0 + sum0;
    l1 = l1 * cr1 + sum1;
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) {
      o[i][0] *= cr0; o[i][1] *= cr0; o[i][2] *= cr1; o[i][3] *= cr1;
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < DMAX / 16; ++d2) {
        if (d2 * 16 < D) {
          uint32_t b[4];
          ldsm_x4_trans(b, sv + (kk * 16 + (lane & 15)) * ld + d2 * 16 + (lane >> 4) * 8);
          mma_bf16(o[2 * d2], a, b[0], b[1]);
          mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
        }
      }
    }
    publish_row_offset(row_off[(iter + 2) % 3], next_off);
    __syncthreads();
  }
  cp_async_wait<0>();

  // epilogue
  if (it.nsplit == 1) {
    __nv_bfloat16* out = (__nv_bfloat16*)p.out;
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (r0 < R) {
      __nv_bfloat16* dst = out + ((size_t)(it.q_start + it.tok0 + r0 / G) * p.Hq + kvh * G + r0 % G) * D;
#pragma unroll
      for (int i = 0; i < DMAX / 8; ++i)
        if (i * 8 < D) *reinterpret_cast<uint32_t*>(dst + i * 8 + (lane & 3) * 2) = pack_bf16(o[i][0] * i0, o[i][1] * i0);
    }
    if (r1 < R) {
      __nv_bfloat16* dst = out + ((size_t)(it.q_start + it.tok0 + r1 / G) * p.Hq + kvh * G + r1 % G) * D;
#pragma unroll
      for (int i = 0; i < DMAX / 8; ++i)
        if (i * 8 < D) *reinterpret_cast<uint32_t*>(dst + i * 8 + (lane & 3) * 2) = pack_bf16(o[i][2] * i1, o[i][3] * i1);
    }
  } else {
    // the running max is in the exp2 domain (scores were multiplied by scale*log2 e); the merge
    // works with natural exponentials, so convert
    const float ln2 = 0.6931471805599453f;
    const size_t slot0 = ((size_t)(it.base + it.split) * p.Hkv + kvh) * p.tile_rows;
    if (r0 < R) {
      float* po = p.part_o + (slot0 + r0) * D;
#pragma unroll
      for (int i = 0; i < DMAX / 8; ++i)
        if (i * 8 < D) *reinterpret_cast<float2*>(po + i * 8 + (lane & 3) * 2) = make_float2(o[i][0], o[i][1]);
      if ((lane & 3) == 0) {
        p.part_ml[(slot0 + r0) * 2] = m0 == -INFINITY ? -INFINITY : m0 * ln2;
        p.part_ml[(slot0 + r0) * 2 + 1] = l0;
      }
    }
    if (r1 < R) {
      float* po = p.part_o + (slot0 + r1) * D;
#pragma unroll
      for (int i = 0; i < DMAX / 8; ++i)
        if (i * 8 < D) *reinterpret_cast<float2*>(po + i * 8 + (lane & 3) * 2) = make_float2(o[i][2], o[i][3]);
      if ((lane & 3) == 0) {
        p.part_ml[(slot0 + r1) * 2] = m1 == -INFINITY ? -INFINITY : m1 * ln2;
        p.part_ml[(slot0 + r1) * 2 + 1] = l1;
      }
    }
  }
}

// The same merge for all rows of one tile by one block (the split that arrived last).  The splits'
// (max, sum) pairs are fetched once into shared memory, a thread per row turns them into weights, and
// then every thread takes (row, four columns) items whose loads over the splits are independent.
// `scratch` holds 3 * tile_rows * nsplit + tile_rows floats.
__device__ __forceinline__ void merge_tile_rows_bf16(const AttnParams& p, const Item& it, int kvh, float* scratch) {
  const int D = p.D, G = p.G, R = it.ntok * G, S = it.nsplit;
  const size_t slot_step = (size_t)p.Hkv * p.tile_rows;
  const size_t slot0 = ((size_t)it.base * p.Hkv + kvh) * p.tile_rows;
  float* sm = scratch;            // [R][S] max, later the weight
  float* sl = sm + R * S;         // [R][S] sum
  float* sinv = sl + R * S;       // [R]
  for (int i = threadIdx.x; i < R * S; i += blockDim.x) {
    const int r = i / S, sp = i % S;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (slot0 + r + sp * slot_step) * 2));
    sm[i] = ml.x;
    sl[i] = ml.y;
  }
  __syncthreads();
  if ((int)threadIdx.x < R) {
    const int r = threadIdx.x;
    float M = -INFINITY;
    for (int sp = 0; sp < S; ++sp) M = fmaxf(M, sm[r * S + sp]);
    float L = 0.f;
    for (int sp = 0; sp < S; ++sp) {  // splits in order
      const float m = sm[r * S + sp];
      const float w = m != -INFINITY ? expf(m - M) : 0.f;
      L += sl[r * S + sp] * w;
      sm[r * S + sp] = w;
    }
    sinv[r] = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  const int quads = D >> 2;  // D is a multiple of 16
  for (int i = threadIdx.x; i < R * quads; i += blockDim.x) {
    const int r = i / quads, d = (i % quads) << 2;
    const float* src = p.part_o + (slot0 + r) * D + d;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int sp = 0; sp < S; ++sp) {
      const float w = sm[r * S + sp];
      const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * slot_step * D));
      acc.x += x.x * w; acc.y += x.y * w; acc.z += x.z * w; acc.w += x.w * w;
    }
    const float inv = sinv[r];
    const int tok = it.q_start + it.tok0 + r / G;
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + ((size_t)tok * p.Hq + kvh * G + r % G) * D + d;
    uint2 pk;
    pk.x = pack_bf16(acc.x * inv, acc.y * inv);
    pk.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(o) = pk;
  }
}

// ----------------------------------------------------------------- decode tiles (at most 16 query rows)
// A step of single decoded tokens has `group` query rows per (request, KV head): too few to fill a
// 64-row tile.  Here the four warps share the 16-row query tile and split each 64-key tile between
// them (16 keys per warp); every warp keeps its own running max / sum / output and the four are merged
// through shared memory at the end.  Key/value tiles arrive through a three-stage cp.async pipeline so
// that two tiles are always in flight per CTA: the kernel's job is to keep HBM busy.
constexpr int kDecRows = 16;
constexpr int kDecStages = 3;

template <int DMAX>
__global__ void __launch_bounds__(128) attention_decode_bf16_kernel(AttnParams p) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const Item it = load_item(p, blockIdx.x);
  if (!it.ok) return;
  const int kvh = blockIdx.y;
  const int D = p.D, G = p.G;
  const int ld = D + 8;
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sk0 = sq + kDecRows * ld;
  __nv_bfloat16* sv0 = sk0 + kDecStages * kBN * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = it.ntok * G;
  const int chunks = D >> 3;
  const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;

  for (int i = threadIdx.x; i < kDecRows * chunks; i += blockDim.x) {
    const int r = i / chunks, c = i % chunks;
    const bool valid = r < R;
    const int tok = it.q_start + it.tok0 + (valid ? r / G : 0);
    const size_t off = ((size_t)tok * p.Hq + kvh * G + (valid ? r % G : 0)) * D + c * 8;
    cp_async16(sq + r * ld + c * 8, q + off, valid);
  }
  const int n_iter = (it.ke - it.kb + kBN - 1) / kBN;
  __shared__ long long row_off[4][kBN];  // offsets of tile t live in row_off[t % 4]
  __shared__ int row_pos[4][kBN];        // block-sparse layers: sequence positions of the tile's keys
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    const long long off = fetch_row_offset(p, it, kvh, it.kb + t * kBN);
    publish_row_offset(row_off[t], off);
    publish_row_position(p, it, kvh, it.kb + t * kBN, row_pos[t], off);
  }
  __syncthreads();
  if (n_iter > 0) load_kv_tile(p, row_off[0], sk0, sv0, ld);
  cp_async_commit();
  if (n_iter > 1) load_kv_tile(p, row_off[1], sk0 + kBN * ld, sv0 + kBN * ld, ld);
  cp_async_commit();

  const int r0 = lane >> 2, r1 = r0 + 8;
  const int pos_base = it.kv_len - it.q_len + it.tok0;
  const int qp0 = r0 < R ? pos_base + r0 / G : -1;
  const int qp1 = r1 < R ? pos_base + r1 / G : -1;
  const int lo0 = p.window > 0 ? qp0 - p.window + 1 : 0;
  const int lo1 = p.window > 0 ? qp1 - p.window + 1 : 0;
  const float sl2 = p.scale * 1.4426950408889634f;

  float o[DMAX / 8][4];
#pragma unroll
  for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int iter = 0; iter < n_iter; ++iter) {
    cp_async_wait<1>();
    __syncthreads();  // tile `iter` has landed for everyone, and everyone is done with tile `iter - 1`
    if (iter + 2 < n_iter) {
      const int st = (iter + 2) % kDecStages;
      load_kv_tile(p, row_off[(iter + 2) & 3], sk0 + st * kBN * ld, sv0 + st * kBN * ld, ld);
    }
    cp_async_commit();
    const long long next_off = fetch_row_offset(p, it, kvh, it.kb + (iter + 3) * kBN);
    const int stage = iter % kDecStages;
    const __nv_bfloat16* sk = sk0 + stage * kBN * ld + warp * 16 * ld;  // this warp's 16 keys
    const __nv_bfloat16* sv = sv0 + stage * kBN * ld + warp * 16 * ld;

    float s[2][4];
    s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DMAX / 16; ++kk) {
      if (kk * 16 < D) {
        uint32_t a[4], b[4];
        ldsm_x4(a, sq + (lane & 15) * ld + kk * 16 + (lane >> 4) * 8);
        ldsm_x4(b, sk + ((lane & 7) + ((lane >> 4) << 3)) * ld + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[0], a, b[0], b[1]);
        mma_bf16(s[1], a, b[2], b[3]);
      }
    }
    const int c0 = it.kb + iter * kBN + warp * 16;
    float mx0 = -INFINITY, mx1 = -INFINITY;
    // a 16-key slice that every row of the tile may read in full needs no mask (rows beyond the
    // tile's last are never stored, so what they compute does not matter)
    const bool interior = p.window == 0 && !p.sel && c0 + 16 <= it.ke && c0 + 16 <= pos_base + 1;
    if (interior) {
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] *= sl2;
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
    } else {
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = n * 8 + (lane & 3) * 2 + e;
          int key = c0 + col;
          const bool in = key < it.ke;
          if (p.sel) key = in ? row_pos[iter & 3][warp * 16 + col] : -1;
          const bool v0 = in && key >= 0 && key <= qp0 && key >= lo0;
          const bool v1 = in && key >= 0 && key <= qp1 && key >= lo1;
          s[n][e] = v0 ? s[n][e] * sl2 : -INFINITY;
          s[n][2 + e] = v1 ? s[n][2 + e] * sl2 : -INFINITY;
          mx0 = fmaxf(mx0, s[n][e]);
          mx1 = fmaxf(mx1, s[n][2 + e]);
        }
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
    const float cr0 = m0 == -INFINITY ? 0.f : fast_exp2(m0 - base0);
    const float cr1 = m1 == -INFINITY ? 0.f : fast_exp2(m1 - base1);
    m0 = mn0; m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      s[n][0] = fast_exp2(s[n][0] - base0); s[n][1] = fast_exp2(s[n][1] - base0);
      s[n][2] = fast_exp2(s[n][2] - base1); s[n][3] = fast_exp2(s[n][3] - base1);
      sum0 += s[n][0] + s[n][1];
      sum1 += s[n][2] + s[n][3];
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * cr0 + sum0;
    l1 = l1 * cr1 + sum1;
    uint32_t a[4];
    a[0] = pack_bf16(s[0][0], s[0][1]);
    a[1] = pack_bf16(s[0][2], s[0][3]);
    a[2] = pack_bf16(s[1][0], s[1][1]);
    a[3] = pack_bf16(s[1][2], s[1][3]);
    // the running maximum rarely moves once a few tiles are in: then nothing has to be rescaled
    if (__any_sync(0xffffffffu, cr0 != 1.f || cr1 != 1.f)) {
#pragma unroll
      for (int i = 0; i < DMAX / 8; ++i) {
        o[i][0] *= cr0; o[i][1] *= cr0; o[i][2] *= cr1; o[i][3] *= cr1;
      }
    }
#pragma unroll
    for (int d2 = 0; d2 < DMAX / 16; ++d2) {
      if (d2 * 16 < D) {
        uint32_t b[4];
        ldsm_x4_trans(b, sv + (lane & 15) * ld + d2 * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * d2], a, b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
      }
    }
    publish_row_offset(row_off[(iter + 3) & 3], next_off);  // read after the next iteration's barrier
    publish_row_position(p, it, kvh, it.kb + (iter + 3) * kBN, row_pos[(iter + 3) & 3], next_off);
  }
  cp_async_wait<0>();
  __syncthreads();  // the key/value stages are free: reuse them for the merge of the four warps

  float* sm_m = reinterpret_cast<float*>(sk0);          // [4][16]
  float* sm_l = sm_m + 4 * kDecRows;                    // [4][16]
  float* sm_o = sm_l + 4 * kDecRows;                    // [4][16][D]
  if ((lane & 3) == 0) {
    sm_m[warp * kDecRows + r0] = m0; sm_m[warp * kDecRows + r1] = m1;
    sm_l[warp * kDecRows + r0] = l0; sm_l[warp * kDecRows + r1] = l1;
  }
#pragma unroll
  for (int i = 0; i < DMAX / 8; ++i) {
    if (i * 8 < D) {
      const int d = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(sm_o + ((size_t)warp * kDecRows + r0) * D + d) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(sm_o + ((size_t)warp * kDecRows + r1) * D + d) = make_float2(o[i][2], o[i][3]);
    }
  }
  __syncthreads();
  const float ln2 = 0.6931471805599453f;
  for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * kDecRows + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm_m[w * kDecRows + r];
      const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      L += sm_l[w * kDecRows + r] * f;
      acc += sm_o[((size_t)w * kDecRows + r) * D + d] * f;
    }
    const int tok = it.q_start + it.tok0 + r / G;
    if (it.nsplit == 1) {
      __nv_bfloat16* out = (__nv_bfloat16*)p.out + ((size_t)tok * p.Hq + kvh * G + r % G) * D;
      out[d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const size_t slot = ((size_t)(it.base + it.split) * p.Hkv + kvh) * p.tile_rows + r;
      p.part_o[slot * D + d] = acc;
      if (d == 0) {
        p.part_ml[slot * 2] = M == -INFINITY ? -INFINITY : M * ln2;
        p.part_ml[slot * 2 + 1] = L;
      }
    }
  }
  if (it.nsplit > 1 && p.arrivals) {
    // the split that finds all the others arrived merges the tile (nobody waits for anybody)
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int* cnt = p.arrivals + (size_t)it.base * p.Hkv + kvh;
      last = atomicAdd(cnt, 1u) == (unsigned)it.nsplit - 1u;
      if (last) *cnt = 0;  // ready for the next launch
    }
    __syncthreads();
    if (last) {
      __threadfence();
      merge_tile_rows_bf16(p, it, kvh, reinterpret_cast<float*>(sk0));
    }
  }
}

template <int DMAX>
static int launch_decode_bf16(const AttnParams& p, cudaStream_t s) {
  const size_t kv = (size_t)2 * kDecStages * kBN * (p.D + 8) * sizeof(__nv_bfloat16);
  const size_t merge = (size_t)(8 * kDecRows + 4 * kDecRows * p.D) * sizeof(float);
  const size_t smem = (size_t)kDecRows * (p.D + 8) * sizeof(__nv_bfloat16) + (kv > merge ? kv : merge);
  auto kern = attention_decode_bf16_kernel<DMAX>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(p.n_items, p.Hkv);
  FTK_LAUNCH(kern, grid, 128, smem, s, p);
  return 0;
}

template <int DMAX>
static int launch_bf16(const AttnParams& p, cudaStream_t s) {
  const size_t smem = (size_t)(kBM + 4 * kBN) * (p.D + 8) * sizeof(__nv_bfloat16);
  auto kern = attention_bf16_kernel<DMAX>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(p.n_items, p.Hkv);
  FTK_LAUNCH(kern, grid, 128, smem, s, p);
  return 0;
}

}  // namespace ftk

#include "attention_tc.cuh"
#include "attention_tc2.cuh"

using namespace ftk;

// Status of the tensor-core attention kernel's bounded waits (merged into ftk_read_status).
int ftk_attention_tc_status(int* out) {
  int host[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(host, g_attn_status, sizeof(host)) != cudaSuccess) return 2;
  out[0] = host[0];
  out[1] = host[1];
  if (host[0]) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_attn_status, zero, sizeof(zero));
  }
  return 0;
}

int ftk_attention_tc_set_status(int code) {
  int host[4] = {code, -1, 0, 0};
  return cudaMemcpyToSymbol(g_attn_status, host, sizeof(host)) == cudaSuccess ? 0 : 2;
}

extern "C" int ftk_attention_tc_fits(int head_dim, int page_size, int group) {
  return attention_tc_fits(head_dim, page_size, group) ? 1 : 0;
}

extern "C" int ftk_attention_tc_few_fits(int head_dim, int page_size, int group) {
  return attention_tc_few_fits(head_dim, page_size, group) ? 1 : 0;
}

enum TcForm { kTcSingle = 0, kTcPair = 1, kTcFew = 2 };

// bfloat16 steps on the tensor-core kernels: tiles of 128 query rows (`items` planned for tile_rows =
// 128), pieces of two such tiles (planned for tile_rows = 256), or tiles of at most 16 rows (decode
// steps; planned for tile_rows = 16 and key pieces that are multiples of 128); `n_tokens` is the number
// of rows of q.
static int paged_attention_tc_impl(const void* q, const void* k_slab, const void* v_slab,
                                   const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                   int n_segs, const int32_t* items, int n_items, float* part_o, float* part_ml,
                                   int n_slots, void* out, int n_tokens, int n_q_heads, int n_kv_heads,
                                   int head_dim, int page_size, int num_pages, float scale, int window,
                                   void* stream, TcForm form) {
  const bool pair = form == kTcPair, few = form == kTcFew;
  FTK_REQUIRE(q && k_slab && v_slab && block_table && seg_info && items && out, "paged_attention_tc: null pointer");
  FTK_REQUIRE(n_q_heads >= 1 && n_kv_heads >= 1 && n_q_heads % n_kv_heads == 0, "paged_attention_tc: %d query heads, %d KV heads",
              n_q_heads, n_kv_heads);
  FTK_REQUIRE(attention_tc_fits(head_dim, page_size, n_q_heads / n_kv_heads),
              "paged_attention_tc: head size %d, pages of %d, %d heads per KV head: takes head size 128, pages of a "
              "multiple of 16, at most 128 heads per KV head", head_dim, page_size, n_q_heads / n_kv_heads);
  FTK_REQUIRE(!few || attention_tc_few_fits(head_dim, page_size, n_q_heads / n_kv_heads),
              "paged_attention_tc: tiles of 16 rows take at most 16 heads per KV head, got %d", n_q_heads / n_kv_heads);
  FTK_REQUIRE(n_tokens >= 1 && n_items >= 0 && n_segs >= 1 && num_pages >= 1 && bt_stride >= 1,
              "paged_attention_tc: bad sizes");
  FTK_REQUIRE(window == 0, "paged_attention_tc: layers with a window run on the other kernels");
  FTK_REQUIRE(n_slots == 0 || (part_o && part_ml), "paged_attention_tc: split tiles need scratch");
  FTK_REQUIRE((((uintptr_t)q | (uintptr_t)k_slab | (uintptr_t)v_slab | (uintptr_t)out) & 15) == 0,
              "paged_attention_tc: 16-byte aligned tensors only");
  if (n_items == 0) return 0;
  AttnParams p;
  p.q = q; p.k = k_slab; p.v = v_slab; p.out = out;
  p.block_table = block_table; p.bt_stride = bt_stride;
  p.seg_info = seg_info; p.n_segs = n_segs; p.items = items; p.n_items = n_items;
  p.part_o = part_o; p.part_ml = part_ml; p.n_slots = n_slots;
  p.Hq = n_q_heads; p.Hkv = n_kv_heads; p.G = n_q_heads / n_kv_heads; p.D = head_dim; p.P = page_size;
  p.num_pages = num_pages; p.tile_rows = pair ? 2 * kTcRows : few ? kTcFewRows : kTcRows; p.scale = scale; p.window = window;
  p.sel = nullptr; p.sel_stride = 0; p.block_size = 0; p.arrivals = nullptr;
  cudaStream_t s = (cudaStream_t)stream;
  note_variant(pair ? "attention: tcgen05, two 128-row query tiles per CTA"
               : few ? "attention: tcgen05, tiles of at most 16 rows, one softmax warp"
                     : "attention: tcgen05, 128-row query tiles");
  const int rc = pair ? launch_attention_tc2(p, n_tokens, s) : launch_attention_tc(p, n_tokens, s);
  FTK_REQUIRE(rc == 0, "paged_attention_tc: cannot set up the kernel (%d)", rc);
  FTK_LAUNCH_CHECK("paged_attention_tc");
  if (n_slots > 0) {
    dim3 grid(n_items, n_kv_heads);
    // a CTA merges its share of a tile's rows, a warp a row at a time (three trips to memory one after the
    // other): tiles of 128 and 256 rows get as many warps as a tile cut in two has rows per CTA / 4
    const int threads = p.tile_rows >= 128 ? 512 : 128;  // (96 registers a thread)
    FTK_LAUNCH(attention_merge_kernel<__nv_bfloat16>, grid, threads, 0, s, p);
    FTK_LAUNCH_CHECK("paged_attention_tc merge");
  }
  return 0;
}

extern "C" int ftk_paged_attention_tc(const void* q, const void* k_slab, const void* v_slab,
                                      const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                      int n_segs, const int32_t* items, int n_items, float* part_o, float* part_ml,
                                      int n_slots, void* out, int n_tokens, int n_q_heads, int n_kv_heads,
                                      int head_dim, int page_size, int num_pages, float scale, int window,
                                      void* stream) {
  return paged_attention_tc_impl(q, k_slab, v_slab, block_table, bt_stride, seg_info, n_segs, items, n_items, part_o,
                                 part_ml, n_slots, out, n_tokens, n_q_heads, n_kv_heads, head_dim, page_size, num_pages,
                                 scale, window, stream, kTcSingle);
}

extern "C" int ftk_paged_attention_tc_pair(const void* q, const void* k_slab, const void* v_slab,
                                           const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                           int n_segs, const int32_t* items, int n_items, float* part_o,
                                           float* part_ml, int n_slots, void* out, int n_tokens, int n_q_heads,
                                           int n_kv_heads, int head_dim, int page_size, int num_pages, float scale,
                                           int window, void* stream) {
  return paged_attention_tc_impl(q, k_slab, v_slab, block_table, bt_stride, seg_info, n_segs, items, n_items, part_o,
                                 part_ml, n_slots, out, n_tokens, n_q_heads, n_kv_heads, head_dim, page_size, num_pages,
                                 scale, window, stream, kTcPair);
}

extern "C" int ftk_paged_attention_tc_few(const void* q, const void* k_slab, const void* v_slab,
                                          const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                          int n_segs, const int32_t* items, int n_items, float* part_o, float* part_ml,
                                          int n_slots, void* out, int n_tokens, int n_q_heads, int n_kv_heads,
                                          int head_dim, int page_size, int num_pages, float scale, int window,
                                          void* stream) {
  return paged_attention_tc_impl(q, k_slab, v_slab, block_table, bt_stride, seg_info, n_segs, items, n_items, part_o,
                                 part_ml, n_slots, out, n_tokens, n_q_heads, n_kv_heads, head_dim, page_size, num_pages,
                                 scale, window, stream, kTcFew);
}

static int paged_attention_impl(const void* q, const void* k_slab, const void* v_slab, int dtype,
                                const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                int n_segs, const int32_t* items, int n_items, float* part_o,
                                float* part_ml, int n_slots, void* out, int n_q_heads, int n_kv_heads,
                                int head_dim, int page_size, int num_pages, int tile_rows, float scale,
                                int window, const int32_t* sel, int sel_stride, int block_size, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "paged_attention: bad dtype %d", dtype);
  FTK_REQUIRE(n_items >= 0 && n_segs >= 0, "paged_attention: bad counts");
  if (n_items == 0) return 0;
  FTK_REQUIRE(q && k_slab && v_slab && block_table && seg_info && items && out, "paged_attention: null pointer");
  FTK_REQUIRE(n_kv_heads >= 1 && n_kv_heads <= 65535 && n_q_heads % n_kv_heads == 0,
              "paged_attention: %d query heads do not divide into %d KV heads", n_q_heads, n_kv_heads);
  FTK_REQUIRE(head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 256,
              "paged_attention: head_dim=%d must be a multiple of 16 in [16, 256]", head_dim);
  FTK_REQUIRE(page_size >= 1 && num_pages >= 1 && bt_stride >= 1, "paged_attention: bad page geometry");
  FTK_REQUIRE(window >= 0, "paged_attention: negative window");
  FTK_REQUIRE(n_slots == 0 || (part_o && part_ml), "paged_attention: split tiles need scratch");
  AttnParams p;
  p.q = q; p.k = k_slab; p.v = v_slab; p.out = out;
  p.block_table = block_table; p.bt_stride = bt_stride;
  p.seg_info = seg_info; p.n_segs = n_segs; p.items = items; p.n_items = n_items;
  p.part_o = part_o; p.part_ml = part_ml; p.n_slots = n_slots;
  p.Hq = n_q_heads; p.Hkv = n_kv_heads; p.G = n_q_heads / n_kv_heads; p.D = head_dim; p.P = page_size;
  p.num_pages = num_pages; p.tile_rows = tile_rows; p.scale = scale; p.window = window;
  p.sel = sel; p.sel_stride = sel_stride; p.block_size = block_size;
  p.arrivals = nullptr;
  if (sel) {
    FTK_REQUIRE(sel_stride >= 1 && block_size >= 1, "paged_attention: bad block selection geometry");
    FTK_REQUIRE(window == 0, "paged_attention: a window cannot be combined with block selection");
    FTK_REQUIRE(tile_rows == 16, "paged_attention: block selection works on one token per tile (16-row tiles), got %d",
                tile_rows);
  }
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_items, n_kv_heads);
  if (dtype == FTK_F32) {
    FTK_REQUIRE(tile_rows == kF32Rows, "paged_attention: the float32 kernel works on %d-row tiles, got %d",
                kF32Rows, tile_rows);
    FTK_REQUIRE(p.G <= kF32Rows, "paged_attention: %d query heads per KV head exceed the %d-row tile", p.G, kF32Rows);
    const size_t smem = ((size_t)kF32Rows * head_dim + (size_t)kF32Chunk * (2 * head_dim + 1)) * sizeof(float);
    note_variant(sel ? "attention: float32, block-sparse" : "attention: float32, warp per row");
    auto kern = attention_f32_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FTK_LAUNCH(kern, grid, kF32Rows * 32, smem, s, p);
    FTK_LAUNCH_CHECK("paged_attention (float32)");
    if (n_slots > 0) {
      FTK_LAUNCH(attention_merge_kernel<float>, grid, 128, 0, s, p);
      FTK_LAUNCH_CHECK("paged_attention merge");
    }
  } else {
    FTK_REQUIRE(tile_rows == kBM || tile_rows == kDecRows,
                "paged_attention: the bfloat16 kernels work on %d-row tiles (%d for decode steps), got %d", kBM,
                kDecRows, tile_rows);
    FTK_REQUIRE(p.G <= tile_rows, "paged_attention: %d query heads per KV head exceed the %d-row tile", p.G, tile_rows);
    bool merged = false;
    if (tile_rows == kDecRows) {
      if (n_slots > 0 && (long long)n_slots * p.Hkv <= kAttnArrivalSlots && p.D % 4 == 0) {
        // the counters live in this device's copy of the array: look the address up once per device
        static unsigned int* arrivals[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        FTK_REQUIRE(dev >= 0 && dev < 64, "paged_attention: device index %d out of range", dev);
        if (!arrivals[dev]) {
          FTK_REQUIRE(cudaGetSymbolAddress((void**)&arrivals[dev], g_attn_arrivals) == cudaSuccess,
                      "paged_attention: cannot find the arrival counters on device %d", dev);
        }
        p.arrivals = arrivals[dev];
        merged = true;
      }
      note_variant(sel ? "attention: bfloat16 mma.sync, 16-row tiles, block-sparse"
                       : merged ? "attention: bfloat16 mma.sync, 16-row tiles, last split merges"
                                : "attention: bfloat16 mma.sync, 16-row tiles");
      if (head_dim <= 64) launch_decode_bf16<64>(p, s);
      else if (head_dim <= 128) launch_decode_bf16<128>(p, s);
      else launch_decode_bf16<256>(p, s);
    } else {
      note_variant("attention: bfloat16 mma.sync, 64-row tiles");
      if (head_dim <= 64) launch_bf16<64>(p, s);
      else if (head_dim <= 128) launch_bf16<128>(p, s);
      else launch_bf16<256>(p, s);
    }
    FTK_LAUNCH_CHECK("paged_attention (bfloat16)");
    if (n_slots > 0 && !merged) {
      FTK_LAUNCH(attention_merge_kernel<__nv_bfloat16>, grid, 128, 0, s, p);
      FTK_LAUNCH_CHECK("paged_attention merge");
    }
  }
  return 0;
}

extern "C" int ftk_paged_attention(const void* q, const void* k_slab, const void* v_slab, int dtype,
                                   const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                   int n_segs, const int32_t* items, int n_items, float* part_o,
                                   float* part_ml, int n_slots, void* out, int n_q_heads, int n_kv_heads,
                                   int head_dim, int page_size, int num_pages, int tile_rows, float scale,
                                   int window, void* stream) {
  return paged_attention_impl(q, k_slab, v_slab, dtype, block_table, bt_stride, seg_info, n_segs, items, n_items, part_o,
                              part_ml, n_slots, out, n_q_heads, n_kv_heads, head_dim, page_size, num_pages, tile_rows,
                              scale, window, nullptr, 0, 0, stream);
}

// Block-sparse layers: `sel [T, n_kv_heads, sel_stride]` lists, per token and KV head, the chosen key
// blocks of `block_size` positions (ascending, -1 padded); the work items then hold one token each
// and their key ranges count chosen keys.
extern "C" int ftk_paged_attention_sparse(const void* q, const void* k_slab, const void* v_slab, int dtype,
                                          const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                          int n_segs, const int32_t* items, int n_items, float* part_o,
                                          float* part_ml, int n_slots, void* out, int n_q_heads, int n_kv_heads,
                                          int head_dim, int page_size, int num_pages, int tile_rows, float scale,
                                          const int32_t* sel, int sel_stride, int block_size, void* stream) {
  FTK_REQUIRE(sel != nullptr, "paged_attention_sparse: no block selection given");
  return paged_attention_impl(q, k_slab, v_slab, dtype, block_table, bt_stride, seg_info, n_segs, items, n_items, part_o,
                              part_ml, n_slots, out, n_q_heads, n_kv_heads, head_dim, page_size, num_pages, tile_rows,
                              scale, 0, sel, sel_stride, block_size, stream);
}

// ================================================================= entry point without allocation
// See no_alloc.h.  The split-tile scratch lives in this file-scope device array; host code must not
// pass the array's name to a kernel (on the host it is only a stand-in), so the device address is
// looked up once per device with cudaGetSymbolAddress and handed to the launch as a pointer.
#include "no_alloc.h"

static __device__ __align__(256) float g_static_scratch[FTK_STATIC_SCRATCH_BYTES / sizeof(float)];

static float* static_scratch_address() {
  constexpr int kMaxDevices = 64;
  static float* addr[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    ftk::set_error("paged_attention_static_scratch: cannot tell the current device");
    return nullptr;
  }
  if (!addr[dev]) {  // set-up, once per device, with that device current
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      ftk::set_error("paged_attention_static_scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    addr[dev] = static_cast<float*>(p);
  }
  return addr[dev];
}

extern "C" int ftk_paged_attention_static_scratch(const void* q, const void* k_slab, const void* v_slab, int dtype,
                                                  const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                                  int n_segs, const int32_t* items_host_copy, const int32_t* items,
                                                  int n_items, void* out, int n_q_heads, int n_kv_heads, int head_dim,
                                                  int page_size, int num_pages, int tile_rows, float scale, int window,
                                                  void* stream) {
  FTK_REQUIRE(n_items >= 0, "paged_attention_static_scratch: bad item count");
  FTK_REQUIRE(n_items == 0 || items_host_copy, "paged_attention_static_scratch: the host copy of the work list is needed to size the scratch");
  // bounded before anything is multiplied, so that the size below cannot wrap
  FTK_REQUIRE(n_kv_heads >= 1 && n_kv_heads <= 65535 && tile_rows >= 1 && tile_rows <= 256 && head_dim >= 1 &&
                  head_dim <= 256,
              "paged_attention_static_scratch: %d KV heads, tiles of %d rows, heads of %d: at most 65535, 256 and 256",
              n_kv_heads, tile_rows, head_dim);
  // slots the work list uses: a split tile owns slots [base, base + n_splits)
  const long long max_slots = FTK_STATIC_SCRATCH_BYTES / 8;  // a slot holds 8 bytes at the very least
  long long n_slots = 0;
  for (int i = 0; i < n_items; ++i) {
    const int32_t* w = items_host_copy + (size_t)i * 8;
    if (w[5] <= 1) continue;
    FTK_REQUIRE(w[5] <= 64 && w[7] >= 0 && (long long)w[7] + w[5] <= max_slots,
                "paged_attention_static_scratch: work item %d is split %d ways from slot %d: at most 64 splits, slots in "
                "[0, %lld)", i, w[5], w[7], max_slots);
    if ((long long)w[7] + w[5] > n_slots) n_slots = (long long)w[7] + w[5];
  }
  const long long rows = n_slots * n_kv_heads * tile_rows;
  const long long need = rows * (head_dim + 2) * (long long)sizeof(float);
  FTK_REQUIRE(need <= (long long)FTK_STATIC_SCRATCH_BYTES,
              "paged_attention_static_scratch: the work list needs %lld bytes of scratch, the static array holds %u "
              "(use ftk_paged_attention with your own scratch, or fewer splits)", need, FTK_STATIC_SCRATCH_BYTES);
  float* base = nullptr;
  if (n_slots > 0) {
    base = static_scratch_address();
    if (!base) return 3;
  }
  float* part_o = base;
  float* part_ml = base ? base + rows * head_dim : nullptr;
  return ftk_paged_attention(q, k_slab, v_slab, dtype, block_table, bt_stride, seg_info, n_segs, items, n_items,
                             part_o, part_ml, (int)n_slots, out, n_q_heads, n_kv_heads, head_dim, page_size, num_pages,
                             tile_rows, scale, window, stream);
}
