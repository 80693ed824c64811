// Block selection of the block-sparse attention layers.
//
// For every new token and index head: the score of a key block is the largest
// index_q . index_k over the block's positions the token may see, unscaled
// (python/freetoken/kernel/triton/minimax_m3_sparse.py:152-170; a block with a NaN among its visible
// products counts as -1e30, :238); the first `init_blocks` blocks score 1e30 and the newest
// `local_blocks` 1e29, the local ones winning an overlap (:232-244); the min(topk, visible) best
// blocks are taken, the lower block winning a tie (:269-284), and written in ascending order, padded
// with -1.  The reference does this with a score kernel (tiled tl.dot, :105-179) plus a bitonic
// top-k kernel (and split/merge variants for decode).  Here:
//   * bfloat16: sparse_score_kernel contracts the index queries of up to 64 (token, head) rows with
//     one key block after the other on the tensor cores (mma.sync m16n8k16, the keys of a block staged
//     in shared memory through the block table with cp.async, two blocks in flight), takes the row
//     maximum over the block's visible keys and writes one float per (token, head, block); every key is
//     read once per tile of tokens, for all index heads together.  sparse_pick_kernel then ranks a
//     token's blocks.
//   * float32, and sizes the first kernel does not take: sparse_select_kernel, one CTA per (token,
//     head) that walks the visible blocks with plain 32-bit products and ranks them itself.
#include "common.cuh"

namespace ftk {

constexpr int kSelThreads = 128;
constexpr int kMaxIndexDim = 256;

// GIVEN: the blocks' scores are read from `given [T, n_heads, max_blocks]` (sparse_score_kernel wrote them)
// instead of being computed here.
template <typename T, bool GIVEN>
__global__ void __launch_bounds__(kSelThreads) sparse_select_kernel(
    const T* __restrict__ iq, const T* __restrict__ ik_slab, const int32_t* __restrict__ block_table, int bt_stride,
    const int32_t* __restrict__ seg_info, int n_segs, int n_heads, int dim, int page_size, int num_pages,
    int block_size, int topk, int local_blocks, int init_blocks, int max_blocks, int32_t* __restrict__ sel,
    const float* __restrict__ given) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sc[];          // [max_blocks] scores
  __shared__ float qv[kMaxIndexDim];
  __shared__ float red_v[kSelThreads / 32];
  __shared__ int red_i[kSelThreads / 32];
  __shared__ int chosen_block;
  unsigned char* pick = reinterpret_cast<unsigned char*>(sc + max_blocks);  // [max_blocks]
  const int h = blockIdx.x, t = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* out = sel + ((size_t)t * n_heads + h) * topk;
  // the token's segment
  int pos = -1, row = 0;
  for (int s = 0; s < n_segs; ++s) {
    const int q_start = seg_info[s * 4], q_len = seg_info[s * 4 + 1];
    if (t >= q_start && t < q_start + q_len) {
      pos = seg_info[s * 4 + 2] - q_len + (t - q_start);
      row = seg_info[s * 4 + 3];
    }
  }
  if (pos < 0) {
    for (int i = threadIdx.x; i < topk; i += blockDim.x) out[i] = -1;
    return;
  }
  int nb = pos / block_size + 1;
  if (nb > max_blocks) nb = max_blocks;  // the host sizes max_blocks for the longest request
  if (!GIVEN)
    for (int d = threadIdx.x; d < dim; d += blockDim.x) qv[d] = to_float(iq[((size_t)t * n_heads + h) * dim + d]);
  __syncthreads();
  for (int b = threadIdx.x; b < nb; b += blockDim.x) {
    if (GIVEN) {
      float best = __ldcg(given + ((size_t)t * n_heads + h) * max_blocks + b);
      if (b < init_blocks) best = 1e30f;
      if (b >= nb - local_blocks) best = 1e29f;
      sc[b] = best;
      pick[b] = 0;
      continue;
    }
    float best = -INFINITY;
    bool saw_nan = false;  // (fmaxf drops a NaN operand: it is remembered apart)
    const int p_end = min((b + 1) * block_size, pos + 1);
    for (int p = b * block_size; p < p_end; ++p) {
      const int page = block_table[(size_t)row * bt_stride + p / page_size];
      if (page < 0 || page >= num_pages) continue;
      const T* kr = ik_slab + ((size_t)page * page_size + p % page_size) * dim;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qv[d], to_float(kr[d]), dot);
      saw_nan = saw_nan || dot != dot;
      best = fmaxf(best, dot);
    }
    if (saw_nan) best = -1e30f;
    if (b < init_blocks) best = 1e30f;
    if (b >= nb - local_blocks) best = 1e29f;
    sc[b] = best;
    pick[b] = 0;
  }
  __syncthreads();
  const int k = min(topk, nb);
  for (int j = 0; j < k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
      const float v = sc[b];
      if (!pick[b] && (v > bv || (v == bv && b < bi))) {
        bv = v;
        bi = b;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      red_v[warp] = bv;
      red_i[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float v = red_v[0];
      int i = red_i[0];
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
        if (red_i[w] != 0x7fffffff && (i == 0x7fffffff || red_v[w] > v || (red_v[w] == v && red_i[w] < i))) {
          v = red_v[w];
          i = red_i[w];
        }
      }
      chosen_block = i;
      if (i != 0x7fffffff) pick[i] = 1;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int n = 0;
    for (int b = 0; b < nb && n < topk; ++b)
      if (pick[b]) out[n++] = b;
    for (; n < topk; ++n) out[n] = -1;
  }
}

// ---------------------------------------------------------------- ranking given scores
// The choice among a token's blocks when their scores are given (sparse_score_kernel wrote them): every
// thread keeps its share of the blocks in registers as order-preserving integers, and each of the top-k
// rounds is two block-wide reductions (the largest value, then the lowest block that has it) instead
// of a walk through shared memory: 16 rounds over 1,024 blocks take a microsecond or two.
__device__ __forceinline__ unsigned int pick_key(float v) {  // larger float <-> larger integer; 0 is kept for "no block"
  if (v != v) v = -1e30f;
  const unsigned int u = __float_as_uint(v + 0.f);
  const unsigned int k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return k == 0u ? 1u : k;
}

template <int PER>
__global__ void __launch_bounds__(kSelThreads) sparse_pick_kernel(
    const float* __restrict__ given, const int32_t* __restrict__ seg_info, int n_segs, int n_heads, int block_size,
    int topk, int local_blocks, int init_blocks, int max_blocks, int32_t* __restrict__ sel) {
  pdl_wait();
  pdl_trigger();
  __shared__ unsigned int red[kSelThreads / 32];
  __shared__ int chosen[64];
  const int h = blockIdx.x, t = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int32_t* out = sel + ((size_t)t * n_heads + h) * topk;
  int pos = -1;
  for (int s = 0; s < n_segs; ++s) {
    const int q_start = seg_info[s * 4], q_len = seg_info[s * 4 + 1];
    if (t >= q_start && t < q_start + q_len) pos = seg_info[s * 4 + 2] - q_len + (t - q_start);
  }
  if (pos < 0) {
    for (int i = tid; i < topk; i += blockDim.x) out[i] = -1;
    return;
  }
  int nb = pos / block_size + 1;
  if (nb > max_blocks) nb = max_blocks;
  const float* row = given + ((size_t)t * n_heads + h) * max_blocks;
  unsigned int key[PER];
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int b = q * kSelThreads + tid;
    float v = b < nb ? __ldcg(row + b) : 0.f;
    if (b < init_blocks) v = 1e30f;
    if (b >= nb - local_blocks) v = 1e29f;
    key[q] = b < nb ? pick_key(v) : 0u;
  }
  const int k = min(min(topk, nb), 64);
  auto block_max = [&](unsigned int v) {
    v = __reduce_max_sync(0xffffffffu, v);
    __syncthreads();  // (the round before is done with `red`)
    if (lane == 0) red[warp] = v;
    __syncthreads();
    unsigned int m = red[0];
#pragma unroll
    for (int w = 1; w < kSelThreads / 32; ++w) m = max(m, red[w]);
    return m;
  };
  for (int j = 0; j < k; ++j) {
    unsigned int best = 0u;
#pragma unroll
    for (int q = 0; q < PER; ++q) best = max(best, key[q]);
    const unsigned int top = block_max(best);
    // the lowest block with that value: as a maximum of inverted indices
    unsigned int mine = 0u;
    if (top != 0u) {
#pragma unroll
      for (int q = PER - 1; q >= 0; --q)
        if (key[q] == top) mine = 0xffffffffu - (unsigned)(q * kSelThreads + tid);
    }
    const unsigned int inv = block_max(mine);
    const int bi = top != 0u ? (int)(0xffffffffu - inv) : -1;
    if (bi >= 0 && bi % kSelThreads == tid) {
#pragma unroll
      for (int q = 0; q < PER; ++q)
        if (q == bi / kSelThreads) key[q] = 0u;
    }
    if (tid == 0) chosen[j] = bi;
  }
  __syncthreads();
  // ascending order: an entry's place is the number of chosen blocks below it
  if (tid < topk) {
    if (tid < k && chosen[tid] >= 0) {
      int rank = 0;
      for (int i = 0; i < k; ++i) rank += (chosen[i] >= 0 && chosen[i] < chosen[tid]) ? 1 : 0;
      out[rank] = chosen[tid];
    }
  }
  __syncthreads();
  int n_ok = 0;
  for (int i = 0; i < k; ++i) n_ok += chosen[i] >= 0 ? 1 : 0;
  for (int i = n_ok + tid; i < topk; i += blockDim.x) out[i] = -1;
}

// ---------------------------------------------------------------- scores on the tensor cores (bfloat16)
constexpr int kScoreRows = 64;     // (token, head) rows per CTA: four warps, one m16 tile each
constexpr int kScoreBlocksMin = 4;  // key blocks per CTA, at least (more when few tiles would leave too many CTAs short-lived)
constexpr int kScoreMaxDim = 256;  // index dim (multiple of 16)

__device__ __forceinline__ void sc_cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void sc_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (chunks of `blocks_per_cta` key blocks, token tiles).  A token tile holds up to 64 / n_heads consecutive
// tokens of one segment; tile y is found by walking the segments.
template <int KS_MAX>
__global__ void __launch_bounds__(128) sparse_score_kernel(
    const __nv_bfloat16* __restrict__ iq, const __nv_bfloat16* __restrict__ ik_slab,
    const int32_t* __restrict__ block_table, int bt_stride, const int32_t* __restrict__ seg_info, int n_segs,
    int n_heads, int dim, int page_size, int num_pages, int block_size, int max_blocks, int blocks_per_cta,
    float* __restrict__ scores) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char score_smem[];
  const int ld = dim + 8;  // elements per staged key row: the 16-byte pad keeps the fragment loads off each other's banks
  __nv_bfloat16* sk = reinterpret_cast<__nv_bfloat16*>(score_smem);  // [2][block_size][ld]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int tpt = max(1, kScoreRows / n_heads);  // tokens per tile
  // this CTA's tile: segment, first token, tokens
  int seg = -1, tok0 = 0, ntok = 0, q_start = 0, pos0 = 0, bt_row = 0;
  {
    int tile = blockIdx.y;
    for (int sidx = 0; sidx < n_segs; ++sidx) {
      const int q_len = seg_info[sidx * 4 + 1];
      const int n = (q_len + tpt - 1) / tpt;
      if (tile < n) {
        seg = sidx;
        tok0 = tile * tpt;
        ntok = min(tpt, q_len - tok0);
        q_start = seg_info[sidx * 4];
        pos0 = seg_info[sidx * 4 + 2] - q_len + tok0;  // position of the tile's first token
        bt_row = seg_info[sidx * 4 + 3];
        break;
      }
      tile -= n;
    }
  }
  if (seg < 0) return;
  const int last_pos = pos0 + ntok - 1;
  const int b_first = blockIdx.x * blocks_per_cta;
  if (b_first * block_size > last_pos) return;  // nothing of this chunk is visible to the tile
  const int b_end = min(min(b_first + blocks_per_cta, last_pos / block_size + 1), max_blocks);
  const int chunks = dim >> 3;  // 16-byte pieces per key
  auto stage = [&](int b, int buf) {
    __nv_bfloat16* dst = sk + (size_t)buf * block_size * ld;
#pragma unroll 4
    for (int i = threadIdx.x; i < block_size * chunks; i += blockDim.x) {
      const int j = i / chunks, c = i % chunks;
      const int p = b * block_size + j;
      bool valid = p <= last_pos;
      long long off = 0;
      if (valid) {
        const int page = block_table[(size_t)bt_row * bt_stride + p / page_size];
        valid = page >= 0 && page < num_pages;
        off = ((long long)page * page_size + p % page_size) * dim + c * 8;
      }
      sc_cp_async16(dst + (size_t)j * ld + c * 8, ik_slab + (valid ? off : 0), valid);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  stage(b_first, 0);
  // this warp's 16 rows: row r = token (r / n_heads) and head (r % n_heads) of the tile
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  const int n_rows = ntok * n_heads;
  const int ks_n = dim >> 4;
  uint32_t a[KS_MAX][4];
  {
    const __nv_bfloat16* q0 = iq + ((size_t)(q_start + tok0) * n_heads + min(r0, n_rows - 1)) * dim;
    const __nv_bfloat16* q1 = iq + ((size_t)(q_start + tok0) * n_heads + min(r1, n_rows - 1)) * dim;
#pragma unroll
    for (int ks = 0; ks < KS_MAX; ++ks) {
      if (ks < ks_n) {
        a[ks][0] = r0 < n_rows ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * tq) : 0u;
        a[ks][1] = r1 < n_rows ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * tq) : 0u;
        a[ks][2] = r0 < n_rows ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * tq) : 0u;
        a[ks][3] = r1 < n_rows ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * tq) : 0u;
      } else {
        a[ks][0] = a[ks][1] = a[ks][2] = a[ks][3] = 0u;
      }
    }
  }
  const int p_r0 = pos0 + r0 / n_heads, p_r1 = pos0 + r1 / n_heads;  // the rows' token positions
  for (int b = b_first; b < b_end; ++b) {
    const int buf = (b - b_first) & 1;
    if (b + 1 < b_end) {
      stage(b + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const __nv_bfloat16* kb = sk + (size_t)buf * block_size * ld;
    float m0 = -INFINITY, m1 = -INFINITY;
    bool nan0 = false, nan1 = false;
    const int nt_n = warp * 16 < n_rows ? block_size / 8 : 0;  // (a warp without rows only helps to stage keys)
    for (int nt = 0; nt < nt_n; ++nt) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      const __nv_bfloat16* krow = kb + (size_t)(nt * 8 + g) * ld + 2 * tq;
#pragma unroll
      for (int ks = 0; ks < KS_MAX; ++ks) {
        if (ks < ks_n) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks * 16);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks * 16 + 8);
          sc_mma(c, a[ks], b0, b1);
        }
      }
      const int kp = b * block_size + nt * 8 + 2 * tq;  // key position of c[0] and c[2]; c[1], c[3] one further
      if (kp <= p_r0) { nan0 = nan0 || c[0] != c[0]; m0 = fmaxf(m0, c[0]); }
      if (kp + 1 <= p_r0) { nan0 = nan0 || c[1] != c[1]; m0 = fmaxf(m0, c[1]); }
      if (kp <= p_r1) { nan1 = nan1 || c[2] != c[2]; m1 = fmaxf(m1, c[2]); }
      if (kp + 1 <= p_r1) { nan1 = nan1 || c[3] != c[3]; m1 = fmaxf(m1, c[3]); }
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
      m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
      nan0 = nan0 || __shfl_xor_sync(0xffffffffu, (int)nan0, o);
      nan1 = nan1 || __shfl_xor_sync(0xffffffffu, (int)nan1, o);
    }
    if (tq == 0) {
      if (r0 < n_rows && b * block_size <= p_r0)
        scores[((size_t)(q_start + tok0) * n_heads + r0) * max_blocks + b] = nan0 ? -1e30f : m0;
      if (r1 < n_rows && b * block_size <= p_r1)
        scores[((size_t)(q_start + tok0) * n_heads + r1) * max_blocks + b] = nan1 ? -1e30f : m1;
    }
    __syncthreads();  // everyone is done with this buffer before it is staged again
  }
}

}  // namespace ftk

using namespace ftk;

// Whether the tensor-core scoring takes these sizes (bfloat16 only; the caller then provides `scores`).
extern "C" int ftk_sparse_score_fits(int n_heads, int dim, int block_size) {
  return n_heads >= 1 && n_heads <= kScoreRows && dim >= 16 && dim <= kScoreMaxDim && dim % 16 == 0 &&
         block_size >= 8 && block_size % 8 == 0 && (size_t)2 * block_size * (dim + 8) * 2 <= 160 * 1024;
}

extern "C" int ftk_sparse_select(const void* iq, const void* ik_slab, int dtype, const int32_t* block_table,
                                 int bt_stride, const int32_t* seg_info, int n_segs, int n_tokens, int n_heads,
                                 int dim, int page_size, int num_pages, int block_size, int topk, int local_blocks,
                                 int init_blocks, int max_blocks, int live_blocks, int32_t* sel, float* scores,
                                 void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "sparse_select: bad dtype %d", dtype);
  FTK_REQUIRE(n_tokens >= 0 && n_heads >= 1 && n_heads <= 65535 && dim >= 1 && dim <= kMaxIndexDim,
              "sparse_select: bad sizes (index dim up to %d)", kMaxIndexDim);
  FTK_REQUIRE(block_size >= 1 && topk >= 1 && local_blocks >= 0 && init_blocks >= 0 && max_blocks >= 1,
              "sparse_select: bad block geometry");
  FTK_REQUIRE(n_tokens <= 65535, "sparse_select: at most 65535 tokens per call");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(iq && ik_slab && block_table && seg_info && sel, "sparse_select: null pointer");
  FTK_REQUIRE(n_segs >= 1, "sparse_select: no segments");
  const size_t smem = (size_t)max_blocks * (sizeof(float) + 1) + 16;
  FTK_REQUIRE(smem <= 160 * 1024, "sparse_select: %d blocks exceed what one CTA can rank", max_blocks);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_heads, n_tokens);
  const bool tensor_cores = dtype == FTK_BF16 && scores != nullptr && ftk_sparse_score_fits(n_heads, dim, block_size) &&
                            page_size >= 1 && (((uintptr_t)iq | (uintptr_t)ik_slab) & 15) == 0;
  if (tensor_cores) {
    const int tpt = kScoreRows / n_heads > 0 ? kScoreRows / n_heads : 1;
    const int tiles = n_segs + (n_tokens + tpt - 1) / tpt;  // an upper bound: a segment's last tile may be short
    FTK_REQUIRE(tiles <= 65535, "sparse_select: too many token tiles (%d)", tiles);
    // key blocks that any request of this step can hold (`live_blocks`, at most max_blocks) are cut into chunks
    // of a few per CTA: few enough that the CTAs about fill the GPU once (three fit an SM)
    const int live = live_blocks >= 1 && live_blocks < max_blocks ? live_blocks : max_blocks;
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int bpc = (int)(((long long)tiles * live + 3LL * sms - 1) / (3LL * sms));
    // (much work, as in a long portion of a prompt, is better cut finely: its CTAs then even out by themselves)
    bpc = bpc < kScoreBlocksMin || bpc > 16 ? kScoreBlocksMin : bpc;
    dim3 sgrid((live + bpc - 1) / bpc, tiles);
    const size_t ssmem = (size_t)2 * block_size * (dim + 8) * sizeof(__nv_bfloat16);
    note_variant("block scores: mma.sync contraction, a block of keys per turn");
#define FTK_SCORE(KS)                                                                                            \
    do {                                                                                                         \
      auto kern = sparse_score_kernel<KS>;                                                                       \
      if (ssmem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ssmem); \
      FTK_LAUNCH(kern, sgrid, 128, ssmem, s, (const __nv_bfloat16*)iq, (const __nv_bfloat16*)ik_slab, block_table,   \
                 bt_stride, seg_info, n_segs, n_heads, dim, page_size, num_pages, block_size, max_blocks, bpc, scores); \
    } while (0)
    if (dim <= 64) FTK_SCORE(4); else if (dim <= 128) FTK_SCORE(8); else FTK_SCORE(16);
#undef FTK_SCORE
    FTK_LAUNCH_CHECK("sparse_select (scores)");
    if (max_blocks <= 64 * kSelThreads && topk <= 64) {
      note_variant("block choice: scores in registers, two reductions a round");
      if (max_blocks <= 8 * kSelThreads)
        FTK_LAUNCH(sparse_pick_kernel<8>, grid, kSelThreads, 0, s, (const float*)scores, seg_info, n_segs, n_heads, block_size,
                   topk, local_blocks, init_blocks, max_blocks, sel);
      else
        FTK_LAUNCH(sparse_pick_kernel<64>, grid, kSelThreads, 0, s, (const float*)scores, seg_info, n_segs, n_heads, block_size,
                   topk, local_blocks, init_blocks, max_blocks, sel);
    } else {
      auto kern = sparse_select_kernel<__nv_bfloat16, true>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      FTK_LAUNCH(kern, grid, kSelThreads, smem, s, (const __nv_bfloat16*)iq, (const __nv_bfloat16*)ik_slab, block_table, bt_stride,
                 seg_info, n_segs, n_heads, dim, page_size, num_pages, block_size, topk, local_blocks, init_blocks,
                 max_blocks, sel, (const float*)scores);
    }
    FTK_LAUNCH_CHECK("sparse_select (choice)");
    return 0;
  }
  note_variant(dtype == FTK_F32 ? "block scores: float32, a CTA per token and head" : "block scores: bfloat16, a CTA per token and head");
  if (dtype == FTK_F32) {
    auto kern = sparse_select_kernel<float, false>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FTK_LAUNCH(kern, grid, kSelThreads, smem, s, (const float*)iq, (const float*)ik_slab, block_table, bt_stride, seg_info, n_segs,
                                         n_heads, dim, page_size, num_pages, block_size, topk, local_blocks, init_blocks,
                                         max_blocks, sel, (const float*)nullptr);
  } else {
    auto kern = sparse_select_kernel<__nv_bfloat16, false>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FTK_LAUNCH(kern, grid, kSelThreads, smem, s, (const __nv_bfloat16*)iq, (const __nv_bfloat16*)ik_slab, block_table, bt_stride,
                                         seg_info, n_segs, n_heads, dim, page_size, num_pages, block_size, topk,
                                         local_blocks, init_blocks, max_blocks, sel, (const float*)nullptr);
  }
  FTK_LAUNCH_CHECK("sparse_select");
  return 0;
}
