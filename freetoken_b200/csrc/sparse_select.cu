// Block selection of the block-sparse attention layers.
//
// For every new token and index head: the score of a key block is the largest
// index_q . index_k over the block's positions the token may see, unscaled
// (python/freetoken/kernel/triton/minimax_m3_sparse.py:152-170; NaN counts as -1e30, :238); the first
// `init_blocks` blocks score 1e30 and the newest `local_blocks` 1e29, the local ones winning an
// overlap (:232-244); the min(topk, visible) best blocks are taken, the lower block winning a tie
// (:269-284), and written in ascending order, padded with -1.  The reference does this with a score
// kernel plus a bitonic top-k kernel (and split/merge variants for decode); this first version is one
// CTA per (token, index head) that walks the visible blocks, which is exact but not yet fast for
// very long sequences.
#include "common.cuh"

namespace ftk {

constexpr int kSelThreads = 128;
constexpr int kMaxIndexDim = 256;

template <typename T>
__global__ void __launch_bounds__(kSelThreads) sparse_select_kernel(
    const T* __restrict__ iq, const T* __restrict__ ik_slab, const int32_t* __restrict__ block_table, int bt_stride,
    const int32_t* __restrict__ seg_info, int n_segs, int n_heads, int dim, int page_size, int num_pages,
    int block_size, int topk, int local_blocks, int init_blocks, int max_blocks, int32_t* __restrict__ sel) {
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
  for (int d = threadIdx.x; d < dim; d += blockDim.x) qv[d] = to_float(iq[((size_t)t * n_heads + h) * dim + d]);
  __syncthreads();
  for (int b = threadIdx.x; b < nb; b += blockDim.x) {
    float best = -INFINITY;
    const int p_end = min((b + 1) * block_size, pos + 1);
    for (int p = b * block_size; p < p_end; ++p) {
      const int page = block_table[(size_t)row * bt_stride + p / page_size];
      if (page < 0 || page >= num_pages) continue;
      const T* kr = ik_slab + ((size_t)page * page_size + p % page_size) * dim;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qv[d], to_float(kr[d]), dot);
      best = fmaxf(best, dot);
    }
    if (best != best) best = -1e30f;
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
      for (int w = 1; w < kSelThreads / 32; ++w) {
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

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_sparse_select(const void* iq, const void* ik_slab, int dtype, const int32_t* block_table,
                                 int bt_stride, const int32_t* seg_info, int n_segs, int n_tokens, int n_heads,
                                 int dim, int page_size, int num_pages, int block_size, int topk, int local_blocks,
                                 int init_blocks, int max_blocks, int32_t* sel, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "sparse_select: bad dtype %d", dtype);
  FTK_REQUIRE(n_tokens >= 0 && n_heads >= 1 && n_heads <= 65535 && dim >= 1 && dim <= kMaxIndexDim,
              "sparse_select: bad sizes (index dim up to %d)", kMaxIndexDim);
  FTK_REQUIRE(block_size >= 1 && topk >= 1 && local_blocks >= 0 && init_blocks >= 0 && max_blocks >= 1,
              "sparse_select: bad block geometry");
  FTK_REQUIRE(n_tokens <= 65535, "sparse_select: at most 65535 tokens per call");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(iq && ik_slab && block_table && seg_info && sel, "sparse_select: null pointer");
  const size_t smem = (size_t)max_blocks * (sizeof(float) + 1) + 16;
  FTK_REQUIRE(smem <= 160 * 1024, "sparse_select: %d blocks exceed what one CTA can rank", max_blocks);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_heads, n_tokens);
  if (dtype == FTK_F32) {
    auto kern = sparse_select_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FTK_LAUNCH(kern, grid, kSelThreads, smem, s, (const float*)iq, (const float*)ik_slab, block_table, bt_stride, seg_info, n_segs,
                                         n_heads, dim, page_size, num_pages, block_size, topk, local_blocks, init_blocks,
                                         max_blocks, sel);
  } else {
    auto kern = sparse_select_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FTK_LAUNCH(kern, grid, kSelThreads, smem, s, (const __nv_bfloat16*)iq, (const __nv_bfloat16*)ik_slab, block_table, bt_stride,
                                         seg_info, n_segs, n_heads, dim, page_size, num_pages, block_size, topk,
                                         local_blocks, init_blocks, max_blocks, sel);
  }
  FTK_LAUNCH_CHECK("sparse_select");
  return 0;
}
