// Grouped expert matrix products on CUDA cores: the true 32-bit path, and the path for sizes the
// tensor-core kernels refuse.
//
// Rows are sorted by expert (expert e owns rows [offsets[e], offsets[e+1])); the row counts are
// only known on the device, so the grid is an upper bound on the row tiles (ceil(R / BM) + E) and a
// block first finds the expert and rows of its tile by walking the offsets.
//   gemm1: out[r, n] = act(x[r] . W1[e][n], x[r] . W1[e][I + n])   (gate and up halves together,
//          activation fused; the two products are rounded to the storage dtype first, where the
//          reference stores them, python/freetoken/moe/fused_nvfp4.py:317-344)
//   gemm2: out[r, n] = (a[r] . W2[e][n]) * weight[route of r]      (weight on the 32-bit
//          accumulator, python/freetoken/kernel/triton/fused_moe.py:292-296)
// The K loop runs in a fixed order that does not depend on how many rows an expert got.
#include "common.cuh"

namespace ftk {

constexpr int kBM = 32, kBN = 64, kBK = 32;

// Find the expert and first row of row-tile `tile`; returns false when the tile is past the end.
__device__ __forceinline__ bool find_tile(const int32_t* offsets, int n_experts, int tile, int& e, int& row0,
                                          int& row_end) {
  int t = tile;
  for (int i = 0; i < n_experts; ++i) {
    const int a = offsets[i], b = offsets[i + 1];
    const int n = (b - a + kBM - 1) / kBM;
    if (t < n) {
      e = i;
      row0 = a + t * kBM;
      row_end = b;
      return true;
    }
    t -= n;
  }
  return false;
}

template <typename T, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                       const int32_t* __restrict__ offsets, int n_experts,
                                                       int K, int N, int w_rows,
                                                       const int32_t* __restrict__ sorted_routes,
                                                       const float* __restrict__ route_weights, int n_routes,
                                                       int act, float alpha, float limit, T* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  __shared__ float As[kBM][kBK + 1];
  __shared__ float Bs[kBN][kBK + 1];
  __shared__ float Bu[GATED ? kBN : 1][kBK + 1];
  __shared__ int tile_info[3];
  if (threadIdx.x == 0) {
    int e = -1, r0 = 0, re = 0;
    if (!find_tile(offsets, n_experts, blockIdx.y, e, r0, re)) e = -1;
    tile_info[0] = e;
    tile_info[1] = r0;
    tile_info[2] = re;
  }
  __syncthreads();
  const int e = tile_info[0], row0 = tile_info[1], row_end = tile_info[2];
  if (e < 0) return;
  const int n0 = blockIdx.x * kBN;
  const T* we = w + (size_t)e * w_rows * K;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;  // 16 x 16 threads: 2 rows x 4 cols each
  float acc[2][4] = {}, accu[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += kBK) {
    for (int i = threadIdx.x; i < kBM * kBK; i += 256) {
      const int r = i / kBK, k = i % kBK;
      const int row = row0 + r;
      As[r][k] = (row < row_end && k0 + k < K) ? to_float(x[(size_t)row * K + k0 + k]) : 0.f;
    }
    for (int i = threadIdx.x; i < kBN * kBK; i += 256) {
      const int n = i / kBK, k = i % kBK;
      const bool ok = n0 + n < N && k0 + k < K;
      Bs[n][k] = ok ? to_float(we[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
      if (GATED) Bu[n][k] = ok ? to_float(we[(size_t)(N + n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kBK; ++k) {
      const float a0 = As[ty * 2][k], a1 = As[ty * 2 + 1][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Bs[tx * 4 + j][k];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
        if (GATED) {
          const float u = Bu[tx * 4 + j][k];
          accu[0][j] = fmaf(a0, u, accu[0][j]);
          accu[1][j] = fmaf(a1, u, accu[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + ty * 2 + i;
    if (row >= row_end) continue;
    float wgt = 1.f;
    if (!GATED) {
      const int route = sorted_routes[row];
      wgt = (route >= 0 && route < n_routes) ? route_weights[route] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v;
      if (GATED) {
        const float g = to_float(from_float<T>(acc[i][j])), u = to_float(from_float<T>(accu[i][j]));
        v = gated_act(g, u, act, alpha, limit);
      } else {
        v = acc[i][j] * wgt;
      }
      out[(size_t)row * N + n] = from_float<T>(v);
    }
  }
}

}  // namespace ftk

using namespace ftk;

// Defined in moe_gemm_tc.cu: the tcgen05 kernels for bfloat16; return -1 when the sizes are not
// theirs (the caller then uses the kernels above).
int ftk_moe_gemm1_act_tc(const void* x, const void* w1, const int32_t* expert_offsets, int n_experts,
                         int n_routes, int hidden, int inter, int act, float alpha, float limit, void* out,
                         const int32_t* sorted_routes, int top_k, int n_tokens, cudaStream_t stream);
int ftk_moe_gemm2_tc(const void* a, const void* w2, const int32_t* expert_offsets, const int32_t* sorted_routes,
                     const float* topk_weights, int n_experts, int n_routes, int hidden, int inter, void* out,
                     cudaStream_t stream);

extern "C" int ftk_moe_gemm1_act(const void* x_sorted, const void* w1, int dtype, const int32_t* expert_offsets,
                                 int n_experts, int n_routes, int hidden, int inter, int act, float alpha,
                                 float limit, void* out, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "moe_gemm1_act: bad dtype %d", dtype);
  FTK_REQUIRE(act == FTK_ACT_SILU || act == FTK_ACT_SWIGLUOAI, "moe_gemm1_act: unknown activation %d", act);
  FTK_REQUIRE(n_experts >= 1 && n_routes >= 0 && hidden >= 1 && inter >= 1, "moe_gemm1_act: bad sizes");
  if (n_routes == 0) return 0;
  FTK_REQUIRE(x_sorted && w1 && expert_offsets && out, "moe_gemm1_act: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == FTK_BF16) {
    const int rc = ftk_moe_gemm1_act_tc(x_sorted, w1, expert_offsets, n_experts, n_routes, hidden, inter, act, alpha,
                                        limit, out, nullptr, 0, 0, s);
    if (rc >= 0) return rc;
  }
  const int tiles = (n_routes + kBM - 1) / kBM + n_experts;
  FTK_REQUIRE(tiles <= 65535, "moe_gemm1_act: too many row tiles (%d)", tiles);
  dim3 grid((inter + kBN - 1) / kBN, tiles);
  note_variant(dtype == FTK_F32 ? "expert gate/up product: float32 on CUDA cores" : "expert gate/up product: bfloat16 on CUDA cores");
  if (dtype == FTK_F32)
    FTK_LAUNCH((moe_gemm_kernel<float, true>), grid, 256, 0, s, (const float*)x_sorted, (const float*)w1, expert_offsets, n_experts,
                                                      hidden, inter, 2 * inter, nullptr, nullptr, n_routes, act, alpha,
                                                      limit, (float*)out);
  else
    FTK_LAUNCH((moe_gemm_kernel<__nv_bfloat16, true>), grid, 256, 0, s, (const __nv_bfloat16*)x_sorted, (const __nv_bfloat16*)w1,
                                                              expert_offsets, n_experts, hidden, inter, 2 * inter, nullptr,
                                                              nullptr, n_routes, act, alpha, limit, (__nv_bfloat16*)out);
  FTK_LAUNCH_CHECK("moe_gemm1_act");
  return 0;
}

// The same from the tokens' rows in their own order: the kernel gathers the rows of each expert itself
// (bfloat16 on the tensor cores only; ftk_moe_gemm1_gather_fits says whether the sizes are taken).
extern "C" int ftk_moe_gemm1_act_gather(const void* x, const void* w1, const int32_t* expert_offsets,
                                        const int32_t* sorted_routes, int top_k, int n_tokens, int n_experts,
                                        int n_routes, int hidden, int inter, int act, float alpha, float limit,
                                        void* out, void* stream) {
  FTK_REQUIRE(act == FTK_ACT_SILU || act == FTK_ACT_SWIGLUOAI, "moe_gemm1_act_gather: unknown activation %d", act);
  FTK_REQUIRE(n_experts >= 1 && n_routes >= 0 && hidden >= 1 && inter >= 1 && top_k >= 1 && n_tokens >= 1,
              "moe_gemm1_act_gather: bad sizes");
  if (n_routes == 0) return 0;
  FTK_REQUIRE(x && w1 && expert_offsets && sorted_routes && out, "moe_gemm1_act_gather: null pointer");
  const int rc = ftk_moe_gemm1_act_tc(x, w1, expert_offsets, n_experts, n_routes, hidden, inter, act, alpha, limit, out,
                                      sorted_routes, top_k, n_tokens, (cudaStream_t)stream);
  FTK_REQUIRE(rc >= 0, "moe_gemm1_act_gather: width %d, expert width %d, %d experts are not taken by the tensor-core "
              "kernel (ask ftk_moe_gemm1_gather_fits first; copy the rows with moe_gather otherwise)", hidden, inter, n_experts);
  return rc;
}

extern "C" int ftk_moe_gemm2(const void* a, const void* w2, int dtype, const int32_t* expert_offsets,
                             const int32_t* sorted_routes, const float* topk_weights, int n_experts, int n_routes,
                             int hidden, int inter, void* out, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "moe_gemm2: bad dtype %d", dtype);
  FTK_REQUIRE(n_experts >= 1 && n_routes >= 0 && hidden >= 1 && inter >= 1, "moe_gemm2: bad sizes");
  if (n_routes == 0) return 0;
  FTK_REQUIRE(a && w2 && expert_offsets && sorted_routes && topk_weights && out, "moe_gemm2: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == FTK_BF16) {
    const int rc = ftk_moe_gemm2_tc(a, w2, expert_offsets, sorted_routes, topk_weights, n_experts, n_routes, hidden,
                                    inter, out, s);
    if (rc >= 0) return rc;
  }
  const int tiles = (n_routes + kBM - 1) / kBM + n_experts;
  FTK_REQUIRE(tiles <= 65535, "moe_gemm2: too many row tiles (%d)", tiles);
  dim3 grid((hidden + kBN - 1) / kBN, tiles);
  note_variant(dtype == FTK_F32 ? "expert down product: float32 on CUDA cores" : "expert down product: bfloat16 on CUDA cores");
  if (dtype == FTK_F32)
    FTK_LAUNCH((moe_gemm_kernel<float, false>), grid, 256, 0, s, (const float*)a, (const float*)w2, expert_offsets, n_experts, inter,
                                                       hidden, hidden, sorted_routes, topk_weights, n_routes, 0, 0.f, 0.f,
                                                       (float*)out);
  else
    FTK_LAUNCH((moe_gemm_kernel<__nv_bfloat16, false>), grid, 256, 0, s, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w2,
                                                               expert_offsets, n_experts, inter, hidden, hidden,
                                                               sorted_routes, topk_weights, n_routes, 0, 0.f, 0.f,
                                                               (__nv_bfloat16*)out);
  FTK_LAUNCH_CHECK("moe_gemm2");
  return 0;
}
