// Router epilogue: scores, bias-corrected choice, top-k, renormalisation and scaling, all float32.
//
// sigmoid form (python/freetoken/models/minimax_m3/moe.py:71-81): s = sigmoid(logits); the experts
// are chosen by s + bias, weighted by the unbiased s, divided by their sum (+1e-20) and multiplied by
// the scaling factor.  softmax form (python/freetoken/moe/fused.py:27-31): s = softmax(logits).
// The logits themselves are a library matrix product in float32, as in the reference (F.linear).
// One warp per token; the largest choice goes first and the lower expert index wins a tie.
#include "common.cuh"

namespace ftk {

constexpr int kRouterWarps = 4;

__global__ void router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                   int n_tokens, int n_experts, int top_k, int scoring, float scale,
                                   int32_t* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouterWarps + warp;
  if (t >= n_tokens) return;
  float* s = sm + (size_t)warp * 2 * n_experts;  // unbiased scores
  float* c = s + n_experts;                      // scores the choice is made by
  const float* row = logits + (size_t)t * n_experts;
  if (scoring == FTK_SCORE_SIGMOID) {
    for (int e = lane; e < n_experts; e += 32) s[e] = 1.f / (1.f + expf(-row[e]));
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, row[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = expf(row[e] - mx);
      s[e] = v;
      sum += v;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < n_experts; e += 32) s[e] = s[e] / sum;
  }
  for (int e = lane; e < n_experts; e += 32) c[e] = bias ? s[e] + bias[e] : s[e];
  __syncwarp();
  float wsum = 0.f;
  for (int j = 0; j < top_k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = c[e];
      if (v > best) {  // ascending e within a lane: the first of equal values stays
        best = v;
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (bi == 0x7fffffff) bi = 0;  // every remaining choice is NaN or -inf
    const float w = s[bi];
    wsum += w;
    if (lane == 0) {
      ids[(size_t)t * top_k + j] = bi;
      weights[(size_t)t * top_k + j] = w;
      c[bi] = -INFINITY;
    }
    __syncwarp();
  }
  const float denom = scoring == FTK_SCORE_SIGMOID ? wsum + 1e-20f : wsum;
  if (lane < top_k || true) {
    for (int j = lane; j < top_k; j += 32) {
      const size_t i = (size_t)t * top_k + j;
      weights[i] = weights[i] / denom * scale;
    }
  }
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_router_topk(const float* logits, const float* bias, int n_tokens, int n_experts, int top_k,
                               int scoring, float scale, int32_t* ids, float* weights, void* stream) {
  FTK_REQUIRE(scoring == FTK_SCORE_SIGMOID || scoring == FTK_SCORE_SOFTMAX, "router_topk: unknown scoring %d", scoring);
  FTK_REQUIRE(n_experts >= 1 && top_k >= 1 && top_k <= n_experts, "router_topk: top_k=%d of %d experts", top_k, n_experts);
  FTK_REQUIRE(n_tokens >= 0, "router_topk: bad token count");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(logits && ids && weights, "router_topk: null pointer");
  const size_t smem = (size_t)kRouterWarps * 2 * n_experts * sizeof(float);
  FTK_REQUIRE(smem <= 200 * 1024, "router_topk: %d experts exceed what one block can hold (6400)", n_experts);
  if (smem > 48 * 1024) cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int blocks = (n_tokens + kRouterWarps - 1) / kRouterWarps;
  router_topk_kernel<<<blocks, kRouterWarps * 32, smem, (cudaStream_t)stream>>>(logits, bias, n_tokens, n_experts, top_k,
                                                                               scoring, scale, ids, weights);
  FTK_LAUNCH_CHECK("router_topk");
  return 0;
}
