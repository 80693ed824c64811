// Sorting a step's routes by expert (counting sort, stable).
//
// Route r = t * top_k + j goes to expert ids[r].  Kernel 1 counts the routes of each expert (one
// block per expert).  Kernel 2 turns the counts into offsets and places the routes: block e walks
// all routes in order and gives its own the next free rows, so rows of one expert keep the order
// of the routes.  No atomics, so the result is the same in every run.  The reference pads each
// expert's rows to the GEMM tile (python/freetoken/kernel/triton/fused_moe.py:5-108); the grouped
// GEMMs here take ragged row counts, so nothing is padded.
#include "common.cuh"

namespace ftk {

constexpr int kPermThreads = 256;

__global__ void moe_count_kernel(const int32_t* __restrict__ ids, int n_routes, int32_t* __restrict__ counts) {
  pdl_wait();
  __shared__ float red[33];
  const int e = blockIdx.x;
  int n = 0;
  for (int r = threadIdx.x; r < n_routes; r += blockDim.x) n += ids[r] == e;
  // counts are far below 2^24, so the float reduction is exact
  const float total = block_sum((float)n, red);
  if (threadIdx.x == 0) counts[e] = (int)total;
}

__global__ void moe_place_kernel(const int32_t* __restrict__ ids, int n_routes, int n_experts,
                                 const int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                 int32_t* __restrict__ sorted_routes, int32_t* __restrict__ route_pos) {
  pdl_wait();
  __shared__ float red[33];
  __shared__ int warp_base[kPermThreads / 32 + 1];
  __shared__ int run;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int before = 0;
  for (int i = threadIdx.x; i < e; i += blockDim.x) before += counts[i];
  const int offset = (int)block_sum((float)before, red);
  if (threadIdx.x == 0) {
    offsets[e] = offset;
    if (e == n_experts - 1) offsets[n_experts] = offset + counts[e];
    run = 0;
  }
  __syncthreads();
  for (int r0 = 0; r0 < n_routes; r0 += blockDim.x) {
    const int r = r0 + threadIdx.x;
    const int id = r < n_routes ? ids[r] : -1;
    const bool mine = id == e;
    const unsigned ball = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) warp_base[warp] = __popc(ball);
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = run;
      for (int w = 0; w < kPermThreads / 32; ++w) {
        const int c = warp_base[w];
        warp_base[w] = acc;
        acc += c;
      }
      run = acc;
    }
    __syncthreads();
    if (mine) {
      const int pos = offset + warp_base[warp] + __popc(ball & ((1u << lane) - 1u));
      sorted_routes[pos] = r;
      route_pos[r] = pos;
    }
    if (e == 0 && r < n_routes && (id < 0 || id >= n_experts)) route_pos[r] = -1;  // no expert: no row
    __syncthreads();
  }
  if (e == n_experts - 1) {  // rows nobody claimed (only when an id named no expert)
    const int end = offset + counts[e];
    for (int i = end + threadIdx.x; i < n_routes; i += blockDim.x) sorted_routes[i] = -1;
  }
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_moe_permute(const int32_t* topk_ids, int n_tokens, int top_k, int n_experts,
                               int32_t* expert_counts, int32_t* expert_offsets, int32_t* sorted_routes,
                               int32_t* route_pos, void* stream) {
  FTK_REQUIRE(n_tokens >= 0 && top_k >= 1 && n_experts >= 1, "moe_permute: bad sizes");
  FTK_REQUIRE((long long)n_tokens * top_k < (1 << 24), "moe_permute: %lld routes exceed 2^24", (long long)n_tokens * top_k);
  FTK_REQUIRE(expert_counts && expert_offsets && (n_tokens == 0 || (topk_ids && sorted_routes && route_pos)),
              "moe_permute: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int n_routes = n_tokens * top_k;
  FTK_LAUNCH(moe_count_kernel, n_experts, kPermThreads, 0, s, topk_ids, n_routes, expert_counts);
  FTK_LAUNCH_CHECK("moe_permute (count)");
  FTK_LAUNCH(moe_place_kernel, n_experts, kPermThreads, 0, s, topk_ids, n_routes, n_experts, expert_counts, expert_offsets,
                                                      sorted_routes, route_pos);
  FTK_LAUNCH_CHECK("moe_permute (place)");
  return 0;
}
