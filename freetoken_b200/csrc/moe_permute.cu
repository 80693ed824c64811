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

// ---------------------------------------------------------------- many routes (long steps)
// The same sort in three short passes.  The routes are cut into segments of kSegRoutes, one warp
// each.  Pass 1 counts every segment's routes per expert.  Pass 2 (one block) walks the segments in
// order per expert: a segment's count becomes the number of that expert's routes in earlier
// segments, the total becomes the expert's count, and a scan over the experts gives the offsets.
// Pass 3: a warp places its routes in order; lanes that hold the same expert find each other with
// match.any and take consecutive rows.  Integer counting only: the same result in every run.
constexpr int kSegRoutes = 128;
constexpr int kSegWarps = 4;
constexpr int kSegScratchInts = 4 * 1024 * 1024;
__device__ int g_seg_counts[kSegScratchInts];  // [segment][expert]

__global__ void __launch_bounds__(kSegWarps * 32)
moe_seg_count_kernel(const int32_t* __restrict__ ids, int n_routes, int n_experts, int* __restrict__ seg_counts) {
  pdl_wait();
  extern __shared__ int cnt[];  // [warp][expert]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kSegWarps * n_experts; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const int seg = blockIdx.x * kSegWarps + warp;
  const int r0 = seg * kSegRoutes;
  for (int i = lane; i < kSegRoutes; i += 32) {
    const int r = r0 + i;
    if (r < n_routes) {
      const int e = ids[r];
      if (e >= 0 && e < n_experts) atomicAdd(&cnt[warp * n_experts + e], 1);
    }
  }
  __syncthreads();
  if (r0 < n_routes)
    for (int e = lane; e < n_experts; e += 32) seg_counts[(size_t)seg * n_experts + e] = cnt[warp * n_experts + e];
}

__global__ void __launch_bounds__(1024)
moe_seg_scan_kernel(int n_segs, int n_experts, int* __restrict__ seg_counts, int32_t* __restrict__ counts,
                    int32_t* __restrict__ offsets) {
  pdl_wait();
  __shared__ int warp_tot[33];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  // An expert's segments are shared by the `parts` threads el, el + round, ...: each adds up its
  // stretch of segments, the stretches' totals are exchanged through shared memory, and each writes the
  // running sums of its stretch (one thread per expert walked all segments, sixteen loads at a time:
  // eight trips to memory for 128 segments).
  __shared__ int part_tot[1024];
  const int round = min((int)blockDim.x, (n_experts + 31) & ~31);  // experts per pass over the block
  const int parts = (int)blockDim.x / round;
  const int el = (int)threadIdx.x % round, q = (int)threadIdx.x / round;
  const int per = (n_segs + parts - 1) / parts;
  const int sg_lo = min(n_segs, q * per), sg_hi = min(n_segs, sg_lo + per);
  for (int e0 = 0; e0 < n_experts; e0 += round) {
    const int e = e0 + el;
    const bool active = e < n_experts && q < parts;
    int sum = 0;
    if (active) {
      for (int sg0 = sg_lo; sg0 < sg_hi; sg0 += 16) {  // sixteen loads in flight
        int v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u)
          v[u] = sg0 + u < sg_hi ? __ldcg(seg_counts + (size_t)(sg0 + u) * n_experts + e) : 0;
#pragma unroll
        for (int u = 0; u < 16; ++u) sum += v[u];
      }
    }
    part_tot[threadIdx.x] = active ? sum : 0;
    __syncthreads();
    int run = 0;  // the expert's total, in the thread of its first stretch; 0 in the others
    if (active) {
      int before = 0, total = 0;
      for (int q2 = 0; q2 < parts; ++q2) {
        const int v = part_tot[q2 * round + el];
        if (q2 < q) before += v;
        total += v;
      }
      for (int sg0 = sg_lo; sg0 < sg_hi; sg0 += 16) {
        int v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u)
          v[u] = sg0 + u < sg_hi ? __ldcg(seg_counts + (size_t)(sg0 + u) * n_experts + e) : 0;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          if (sg0 + u < sg_hi) seg_counts[(size_t)(sg0 + u) * n_experts + e] = before;
          before += v[u];
        }
      }
      if (q == 0) {
        run = total;
        counts[e] = total;
      }
    }
    const bool owner = active && q == 0;
    // exclusive scan of this round's totals over the block, on top of the rounds before
    int incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int nw = blockDim.x >> 5;
      int t = lane < nw ? warp_tot[lane] : 0;
      int ti = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, ti, o);
        if (lane >= o) ti += v;
      }
      warp_tot[lane] = ti - t;          // exclusive over the warps
      if (lane == 31) warp_tot[32] = ti;  // this round's total
    }
    __syncthreads();
    if (owner) offsets[e] = carry + warp_tot[warp] + incl - run;
    __syncthreads();
    if (threadIdx.x == 0) carry += warp_tot[32];
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[n_experts] = carry;
}

__global__ void __launch_bounds__(kSegWarps * 32)
moe_seg_place_kernel(const int32_t* __restrict__ ids, int n_routes, int n_experts, const int* __restrict__ seg_counts,
                     const int32_t* __restrict__ offsets, int32_t* __restrict__ sorted_routes,
                     int32_t* __restrict__ route_pos) {
  pdl_wait();
  extern __shared__ int run[];  // [warp][expert]: next free row of the expert for this segment
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = blockIdx.x * kSegWarps + warp;
  const int r0 = seg * kSegRoutes;
  int* mine = run + warp * n_experts;
  if (r0 < n_routes)
    for (int e = lane; e < n_experts; e += 32) mine[e] = offsets[e] + seg_counts[(size_t)seg * n_experts + e];
  __syncwarp();
  if (r0 < n_routes) {
    for (int i = 0; i < kSegRoutes; i += 32) {
      const int r = r0 + i + lane;
      int e = r < n_routes ? ids[r] : -1;
      if (e < 0 || e >= n_experts) e = -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      const int leader = __ffs(peers) - 1;
      const int rank = __popc(peers & ((1u << lane) - 1u));
      int base = 0;
      if (lane == leader && e >= 0) {
        base = mine[e];
        mine[e] = base + __popc(peers);
      }
      base = __shfl_sync(0xffffffffu, base, leader);
      __syncwarp();
      if (r < n_routes) {
        if (e >= 0) {
          sorted_routes[base + rank] = r;
          route_pos[r] = base + rank;
        } else {
          route_pos[r] = -1;  // no expert: no row
        }
      }
    }
  }
  if (blockIdx.x == 0) {  // rows nobody claimed (only when an id named no expert)
    const int end = offsets[n_experts];
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
  const int n_segs = (n_routes + kSegRoutes - 1) / kSegRoutes;
  const size_t seg_smem = (size_t)kSegWarps * n_experts * sizeof(int);
  if (n_routes > 2048 && (long long)n_segs * n_experts <= kSegScratchInts && seg_smem <= 48 * 1024) {
    static int* seg_counts_of[64] = {};  // the scratch lives in each device's copy of the array
    int dev = 0;
    cudaGetDevice(&dev);
    FTK_REQUIRE(dev >= 0 && dev < 64, "moe_permute: device index %d out of range", dev);
    if (!seg_counts_of[dev]) {
      FTK_REQUIRE(cudaGetSymbolAddress((void**)&seg_counts_of[dev], g_seg_counts) == cudaSuccess,
                  "moe_permute: cannot find the segment counters on device %d", dev);
    }
    int* seg_counts = seg_counts_of[dev];
    note_variant("route sort: three passes over 128-route segments");
    const int blocks = (n_segs + kSegWarps - 1) / kSegWarps;
    FTK_LAUNCH(moe_seg_count_kernel, blocks, kSegWarps * 32, seg_smem, s, topk_ids, n_routes, n_experts, seg_counts);
    FTK_LAUNCH_CHECK("moe_permute (segment counts)");
    FTK_LAUNCH(moe_seg_scan_kernel, 1, 1024, 0, s, n_segs, n_experts, seg_counts, expert_counts, expert_offsets);
    FTK_LAUNCH_CHECK("moe_permute (scan)");
    FTK_LAUNCH(moe_seg_place_kernel, blocks, kSegWarps * 32, seg_smem, s, topk_ids, n_routes, n_experts,
               (const int*)seg_counts, (const int32_t*)expert_offsets, sorted_routes, route_pos);
    FTK_LAUNCH_CHECK("moe_permute (segment place)");
    return 0;
  }
  note_variant("route sort: one block per expert");
  FTK_LAUNCH(moe_count_kernel, n_experts, kPermThreads, 0, s, topk_ids, n_routes, expert_counts);
  FTK_LAUNCH_CHECK("moe_permute (count)");
  FTK_LAUNCH(moe_place_kernel, n_experts, kPermThreads, 0, s, topk_ids, n_routes, n_experts, expert_counts, expert_offsets,
                                                      sorted_routes, route_pos);
  FTK_LAUNCH_CHECK("moe_permute (place)");
  return 0;
}
