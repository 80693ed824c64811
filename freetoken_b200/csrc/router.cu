// Router epilogue: scores, bias-corrected choice, top-k, renormalisation and scaling, all float32.
//
// sigmoid form (python/freetoken/models/minimax_m3/moe.py:71-81): s = sigmoid(logits); the experts
// are chosen by s + bias, weighted by the unbiased s, divided by their sum (+1e-20) and multiplied by
// the scaling factor.  softmax form (python/freetoken/moe/fused.py:27-31): s = softmax(logits).
// One warp per token; the largest choice goes first and the lower expert index wins a tie.
// For long steps the logits are a library matrix product in float32, as in the reference (F.linear),
// and router_topk_kernel takes them; for short steps moe_route_kernel computes them itself and also
// sorts the routes by expert, all in one launch.
#include "common.cuh"

namespace ftk {

constexpr int kRouterWarps = 4;

// A token's logit of expert e: the row holds n_parts blocks of n_experts values that are added in their
// order (one block: the logits themselves; three: the products of the activations with the three
// bfloat16 pieces of the float32 router weights, largest first).
__device__ __forceinline__ float logit_of(const float* __restrict__ row, int e, int n_experts, int n_parts) {
  float v = __ldcg(row + e);
  for (int q = 1; q < n_parts; ++q) v += __ldcg(row + (size_t)q * n_experts + e);
  return v;
}

// Scores, choice and weights of one token, by one warp.  `s` and `c` hold n_experts floats each.
__device__ __forceinline__ void route_token(const float* __restrict__ row, int n_parts, const float* __restrict__ bias,
                                            int n_experts, int top_k, int scoring, float scale, float* s, float* c,
                                            int32_t* __restrict__ ids, float* __restrict__ weights,
                                            int32_t* ids_copy) {
  const int lane = threadIdx.x & 31;
  if (scoring == FTK_SCORE_SIGMOID) {
    for (int e = lane; e < n_experts; e += 32) s[e] = 1.f / (1.f + expf(-logit_of(row, e, n_experts, n_parts)));
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, logit_of(row, e, n_experts, n_parts));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = expf(logit_of(row, e, n_experts, n_parts) - mx);
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
      ids[j] = bi;
      if (ids_copy) ids_copy[j] = bi;
      weights[j] = w;
      c[bi] = -INFINITY;
    }
    __syncwarp();
  }
  const float denom = scoring == FTK_SCORE_SIGMOID ? wsum + 1e-20f : wsum;
  for (int j = lane; j < top_k; j += 32) weights[j] = weights[j] / denom * scale;
}

// The same with the token's scores in registers (n_experts <= 32 * PER): the largest remaining choice
// is found with two warp reductions, first over the values (as order-preserving integers, NaN lowest),
// then over the indices of those that have it.  Same results as route_token.
__device__ __forceinline__ unsigned int order_key(float v) {
  if (v != v) return 0u;
  const unsigned int u = __float_as_uint(v + 0.f);  // -0 becomes +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <int PER>
__device__ __forceinline__ void route_token_regs(const float* __restrict__ row, int n_parts, const float* __restrict__ bias,
                                                 int n_experts, int top_k, int scoring, float scale, float* wbuf,
                                                 int32_t* __restrict__ ids, float* __restrict__ weights,
                                                 int32_t* ids_copy) {
  const int lane = threadIdx.x & 31;
  float sv[PER];
  unsigned int key[PER];
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int e = q * 32 + lane;
    sv[q] = e < n_experts ? logit_of(row, e, n_experts, n_parts) : -INFINITY;
  }
  if (scoring == FTK_SCORE_SIGMOID) {
#pragma unroll
    for (int q = 0; q < PER; ++q) sv[q] = 1.f / (1.f + expf(-sv[q]));
  } else {
    float mx = -INFINITY;
#pragma unroll
    for (int q = 0; q < PER; ++q) mx = fmaxf(mx, sv[q]);
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int q = 0; q < PER; ++q) {
      sv[q] = q * 32 + lane < n_experts ? expf(sv[q] - mx) : 0.f;
      sum += sv[q];
    }
    // the sum runs over experts in the order route_token takes them: lane by lane, then across lanes
    sum = warp_sum(sum);
#pragma unroll
    for (int q = 0; q < PER; ++q) sv[q] = sv[q] / sum;
  }
  const unsigned int floor_key = order_key(-INFINITY);  // never chosen: -inf and NaN
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int e = q * 32 + lane;
    key[q] = e < n_experts ? order_key(bias ? sv[q] + bias[e] : sv[q]) : 0u;
  }
  float wsum = 0.f;
  for (int j = 0; j < top_k; ++j) {
    unsigned int best = 0u;
    int slot = 0;
#pragma unroll
    for (int q = 0; q < PER; ++q)
      if (key[q] > best) {
        best = key[q];
        slot = q;
      }
    const unsigned int top = __reduce_max_sync(0xffffffffu, best);
    int bi = 0;
    if (top > floor_key) bi = (int)__reduce_min_sync(0xffffffffu, best == top ? (unsigned)(slot * 32 + lane) : 0x7fffffffu);
    const int owner = bi & 31, oslot = bi >> 5;
    float mine = 0.f;
#pragma unroll
    for (int q = 0; q < PER; ++q)
      if (q == oslot) mine = sv[q];
    const float w = __shfl_sync(0xffffffffu, mine, owner);
    wsum += w;
    if (lane == owner && top > floor_key) {
#pragma unroll
      for (int q = 0; q < PER; ++q)
        if (q == oslot) key[q] = 0u;
    }
    if (lane == 0) {
      ids[j] = bi;
      if (ids_copy) ids_copy[j] = bi;
      wbuf[j] = w;
    }
  }
  __syncwarp();
  const float denom = scoring == FTK_SCORE_SIGMOID ? wsum + 1e-20f : wsum;
  for (int j = lane; j < top_k; j += 32) weights[j] = wbuf[j] / denom * scale;
  __syncwarp();
}

// One token by one warp, in registers where the experts fit; `s` holds 2 * n_experts floats.
__device__ __forceinline__ void route_one(const float* __restrict__ row, int n_parts, const float* __restrict__ bias, int n_experts,
                                          int top_k, int scoring, float scale, float* s, int32_t* __restrict__ ids,
                                          float* __restrict__ weights, int32_t* ids_copy) {
  if (n_experts <= 128)
    route_token_regs<4>(row, n_parts, bias, n_experts, top_k, scoring, scale, s, ids, weights, ids_copy);
  else if (n_experts <= 256)
    route_token_regs<8>(row, n_parts, bias, n_experts, top_k, scoring, scale, s, ids, weights, ids_copy);
  else if (n_experts <= 512)
    route_token_regs<16>(row, n_parts, bias, n_experts, top_k, scoring, scale, s, ids, weights, ids_copy);
  else
    route_token(row, n_parts, bias, n_experts, top_k, scoring, scale, s, s + n_experts, ids, weights, ids_copy);
}

__global__ void router_topk_kernel(const float* __restrict__ logits, int n_parts, const float* __restrict__ bias,
                                   int n_tokens, int n_experts, int top_k, int scoring, float scale,
                                   int32_t* __restrict__ ids, float* __restrict__ weights) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x * kRouterWarps + warp;
  if (t >= n_tokens) return;
  float* s = sm + (size_t)warp * 2 * n_experts;  // unbiased scores
  route_one(logits + (size_t)t * n_parts * n_experts, n_parts, bias, n_experts, top_k, scoring, scale, s,
            ids + (size_t)t * top_k, weights + (size_t)t * top_k, nullptr);
}

// The whole routing of a small step in one launch: router logits (a float32 matrix-vector product
// per token, python/freetoken/models/minimax_m3/moe.py:71-73), then, in the block that finishes
// last, the choice of every token (route_one) and the sort of the routes by expert (what moe_permute
// does).  A block holds kRouteExperts experts; its warps share their weight rows (a thread's piece of
// them is on its way before the kernel waits for the one before it) and add their parts in a fixed
// order, so a token's logits never depend on the batch.  Blocks count their arrival in
// g_route_arrivals; nobody waits for anybody.
constexpr int kRouteWarps = 24;   // all of them share the block's weight rows, each a part of the width
constexpr int kRouteExperts = 2;  // experts per block: a token's activations are loaded once for all of them
constexpr int kRouteTokens = 8;   // tokens per pass over the weight rows
constexpr int kRouteVals = kRouteExperts * kRouteTokens;  // sums a thread carries
static_assert(kRouteVals == 16, "warp_sum16 adds sixteen values per lane");
__device__ unsigned int g_route_arrivals = 0;

// Sixteen sums over the warp with sixteen shuffles: the lanes swap halves of what they carry and keep
// the other half, four times; lanes 2 i and 2 i + 1 end up with the warp's sum of value i.
__device__ __forceinline__ float warp_sum16(float (&v)[16], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float give = b4 ? v[i] : v[i + 8], keep = b4 ? v[i + 8] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float give = b3 ? v[i] : v[i + 4], keep = b3 ? v[i + 4] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float give = b2 ? v[i] : v[i + 2], keep = b2 ? v[i + 2] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, give, 4);
  }
  {
    const float give = b1 ? v[0] : v[1], keep = b1 ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, give, 2);
  }
  return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}

__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                 int n_tokens, int hidden, int n_experts, int top_k, int scoring, float scale,
                 float* __restrict__ logits, int32_t* __restrict__ ids, float* __restrict__ weights,
                 int32_t* __restrict__ counts, int32_t* __restrict__ offsets, int32_t* __restrict__ routes,
                 int32_t* __restrict__ pos, int do_sort) {
  extern __shared__ float sm[];
  __shared__ float part[kRouteVals][kRouteWarps + 1];
  __shared__ bool last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e0 = blockIdx.x * kRouteExperts;
  const int h4 = hidden >> 2;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const float4* x4 = reinterpret_cast<const float4*>(x);
  // the router's weights never depend on the kernel before: a thread's first pieces of them are on
  // their way before the wait
  float4 w_first[kRouteExperts];
#pragma unroll
  for (int j = 0; j < kRouteExperts; ++j)
    w_first[j] = tid < h4 ? __ldg(w4 + (size_t)min(e0 + j, n_experts - 1) * h4 + tid) : make_float4(0.f, 0.f, 0.f, 0.f);
  pdl_wait();
  // every block fetches the bias now, under the matrix product, so that the one that turns out to
  // be last does not wait for it
  float* sbias = sm + (size_t)kRouteWarps * 2 * n_experts;
  if (bias)
    for (int i = tid; i < n_experts; i += blockDim.x) sbias[i] = __ldg(bias + i);
  for (int t0 = 0; t0 < n_tokens; t0 += kRouteTokens) {
    const int nt = min(kRouteTokens, n_tokens - t0);
    float acc[kRouteVals];  // [expert][token]
#pragma unroll
    for (int i = 0; i < kRouteVals; ++i) acc[i] = 0.f;
#pragma unroll 2
    for (int i = tid; i < h4; i += kRouteWarps * 32) {
      float4 wv[kRouteExperts], xv[kRouteTokens];
#pragma unroll
      for (int j = 0; j < kRouteExperts; ++j)
        wv[j] = i == tid ? w_first[j] : __ldg(w4 + (size_t)min(e0 + j, n_experts - 1) * h4 + i);
#pragma unroll
      for (int u = 0; u < kRouteTokens; ++u)  // (rows past the step's tokens are never stored: no load for them)
        xv[u] = u < nt ? __ldg(x4 + (size_t)(t0 + u) * h4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < kRouteExperts; ++j)
#pragma unroll
        for (int u = 0; u < kRouteTokens; ++u) {
          float a = acc[j * kRouteTokens + u];
          a = fmaf(wv[j].x, xv[u].x, a);
          a = fmaf(wv[j].y, xv[u].y, a);
          a = fmaf(wv[j].z, xv[u].z, a);
          a = fmaf(wv[j].w, xv[u].w, a);
          acc[j * kRouteTokens + u] = a;
        }
    }
    const float total = warp_sum16(acc, lane);
    if (!(lane & 1)) part[lane >> 1][warp] = total;
    __syncthreads();
    if (tid < kRouteVals) {
      const int j = tid / kRouteTokens, u = tid % kRouteTokens;
      if (u < nt && e0 + j < n_experts) {
        float v = part[tid][0];
#pragma unroll
        for (int q = 1; q < kRouteWarps; ++q) v += part[tid][q];
        logits[(size_t)(t0 + u) * n_experts + e0 + j] = v;
      }
    }
    __syncthreads();
  }
  if (tid < kRouteVals) __threadfence();
  __syncthreads();
  if (tid == 0) last = atomicAdd(&g_route_arrivals, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  // ---- the last block: every token's choice
  const int n_routes = n_tokens * top_k;
  int* sid = reinterpret_cast<int*>(sbias + n_experts);  // n_routes: the routes' experts
  float* s = sm + (size_t)warp * 2 * n_experts;
  for (int t = warp; t < n_tokens; t += kRouteWarps)
    route_one(logits + (size_t)t * n_experts, 1, bias ? sbias : nullptr, n_experts, top_k, scoring, scale, s,
              ids + (size_t)t * top_k, weights + (size_t)t * top_k, do_sort ? sid + (size_t)t * top_k : nullptr);
  if (!do_sort) {  // the caller's kernels take the routes in token order
    if (tid == 0) g_route_arrivals = 0;
    return;
  }
  __syncthreads();
  // ---- the routes sorted by expert; rows of one expert keep the order of the routes.  A route's
  // place is the number of routes that come before it, an expert's offset the number of routes to
  // experts below it: every thread counts for itself, nothing is scanned or scattered.
  for (int r = tid; r < n_routes; r += blockDim.x) {
    const int e = sid[r];
    int before = 0;
    for (int q = 0; q < n_routes; ++q) {
      const int eq = sid[q];
      before += (eq < e || (eq == e && q < r)) ? 1 : 0;
    }
    routes[before] = r;
    pos[r] = before;
  }
  for (int i = tid; i <= n_experts; i += blockDim.x) {
    int below = 0, same = 0;
    for (int q = 0; q < n_routes; ++q) {
      const int eq = sid[q];
      below += eq < i ? 1 : 0;
      same += eq == i ? 1 : 0;
    }
    offsets[i] = below;
    if (i < n_experts) counts[i] = same;
  }
  if (tid == 0) g_route_arrivals = 0;  // every block has arrived: ready for the next launch
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_router_topk(const float* logits, int n_parts, const float* bias, int n_tokens, int n_experts, int top_k,
                               int scoring, float scale, int32_t* ids, float* weights, void* stream) {
  FTK_REQUIRE(n_parts >= 1 && n_parts <= 4, "router_topk: %d blocks of logits per token (1 to 4)", n_parts);
  FTK_REQUIRE(scoring == FTK_SCORE_SIGMOID || scoring == FTK_SCORE_SOFTMAX, "router_topk: unknown scoring %d", scoring);
  FTK_REQUIRE(n_experts >= 1 && top_k >= 1 && top_k <= n_experts, "router_topk: top_k=%d of %d experts", top_k, n_experts);
  FTK_REQUIRE(n_tokens >= 0, "router_topk: bad token count");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(logits && ids && weights, "router_topk: null pointer");
  const size_t smem = (size_t)kRouterWarps * 2 * n_experts * sizeof(float);
  FTK_REQUIRE(smem <= 200 * 1024, "router_topk: %d experts exceed what one block can hold (6400)", n_experts);
  if (smem > 48 * 1024) cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int blocks = (n_tokens + kRouterWarps - 1) / kRouterWarps;
  note_variant(n_parts > 1 ? "routing: expert choice from logits given in pieces" : "routing: expert choice from given logits");
  FTK_LAUNCH(router_topk_kernel, blocks, kRouterWarps * 32, smem, (cudaStream_t)stream, logits, n_parts, bias, n_tokens, n_experts, top_k,
                                                                               scoring, scale, ids, weights);
  FTK_LAUNCH_CHECK("router_topk");
  return 0;
}

static size_t route_smem(int n_tokens, int n_experts, int top_k) {
  return (size_t)(kRouteWarps * 2 + 1) * n_experts * sizeof(float) + (size_t)(n_tokens * top_k) * sizeof(int);
}

extern "C" int ftk_moe_route_fits(int n_tokens, int hidden, int n_experts, int top_k) {
  return n_tokens >= 1 && n_tokens <= 32 && hidden % 4 == 0 && n_experts >= 1 && top_k >= 1 && top_k <= n_experts &&
         route_smem(n_tokens, n_experts, top_k) <= 160 * 1024;
}

extern "C" int ftk_moe_route(const float* x, const float* gate_w, const float* bias, int n_tokens, int hidden,
                             int n_experts, int top_k, int scoring, float scale, float* logits, int32_t* ids,
                             float* weights, int32_t* counts, int32_t* offsets, int32_t* routes, int32_t* pos,
                             int do_sort, void* stream) {
  FTK_REQUIRE(scoring == FTK_SCORE_SIGMOID || scoring == FTK_SCORE_SOFTMAX, "moe_route: unknown scoring %d", scoring);
  FTK_REQUIRE(ftk_moe_route_fits(n_tokens, hidden, n_experts, top_k),
              "moe_route: %d tokens, width %d, %d experts, top %d do not fit the one-launch routing (at most 32 tokens, "
              "a width that is a multiple of 4); use the matrix product + router_topk + moe_permute",
              n_tokens, hidden, n_experts, top_k);
  FTK_REQUIRE(x && gate_w && logits && ids && weights, "moe_route: null pointer");
  FTK_REQUIRE(!do_sort || (counts && offsets && routes && pos), "moe_route: the sort needs its four outputs");
  FTK_REQUIRE(((uintptr_t)x | (uintptr_t)gate_w) % 16 == 0, "moe_route: x and the gate weight must be 16-byte aligned");
  const size_t smem = route_smem(n_tokens, n_experts, top_k);
  if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int blocks = (n_experts + kRouteExperts - 1) / kRouteExperts;
  note_variant(do_sort ? "routing: product, choice and sort in one launch" : "routing: product and choice in one launch");
  FTK_LAUNCH(moe_route_kernel, blocks, kRouteWarps * 32, smem, (cudaStream_t)stream, 
      x, gate_w, bias, n_tokens, hidden, n_experts, top_k, scoring, scale, logits, ids, weights, counts, offsets, routes, pos,
      do_sort);
  FTK_LAUNCH_CHECK("moe_route");
  return 0;
}
