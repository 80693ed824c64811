// Matrix products for steps of very few tokens: the weights are streamed once, by every SM at once.
//
// A decode step of one to four tokens multiplies each weight matrix by one to four vectors: the time is
// the time to read the weights, and a tensor-core tile (128 weight rows x 16 and more tokens) leaves most
// of its rows of accumulator idle while it pays its set-up per tile.  Here a warp owns a few weight rows,
// its lanes walk them in 16-byte pieces (8 bfloat16 weights) with many loads in flight, multiply with the
// activations (read from L2), and add up with shuffles at the end; sums are float32, in an order that
// depends on the sizes only.  Three forms:
//   small_linear      out[t, n] = x[t] . W[n]                      (qkv and output projections)
//   routed_gate_up    a[r, i]   = act(h[t(r)] . W1[e(r)][i], h[t(r)] . W1[e(r)][I + i])
//   routed_down       y[r, n]   = (a[r] . W2[e(r)][n]) * weight[r]
// The routed forms take the routes as the router wrote them (route r = t * top_k + j goes to expert
// ids[r]): no sort by expert, no gathered copy of the activations.  The reference has a kernel of this
// kind for its decode steps too (python/freetoken/kernel/triton/decode_moe.py:5-75); rounding points are
// those of the grouped kernels (gate and up rounded before the activation, the route weight on the
// float32 sum: python/freetoken/moe/fused_nvfp4.py:317-344, python/freetoken/kernel/triton/fused_moe.py:292-296).
#include "common.cuh"

namespace ftk {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kGemvMaxTokens = 4;
#ifndef FTK_GEMV_TURN
#define FTK_GEMV_TURN 4
#endif
constexpr int kGemvTurn = FTK_GEMV_TURN;  // 16-byte pieces per lane and row in flight
constexpr int kGemvTaskBytes = 24576;  // weights one warp streams, about

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = __uint_as_float(v.x << 16);
  f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16);
  f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16);
  f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16);
  f[7] = __uint_as_float(v.w & 0xffff0000u);
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {  // weights are read once: do not keep them in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float dot8(const float (&a)[8], const float (&b)[8], float acc) {
#pragma unroll
  for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
  return acc;
}

// A block's eight warps are laid out as KS slices of the row length times 8 / KS groups of R rows.  A warp
// multiplies its slice of its R rows with the same slice of the T activation rows (staged in shared memory
// once per block): it walks the slice in turns of U pieces per lane and row, R * U loads in flight per lane,
// the first turn's issued before the wait on the kernel before (weights never depend on it).  A warp's
// task is kept long (about 24 KB of weights): short tasks spend their time starting and ending.  The
// slices' partial sums meet in shared memory and are added in slice order.
template <int R, int U>
__device__ __forceinline__ void load_turn(const uint4* const (&wr)[R], int c0, int c_end, int lane, uint4 (&wv)[R][U]) {
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * 32 + lane;
      wv[r][u] = c < c_end ? ld_stream(wr[r] + c) : make_uint4(0, 0, 0, 0);
    }
}

template <int T, int R, int U>
__device__ __forceinline__ void stream_rows(const uint4* const (&wr)[R], const uint4* sx, int k8, int c_begin, int c_end,
                                            int lane, uint4 (&wv)[R][U], float (&acc)[R][T]) {
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
  for (int c0 = c_begin; c0 < c_end; c0 += 32 * U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * 32 + lane;
      if (c < c_end) {
        float wf[R][8];
#pragma unroll
        for (int r = 0; r < R; ++r) unpack8(wv[r][u], wf[r]);
#pragma unroll
        for (int t = 0; t < T; ++t) {
          float xf[8];
          unpack8(sx[t * k8 + c], xf);
#pragma unroll
          for (int r = 0; r < R; ++r) acc[r][t] = dot8(wf[r], xf, acc[r][t]);
        }
      }
    }
    // (refilling each slot as soon as it is read, instead of a turn at a time, measured slower: 33 against
    // 26.5 microseconds for the gate/up product of one token)
    if (c0 + 32 * U < c_end) load_turn<R, U>(wr, c0 + 32 * U, c_end, lane, wv);
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) acc[r][t] = warp_sum(acc[r][t]);
}

// Adds the slices' sums in slice order; afterwards the threads with `threadIdx.x < groups * R * T` hold, for
// (group, r, t) = (threadIdx.x / (R * T), threadIdx.x / T % R, threadIdx.x % T), the full sum.
template <int T, int R>
__device__ __forceinline__ float meet(float (&acc)[R][T], float* part, int ks, int n_ks, int rg, int lane) {
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) part[((rg * n_ks + ks) * R + r) * T + t] = acc[r][t];
  }
  __syncthreads();
  const int groups = kGemvWarps / n_ks;
  float v = 0.f;
  if (threadIdx.x < groups * R * T) {
    const int g = threadIdx.x / (R * T), rt = threadIdx.x % (R * T);
    for (int k = 0; k < n_ks; ++k) v += part[(g * n_ks + k) * R * T + rt];
  }
  return v;
}

// ---------------------------------------------------------------- out = x W^T
template <int T, int R>
__global__ void __launch_bounds__(kGemvThreads) small_linear_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    const __nv_bfloat16* __restrict__ w,
                                                                    __nv_bfloat16* __restrict__ out, int N, int K,
                                                                    int n_ks) {
  extern __shared__ uint4 sx[];  // [T][K / 8]
  __shared__ float part[kGemvWarps * R * T];
  constexpr int U = kGemvTurn;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k8 = K >> 3;
  const int ks = warp % n_ks, rg = warp / n_ks, groups = kGemvWarps / n_ks;
  const int row0 = (blockIdx.x * groups + rg) * R;
  const int c_begin = ks * (k8 / n_ks), c_end = ks == n_ks - 1 ? k8 : c_begin + k8 / n_ks;
  const uint4* wr[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wr[r] = reinterpret_cast<const uint4*>(w + (size_t)min(row0 + r, N - 1) * K);
  uint4 wv[R][U];
  load_turn<R, U>(wr, c_begin, c_end, lane, wv);
  pdl_wait();
  // the kernel after this one may bring its blocks onto the SMs as the last of these finish: it touches
  // nothing of this kernel's before its own wait, and has its first weights on their way by then
  pdl_trigger();
  const uint4* x4 = reinterpret_cast<const uint4*>(x);
  for (int i = threadIdx.x; i < T * k8; i += kGemvThreads) sx[i] = x4[i];
  __syncthreads();
  float acc[R][T];
  stream_rows<T, R, U>(wr, sx, k8, c_begin, c_end, lane, wv, acc);
  const float v = meet<T, R>(acc, part, ks, n_ks, rg, lane);
  if (threadIdx.x < groups * R * T) {
    const int g = threadIdx.x / (R * T), r = threadIdx.x / T % R, t = threadIdx.x % T;
    const int row = (blockIdx.x * groups + g) * R + r;
    if (row < N) out[(size_t)t * N + row] = __float2bfloat16_rn(v);
  }
}

// ---------------------------------------------------------------- a[r] = act(h[t] W1[e]^T)
// Block (x, route): a warp's rows are RA gate rows and the RA up rows of the same activation columns.
template <int RA>
__global__ void __launch_bounds__(kGemvThreads) routed_gate_up_kernel(
    const __nv_bfloat16* __restrict__ h, const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ w1,
    __nv_bfloat16* __restrict__ a, int H, int I, int top_k, int n_experts, int act, float alpha, float limit,
    int n_ks) {
  constexpr int R = 2 * RA, U = kGemvTurn;
  extern __shared__ uint4 sx[];  // [H / 8]
  __shared__ float part[kGemvWarps * R];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k8 = H >> 3;
  const int ks = warp % n_ks, rg = warp / n_ks, groups = kGemvWarps / n_ks;
  const int c_begin = ks * (k8 / n_ks), c_end = ks == n_ks - 1 ? k8 : c_begin + k8 / n_ks;
  const int route = blockIdx.y, t = route / top_k;
  const int i0 = (blockIdx.x * groups + rg) * RA;
  pdl_wait();
  pdl_trigger();
  const int e = ids[route];
  if (e < 0 || e >= n_experts) {  // a route to no expert contributes nothing
    for (int i = threadIdx.x; i < groups * RA; i += kGemvThreads) {
      const int col = blockIdx.x * groups * RA + i;
      if (col < I) a[(size_t)route * I + col] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const __nv_bfloat16* we = w1 + (size_t)e * 2 * I * H;
  const uint4* wr[R];
#pragma unroll
  for (int r = 0; r < RA; ++r) {
    const int i = min(i0 + r, I - 1);
    wr[r] = reinterpret_cast<const uint4*>(we + (size_t)i * H);
    wr[RA + r] = reinterpret_cast<const uint4*>(we + (size_t)(I + i) * H);
  }
  uint4 wv[R][U];
  load_turn<R, U>(wr, c_begin, c_end, lane, wv);
  const uint4* x4 = reinterpret_cast<const uint4*>(h + (size_t)t * H);
  for (int i = threadIdx.x; i < k8; i += kGemvThreads) sx[i] = x4[i];
  __syncthreads();
  float acc[R][1];
  stream_rows<1, R, U>(wr, sx, k8, c_begin, c_end, lane, wv, acc);
  const float v = meet<1, R>(acc, part, ks, n_ks, rg, lane);
  // thread (g, r): r < RA holds a gate sum, r >= RA the up sum of column r - RA: pair them up through shared memory
  __syncthreads();
  if (threadIdx.x < groups * R) part[threadIdx.x] = v;
  __syncthreads();
  if (threadIdx.x < groups * RA) {
    const int g = threadIdx.x / RA, r = threadIdx.x % RA;
    const int col = (blockIdx.x * groups + g) * RA + r;
    if (col < I) {
      const float gate = __bfloat162float(__float2bfloat16_rn(part[g * R + r]));
      const float up = __bfloat162float(__float2bfloat16_rn(part[g * R + RA + r]));
      a[(size_t)route * I + col] = __float2bfloat16_rn(gated_act(gate, up, act, alpha, limit));
    }
  }
}

// ---------------------------------------------------------------- y[r] = (a[r] W2[e]^T) * weight[r]
template <int R>
__global__ void __launch_bounds__(kGemvThreads) routed_down_kernel(
    const __nv_bfloat16* __restrict__ a, const int32_t* __restrict__ ids, const float* __restrict__ weights,
    const __nv_bfloat16* __restrict__ w2, __nv_bfloat16* __restrict__ y, int H, int I, int n_experts, int n_ks) {
  constexpr int U = kGemvTurn;
  extern __shared__ uint4 sx[];  // [I / 8]
  __shared__ float part[kGemvWarps * R];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k8 = I >> 3;
  const int ks = warp % n_ks, rg = warp / n_ks, groups = kGemvWarps / n_ks;
  const int c_begin = ks * (k8 / n_ks), c_end = ks == n_ks - 1 ? k8 : c_begin + k8 / n_ks;
  const int route = blockIdx.y;
  const int row0 = (blockIdx.x * groups + rg) * R;
  // The expert ids come from the routing kernel, at least two launches back, which has ended (every kernel
  // waits for the one before it before it lets the next one in, or ends): the id is read and the first
  // weights are on their way while the gate/up kernel before this one still runs.
  const int e = ids[route];
  const bool routed = e >= 0 && e < n_experts;
  const __nv_bfloat16* we = w2 + (size_t)(routed ? e : 0) * H * I;
  const uint4* wr[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wr[r] = reinterpret_cast<const uint4*>(we + (size_t)min(row0 + r, H - 1) * I);
  uint4 wv[R][U];
  if (routed) load_turn<R, U>(wr, c_begin, c_end, lane, wv);
  pdl_wait();
  pdl_trigger();
  if (!routed) {  // a route to no expert contributes nothing
    for (int i = threadIdx.x; i < groups * R; i += kGemvThreads) {
      const int n = blockIdx.x * groups * R + i;
      if (n < H) y[(size_t)route * H + n] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const uint4* x4 = reinterpret_cast<const uint4*>(a + (size_t)route * I);
  for (int i = threadIdx.x; i < k8; i += kGemvThreads) sx[i] = x4[i];
  __syncthreads();
  float acc[R][1];
  stream_rows<1, R, U>(wr, sx, k8, c_begin, c_end, lane, wv, acc);
  const float v = meet<1, R>(acc, part, ks, n_ks, rg, lane);
  if (threadIdx.x < groups * R) {
    const int row = blockIdx.x * groups * R + threadIdx.x;
    if (row < H) y[(size_t)route * H + row] = __float2bfloat16_rn(v * weights[route]);
  }
}

// How a block's eight warps share the work.  Rows per warp: 4 where there are that many; slices along the
// row (a power of two, at most 8): so that a warp streams about kGemvTaskBytes, but enough of them that the
// rows make at least one block per SM.
struct GemvShape {
  int r, n_ks, groups, blocks;
};
static int sm_count() {
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev] > 0 ? sms[dev] : 148;
}
static GemvShape gemv_shape(int n_rows, int k, int n_products, int max_r) {
  GemvShape g;
  g.r = n_rows >= 4 && max_r >= 4 ? 4 : (n_rows >= 2 && max_r >= 2 ? 2 : 1);
  const int k8 = k >> 3;
  g.n_ks = 1;
  while (g.n_ks < kGemvWarps && k8 % (2 * g.n_ks) == 0 && k8 / (2 * g.n_ks) >= 32 &&
         ((long long)g.r * k * 2 / g.n_ks > kGemvTaskBytes ||
          (long long)((n_rows + g.r - 1) / g.r) * g.n_ks * n_products < (long long)kGemvWarps * sm_count()))
    g.n_ks <<= 1;
  g.groups = kGemvWarps / g.n_ks;
  g.blocks = (n_rows + g.groups * g.r - 1) / (g.groups * g.r);
  return g;
}

// (Dynamic plus the kernels' own static shared memory must stay under the default 48 KB, else the larger
// size has to be asked for: hence the 40 KB mark below.)
template <int T>
static void launch_small_linear(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* out, int N, int K,
                                cudaStream_t s) {
  const GemvShape g = gemv_shape(N, K, 1, T <= 2 ? 4 : 2);
  const size_t smem = (size_t)T * K * 2;
#define FTK_SL(RR)                                                                                           \
  do {                                                                                                       \
    auto kern = small_linear_kernel<T, RR>;                                                                  \
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    FTK_LAUNCH(kern, g.blocks, kGemvThreads, smem, s, x, w, out, N, K, g.n_ks);                              \
  } while (0)
  if (g.r == 4) FTK_SL(4); else if (g.r == 2) FTK_SL(2); else FTK_SL(1);
#undef FTK_SL
}

static void launch_gate_up(const __nv_bfloat16* h, const int32_t* ids, const __nv_bfloat16* w1, __nv_bfloat16* a,
                           int n_routes, int top_k, int n_experts, int H, int I, int act, float alpha, float limit,
                           cudaStream_t s) {
  const GemvShape g = gemv_shape(I, H, n_routes, 2);  // r activation columns = 2 r weight rows a warp
  const size_t smem = (size_t)H * 2;
  dim3 grid(g.blocks, n_routes);
#define FTK_GU(RA)                                                                                           \
  do {                                                                                                       \
    auto kern = routed_gate_up_kernel<RA>;                                                                   \
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    FTK_LAUNCH(kern, grid, kGemvThreads, smem, s, h, ids, w1, a, H, I, top_k, n_experts, act, alpha, limit, g.n_ks); \
  } while (0)
  if (g.r == 2) FTK_GU(2); else FTK_GU(1);
#undef FTK_GU
}

static void launch_down(const __nv_bfloat16* a, const int32_t* ids, const float* weights, const __nv_bfloat16* w2,
                        __nv_bfloat16* y, int n_routes, int n_experts, int H, int I, cudaStream_t s) {
  const GemvShape g = gemv_shape(H, I, n_routes, 4);
  const size_t smem = (size_t)I * 2;
  dim3 grid(g.blocks, n_routes);
#define FTK_DN(RR)                                                                                           \
  do {                                                                                                       \
    auto kern = routed_down_kernel<RR>;                                                                      \
    if (smem > 40 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    FTK_LAUNCH(kern, grid, kGemvThreads, smem, s, a, ids, weights, w2, y, H, I, n_experts, g.n_ks);          \
  } while (0)
  if (g.r == 4) FTK_DN(4); else if (g.r == 2) FTK_DN(2); else FTK_DN(1);
#undef FTK_DN
}

}  // namespace ftk

using namespace ftk;

// Whether the kernels of this file take a product of `n_tokens` rows with a [n_out, k] bfloat16 matrix.
extern "C" int ftk_small_linear_fits(int n_tokens, int n_out, int k) {
  return n_tokens >= 1 && n_tokens <= kGemvMaxTokens && n_out >= 1 && k >= 8 && k % 8 == 0 &&
         (size_t)n_tokens * k * 2 <= 96 * 1024;
}

extern "C" int ftk_small_linear(const void* x, const void* w, void* out, int n_tokens, int n_out, int k, void* stream) {
  FTK_REQUIRE(ftk_small_linear_fits(n_tokens, n_out, k),
              "small_linear: %d tokens, %d x %d weights: takes 1 to %d tokens and rows of a multiple of 8 elements",
              n_tokens, n_out, k, kGemvMaxTokens);
  FTK_REQUIRE(x && w && out, "small_linear: null pointer");
  FTK_REQUIRE((((uintptr_t)x | (uintptr_t)w) & 15) == 0, "small_linear: x and w must be 16-byte aligned");
  const auto* xb = (const __nv_bfloat16*)x;
  const auto* wb = (const __nv_bfloat16*)w;
  auto* ob = (__nv_bfloat16*)out;
  cudaStream_t s = (cudaStream_t)stream;
  note_variant("few-token product: weights streamed by warps");
  switch (n_tokens) {
    case 1: launch_small_linear<1>(xb, wb, ob, n_out, k, s); break;
    case 2: launch_small_linear<2>(xb, wb, ob, n_out, k, s); break;
    case 3: launch_small_linear<3>(xb, wb, ob, n_out, k, s); break;
    default: launch_small_linear<4>(xb, wb, ob, n_out, k, s); break;
  }
  FTK_LAUNCH_CHECK("small_linear");
  return 0;
}

// Whether the routed kernels take a step of `n_tokens` tokens (bfloat16 only).
extern "C" int ftk_moe_small_fits(int n_tokens, int hidden, int inter, int top_k) {
  return n_tokens >= 1 && n_tokens <= kGemvMaxTokens && top_k >= 1 && (long long)n_tokens * top_k <= 65535 &&
         hidden >= 8 && hidden % 8 == 0 && inter >= 8 && inter % 8 == 0 && hidden * 2 <= 96 * 1024 && inter * 2 <= 96 * 1024;
}

extern "C" int ftk_moe_small_gate_up(const void* h, const int32_t* ids, const void* w1, void* a, int n_tokens, int top_k,
                                     int n_experts, int hidden, int inter, int act, float alpha, float limit,
                                     void* stream) {
  FTK_REQUIRE(ftk_moe_small_fits(n_tokens, hidden, inter, top_k), "moe_small_gate_up: %d tokens, width %d, expert width %d "
              "do not fit the few-token kernels", n_tokens, hidden, inter);
  FTK_REQUIRE(act == FTK_ACT_SILU || act == FTK_ACT_SWIGLUOAI, "moe_small_gate_up: unknown activation %d", act);
  FTK_REQUIRE(h && ids && w1 && a && n_experts >= 1, "moe_small_gate_up: null pointer");
  FTK_REQUIRE((((uintptr_t)h | (uintptr_t)w1) & 15) == 0, "moe_small_gate_up: h and w1 must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  note_variant("expert gate/up product: few tokens, weights streamed by warps");
  launch_gate_up((const __nv_bfloat16*)h, ids, (const __nv_bfloat16*)w1, (__nv_bfloat16*)a, n_tokens * top_k, top_k,
                 n_experts, hidden, inter, act, alpha, limit, s);
  FTK_LAUNCH_CHECK("moe_small_gate_up");
  return 0;
}

extern "C" int ftk_moe_small_down(const void* a, const int32_t* ids, const float* weights, const void* w2, void* y,
                                  int n_tokens, int top_k, int n_experts, int hidden, int inter, void* stream) {
  FTK_REQUIRE(ftk_moe_small_fits(n_tokens, hidden, inter, top_k), "moe_small_down: %d tokens, width %d, expert width %d do "
              "not fit the few-token kernels", n_tokens, hidden, inter);
  FTK_REQUIRE(a && ids && weights && w2 && y && n_experts >= 1, "moe_small_down: null pointer");
  FTK_REQUIRE((((uintptr_t)a | (uintptr_t)w2) & 15) == 0, "moe_small_down: a and w2 must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  note_variant("expert down product: few tokens, weights streamed by warps");
  launch_down((const __nv_bfloat16*)a, ids, weights, (const __nv_bfloat16*)w2, (__nv_bfloat16*)y, n_tokens * top_k,
              n_experts, hidden, inter, s);
  FTK_LAUNCH_CHECK("moe_small_down");
  return 0;
}
