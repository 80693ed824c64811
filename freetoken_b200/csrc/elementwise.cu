// Row-wise kernels: embedding gather, RMSNorm with fused residual sum, gated activation, casts,
// block-table updates, expert-row gather and the sum over a token's routes.
//
// All of them are memory-bound; each row is read once, in 8- or 16-byte pieces where the row
// length allows it (a scalar path takes every other length), and all arithmetic is float32.
#include "common.cuh"

namespace ftk {

// ---------------------------------------------------------------- 4-element access helpers
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&t.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------- embedding gather
// out[t, :] = float(table[ids[t], :])   (python/freetoken/kernel/csrc/jit/index.cu:31-59)
template <typename T, bool VEC>
__global__ void embedding_gather_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                                        int hidden, int vocab, float* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * hidden;
  const bool ok = id >= 0 && id < vocab;  // an id outside the table gives a zero row, never a fault
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (ok) Vec4<T>::load(src + i, v);
      Vec4<float>::store(o + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = ok ? to_float(src[i]) : 0.f;
  }
}

// ---------------------------------------------------------------- RMSNorm (+ residual sum)
// z = x + residual (32-bit); residual <- z; out = z * rsqrt(mean(z^2) + eps) * (1 + w)
// (python/freetoken/kernel/triton/norm.py:65-75,101-112).  One block per row; the row's z is
// kept in shared memory between the two passes.
// With `route_pos`, x holds the rows of the routed experts' outputs and the row that is added is
// sum_j x[route_pos[row * top_k + j]] (+ shared[row]), a 32-bit sum in route order rounded to XT: the
// sum over routes (moe_combine_kernel) without its trip through memory.
template <typename XT, typename OT, bool VEC>
__global__ void add_rmsnorm_kernel(const XT* __restrict__ x, float* __restrict__ residual,
                                   const float* __restrict__ weight, OT* __restrict__ out,
                                   float* __restrict__ out_f32, const int32_t* __restrict__ rows,
                                   int hidden, float eps, int gemma, const int32_t* __restrict__ route_pos,
                                   int top_k, int n_routes, const XT* __restrict__ shared) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float zrow[];
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int src_row = rows ? rows[r] : r;
  const size_t src = (size_t)src_row * hidden;
  const size_t dst = (size_t)r * hidden;
  const bool update = residual != nullptr && x != nullptr && rows == nullptr;
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float z[4] = {0.f, 0.f, 0.f, 0.f};
      if (residual) Vec4<float>::load(residual + src + i, z);
      if (x && route_pos) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j0 = 0; j0 < top_k; j0 += 8) {  // eight rows' loads in flight before the first is added
          int ps[8];
          float xv[8][4];
#pragma unroll
          for (int u = 0; u < 8; ++u) ps[u] = j0 + u < top_k ? __ldg(route_pos + (size_t)src_row * top_k + j0 + u) : -1;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (ps[u] >= 0 && ps[u] < n_routes) {
              Vec4<XT>::load(x + (size_t)ps[u] * hidden + i, xv[u]);
            } else {
              xv[u][0] = xv[u][1] = xv[u][2] = xv[u][3] = 0.f;
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u)  // route order
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[q] += xv[u][q];
        }
        if (shared) {
          float xv[4];
          Vec4<XT>::load(shared + src + i, xv);
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[q] += xv[q];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) z[q] += to_float(from_float<XT>(acc[q]));
      } else if (x) {
        float xv[4];
        Vec4<XT>::load(x + src + i, xv);
#pragma unroll
        for (int j = 0; j < 4; ++j) z[j] += xv[j];
      }
      if (update) Vec4<float>::store(residual + src + i, z);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        zrow[i + j] = z[j];
        ss += z[j] * z[j];
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float z = residual ? residual[src + i] : 0.f;
      if (x && route_pos) {
        float acc = 0.f;
        for (int j = 0; j < top_k; ++j) {
          const int p = route_pos[(size_t)src_row * top_k + j];
          if (p >= 0 && p < n_routes) acc += to_float(x[(size_t)p * hidden + i]);
        }
        if (shared) acc += to_float(shared[src + i]);
        z += to_float(from_float<XT>(acc));
      } else if (x) {
        z += to_float(x[src + i]);
      }
      if (update) residual[src + i] = z;
      zrow[i] = z;
      ss += z * z;
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  const float one = gemma ? 1.f : 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float w[4], y[4];
      Vec4<float>::load(weight + i, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = zrow[i + j] * inv * (w[j] + one);
      Vec4<OT>::store(out + dst + i, y);
      if (out_f32) {
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] = to_float(from_float<OT>(y[j]));
        Vec4<float>::store(out_f32 + dst + i, y);
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const OT y = from_float<OT>(zrow[i] * inv * (weight[i] + one));
      out[dst + i] = y;
      if (out_f32) out_f32[dst + i] = to_float(y);
    }
  }
}

// ---------------------------------------------------------------- gated activation
template <typename T>
__global__ void act_and_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int act,
                                   float alpha, float limit) {
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const T* g = gate_up + row * 2 * (size_t)inter;
  out[row * inter + i] = from_float<T>(gated_act(to_float(g[i]), to_float(g[inter + i]), act, alpha, limit));
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ src, D* __restrict__ dst, long long n) {
  pdl_wait();
  pdl_trigger();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = from_float<D>(to_float(src[i]));
}

__global__ void table_update_kernel(int32_t* table, long long table_len, const int32_t* updates, int n) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long idx = updates[2 * i];
  if (idx >= 0 && idx < table_len) table[idx] = updates[2 * i + 1];
}

// dst[pairs[i][0]] = src[pairs[i][1]]: tokens sampled by the previous step become inputs of this one
// without a round trip through the host.  Values outside [0, vocab) become 0.
__global__ void copy_tokens_kernel(int32_t* dst, int dst_len, const int32_t* pairs, const int32_t* src, int src_len,
                                   int n, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = pairs[2 * i], s = pairs[2 * i + 1];
  if (d < 0 || d >= dst_len || s < 0 || s >= src_len) return;
  const int v = src[s];
  dst[d] = (v >= 0 && v < vocab) ? v : 0;
}

// out[r, :] = h[sorted_routes[r] / top_k, :]
template <typename T, bool VEC>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int32_t* __restrict__ sorted_routes,
                                  int top_k, int hidden, int n_tokens, T* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int route = sorted_routes[r];
  const int t = route / top_k;
  if (route < 0 || t >= n_tokens) return;
  const T* src = h + (size_t)t * hidden;
  T* dst = out + (size_t)r * hidden;
  if (VEC) {
    const int per = 16 / (int)sizeof(T);
    for (int i = threadIdx.x * per; i < hidden; i += blockDim.x * per)
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

// out[t] = sum_j y[route_pos[t*k + j]] (+ shared[t]), 32-bit sum in route order
// (python/freetoken/kernel/triton/fused_moe.py:111-153).
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int32_t* __restrict__ route_pos, int top_k,
                                   int hidden, int n_routes, const T* __restrict__ shared, T* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= hidden) return;
  float acc = 0.f;
  for (int j = 0; j < top_k; ++j) {
    const int p = route_pos[t * top_k + j];
    if (p >= 0 && p < n_routes) acc += to_float(y[(size_t)p * hidden + i]);
  }
  if (shared) acc += to_float(shared[(size_t)t * hidden + i]);
  out[(size_t)t * hidden + i] = from_float<T>(acc);
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_embedding_gather(const void* table, int dtype, const int32_t* ids, int n_tokens, int hidden,
                                    int vocab, float* out, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "embedding_gather: bad dtype %d", dtype);
  FTK_REQUIRE(table && ids && out, "embedding_gather: null pointer");
  FTK_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embedding_gather: bad sizes T=%d H=%d V=%d", n_tokens,
              hidden, vocab);
  if (n_tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = hidden % 4 == 0 && aligned16(table) && aligned16(out) && (dtype == FTK_F32 || hidden % 8 == 0);
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == FTK_F32) {
    if (vec) FTK_LAUNCH((embedding_gather_kernel<float, true>), n_tokens, threads, 0, s, (const float*)table, ids, hidden, vocab, out);
    else FTK_LAUNCH((embedding_gather_kernel<float, false>), n_tokens, threads, 0, s, (const float*)table, ids, hidden, vocab, out);
  } else {
    if (vec) FTK_LAUNCH((embedding_gather_kernel<__nv_bfloat16, true>), n_tokens, threads, 0, s, (const __nv_bfloat16*)table, ids, hidden, vocab, out);
    else FTK_LAUNCH((embedding_gather_kernel<__nv_bfloat16, false>), n_tokens, threads, 0, s, (const __nv_bfloat16*)table, ids, hidden, vocab, out);
  }
  FTK_LAUNCH_CHECK("embedding_gather");
  return 0;
}

template <typename XT, typename OT>
static int launch_norm(const void* x, float* residual, const float* weight, void* out, float* out_f32,
                       const int32_t* rows, int n_rows, int hidden, float eps, int gemma, cudaStream_t s,
                       const int32_t* route_pos = nullptr, int top_k = 0, int n_routes = 0, const void* shared = nullptr) {
  const bool vec = hidden % 4 == 0 && aligned16(x) && aligned16(residual) && aligned16(weight) &&
                   aligned16(out) && aligned16(out_f32) && (hidden % 8 == 0) && aligned16(shared);
  int threads = hidden >= 2048 ? 256 : 128;
  // few rows: a thread per four elements, so that every load of a row is in flight at once
  if (n_rows <= 64 && vec) threads = hidden / 4 >= 1024 ? 1024 : (hidden / 4 + 31) / 32 * 32 > threads ? (hidden / 4 + 31) / 32 * 32 : threads;
  const size_t smem = (size_t)hidden * sizeof(float);
  auto kv = add_rmsnorm_kernel<XT, OT, true>;
  auto ks = add_rmsnorm_kernel<XT, OT, false>;
  if (smem > 48 * 1024) {
    FTK_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: hidden=%d is too wide for one block (max 51200)", hidden);
    cudaFuncSetAttribute(kv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(ks, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  if (vec) FTK_LAUNCH(kv, n_rows, threads, smem, s, (const XT*)x, residual, weight, (OT*)out, out_f32, rows, hidden, eps, gemma,
                      route_pos, top_k, n_routes, (const XT*)shared);
  else FTK_LAUNCH(ks, n_rows, threads, smem, s, (const XT*)x, residual, weight, (OT*)out, out_f32, rows, hidden, eps, gemma,
                  route_pos, top_k, n_routes, (const XT*)shared);
  FTK_LAUNCH_CHECK("add_rmsnorm");
  return 0;
}

extern "C" int ftk_add_rmsnorm(const void* x, int x_dtype, float* residual, const float* weight, void* out,
                               int out_dtype, float* out_f32, const int32_t* rows, int n_rows, int hidden,
                               float eps, int gemma, void* stream) {
  FTK_REQUIRE(dtype_ok(x_dtype) && dtype_ok(out_dtype), "add_rmsnorm: bad dtype");
  FTK_REQUIRE(weight && out && (x || residual), "add_rmsnorm: null pointer");
  FTK_REQUIRE(n_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d H=%d", n_rows, hidden);
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (x_dtype == FTK_F32 && out_dtype == FTK_F32)
    return launch_norm<float, float>(x, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma, s);
  if (x_dtype == FTK_BF16 && out_dtype == FTK_BF16)
    return launch_norm<__nv_bfloat16, __nv_bfloat16>(x, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma, s);
  if (x_dtype == FTK_F32 && out_dtype == FTK_BF16)
    return launch_norm<float, __nv_bfloat16>(x, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma, s);
  return launch_norm<__nv_bfloat16, float>(x, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma, s);
}

// The sum over a token's routes (rows of y), the residual sum and the norm in one pass.
extern "C" int ftk_add_rmsnorm_routes(const void* y, int y_dtype, const int32_t* route_pos, int top_k, int n_routes,
                                      const void* shared, float* residual, const float* weight, void* out,
                                      int out_dtype, float* out_f32, const int32_t* rows, int n_rows, int hidden,
                                      float eps, int gemma, void* stream) {
  FTK_REQUIRE(dtype_ok(y_dtype) && dtype_ok(out_dtype), "add_rmsnorm_routes: bad dtype");
  FTK_REQUIRE(y && route_pos && residual && weight && out, "add_rmsnorm_routes: null pointer");
  FTK_REQUIRE(n_rows >= 0 && hidden > 0 && top_k >= 1 && n_routes >= 0, "add_rmsnorm_routes: bad sizes");
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (y_dtype == FTK_F32 && out_dtype == FTK_F32)
    return launch_norm<float, float>(y, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma, s, route_pos,
                                     top_k, n_routes, shared);
  if (y_dtype == FTK_BF16 && out_dtype == FTK_BF16)
    return launch_norm<__nv_bfloat16, __nv_bfloat16>(y, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma,
                                                     s, route_pos, top_k, n_routes, shared);
  if (y_dtype == FTK_F32 && out_dtype == FTK_BF16)
    return launch_norm<float, __nv_bfloat16>(y, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma, s,
                                             route_pos, top_k, n_routes, shared);
  return launch_norm<__nv_bfloat16, float>(y, residual, weight, out, out_f32, rows, n_rows, hidden, eps, gemma, s,
                                           route_pos, top_k, n_routes, shared);
}

extern "C" int ftk_act_and_mul(const void* gate_up, int dtype, int n_rows, int inter, int act, float alpha,
                               float limit, void* out, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "act_and_mul: bad dtype %d", dtype);
  FTK_REQUIRE(gate_up && out, "act_and_mul: null pointer");
  FTK_REQUIRE(act == FTK_ACT_SILU || act == FTK_ACT_SWIGLUOAI, "act_and_mul: unknown activation %d", act);
  FTK_REQUIRE(n_rows >= 0 && inter > 0 && n_rows <= 65535 * 1024, "act_and_mul: bad sizes");
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  for (int r0 = 0; r0 < n_rows; r0 += 65535) {  // grid.y limit
    const int nr = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
    dim3 grid((inter + 255) / 256, nr);
    if (dtype == FTK_F32)
      FTK_LAUNCH(act_and_mul_kernel<float>, grid, 256, 0, s, (const float*)gate_up + (size_t)r0 * 2 * inter,
                                                     (float*)out + (size_t)r0 * inter, inter, act, alpha, limit);
    else
      FTK_LAUNCH(act_and_mul_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)gate_up + (size_t)r0 * 2 * inter,
                                                             (__nv_bfloat16*)out + (size_t)r0 * inter, inter, act, alpha, limit);
  }
  FTK_LAUNCH_CHECK("act_and_mul");
  return 0;
}

extern "C" int ftk_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, void* stream) {
  FTK_REQUIRE(dtype_ok(src_dtype) && dtype_ok(dst_dtype), "cast: bad dtype");
  FTK_REQUIRE(n >= 0 && (n == 0 || (src && dst)), "cast: bad arguments");
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (src_dtype == FTK_F32 && dst_dtype == FTK_BF16)
    FTK_LAUNCH((cast_kernel<float, __nv_bfloat16>), (int)blocks, 256, 0, s, (const float*)src, (__nv_bfloat16*)dst, n);
  else if (src_dtype == FTK_BF16 && dst_dtype == FTK_F32)
    FTK_LAUNCH((cast_kernel<__nv_bfloat16, float>), (int)blocks, 256, 0, s, (const __nv_bfloat16*)src, (float*)dst, n);
  else if (src_dtype == FTK_F32)
    FTK_LAUNCH((cast_kernel<float, float>), (int)blocks, 256, 0, s, (const float*)src, (float*)dst, n);
  else
    FTK_LAUNCH((cast_kernel<__nv_bfloat16, __nv_bfloat16>), (int)blocks, 256, 0, s, (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, n);
  FTK_LAUNCH_CHECK("cast");
  return 0;
}

extern "C" int ftk_table_update(int32_t* table, long long table_len, const int32_t* updates, int n_updates,
                                void* stream) {
  FTK_REQUIRE(n_updates >= 0 && table_len >= 0, "table_update: bad sizes");
  if (n_updates == 0) return 0;
  FTK_REQUIRE(table && updates, "table_update: null pointer");
  FTK_LAUNCH(table_update_kernel, (n_updates + 127) / 128, 128, 0, (cudaStream_t)stream, table, table_len, updates, n_updates);
  FTK_LAUNCH_CHECK("table_update");
  return 0;
}

extern "C" int ftk_copy_tokens(int32_t* dst, int dst_len, const int32_t* pairs, const int32_t* src, int src_len, int n,
                               int vocab, void* stream) {
  FTK_REQUIRE(n >= 0 && dst_len >= 0 && src_len >= 0 && vocab >= 1, "copy_tokens: bad sizes");
  if (n == 0) return 0;
  FTK_REQUIRE(dst && pairs && src, "copy_tokens: null pointer");
  FTK_LAUNCH(copy_tokens_kernel, (n + 127) / 128, 128, 0, (cudaStream_t)stream, dst, dst_len, pairs, src, src_len, n, vocab);
  FTK_LAUNCH_CHECK("copy_tokens");
  return 0;
}

extern "C" int ftk_moe_gather(const void* h, int dtype, const int32_t* sorted_routes, int n_routes, int top_k,
                              int hidden, void* out, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "moe_gather: bad dtype %d", dtype);
  FTK_REQUIRE(n_routes >= 0 && top_k > 0 && hidden > 0 && n_routes % top_k == 0, "moe_gather: bad sizes");
  if (n_routes == 0) return 0;
  FTK_REQUIRE(h && sorted_routes && out, "moe_gather: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int n_tokens = n_routes / top_k;
  const bool vec = aligned16(h) && aligned16(out) && (hidden * dtype_size(dtype)) % 16 == 0;
  const int threads = hidden >= 2048 ? 256 : 128;
  if (dtype == FTK_F32) {
    if (vec) FTK_LAUNCH((moe_gather_kernel<float, true>), n_routes, threads, 0, s, (const float*)h, sorted_routes, top_k, hidden, n_tokens, (float*)out);
    else FTK_LAUNCH((moe_gather_kernel<float, false>), n_routes, threads, 0, s, (const float*)h, sorted_routes, top_k, hidden, n_tokens, (float*)out);
  } else {
    if (vec) FTK_LAUNCH((moe_gather_kernel<__nv_bfloat16, true>), n_routes, threads, 0, s, (const __nv_bfloat16*)h, sorted_routes, top_k, hidden, n_tokens, (__nv_bfloat16*)out);
    else FTK_LAUNCH((moe_gather_kernel<__nv_bfloat16, false>), n_routes, threads, 0, s, (const __nv_bfloat16*)h, sorted_routes, top_k, hidden, n_tokens, (__nv_bfloat16*)out);
  }
  FTK_LAUNCH_CHECK("moe_gather");
  return 0;
}

extern "C" int ftk_moe_combine(const void* y, int dtype, const int32_t* route_pos, int n_tokens, int top_k,
                               int hidden, const void* shared, void* out, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "moe_combine: bad dtype %d", dtype);
  FTK_REQUIRE(n_tokens >= 0 && top_k > 0 && hidden > 0, "moe_combine: bad sizes");
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(y && route_pos && out, "moe_combine: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
    const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
    dim3 grid((hidden + 255) / 256, nt);
    if (dtype == FTK_F32)
      FTK_LAUNCH(moe_combine_kernel<float>, grid, 256, 0, s, (const float*)y, route_pos + (size_t)t0 * top_k, top_k, hidden,
                                                     n_tokens * top_k, shared ? (const float*)shared + (size_t)t0 * hidden : nullptr,
                                                     (float*)out + (size_t)t0 * hidden);
    else
      FTK_LAUNCH(moe_combine_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)y, route_pos + (size_t)t0 * top_k, top_k, hidden,
                                                             n_tokens * top_k, shared ? (const __nv_bfloat16*)shared + (size_t)t0 * hidden : nullptr,
                                                             (__nv_bfloat16*)out + (size_t)t0 * hidden);
  }
  FTK_LAUNCH_CHECK("moe_combine");
  return 0;
}
