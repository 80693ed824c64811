// Sampling from float32 logits, one thread block per row.
//
// temperature <= 0: argmax, lowest index on a tie (python/freetoken/engine/sample.py:78-79).
// Otherwise (sample.py:63-73, python/freetoken/kernel/triton/sampling.py:123-143,342-425,576-618):
// e_i = exp((logit_i - max) / T); top-k keeps e_i >= the k-th largest value; top-p then keeps
// e_i >= th for the largest th whose kept mass reaches top_p of the mass left by top-k; the drawn
// token is the first index whose running kept mass exceeds u times the kept mass.  The thresholds
// are found by bisection on the bit pattern of e (monotonic for positive floats), so no sort and no
// scratch memory are needed; every sum is a fixed-order block reduction.  The uniform number u
// comes from the host (a counter-based generator keyed by seed, request and step), so a draw does
// not depend on what else is in the batch.
#include "common.cuh"

namespace ftk {

constexpr int kSampleThreads = 1024;

struct RowView {
  const float* row;
  int vocab;
  float mx, inv_t;
  __device__ __forceinline__ float e(int i) const { return expf((row[i] - mx) * inv_t); }
};

// (count, mass) of entries with e >= th, over the block.
__device__ __forceinline__ void count_mass(const RowView& v, float th, float* red, float& count, float& mass) {
  float c = 0.f, m = 0.f;
  for (int i = threadIdx.x; i < v.vocab; i += blockDim.x) {
    const float x = v.e(i);
    if (x >= th) {
      c += 1.f;
      m += x;
    }
  }
  count = block_sum(c, red);
  mass = block_sum(m, red);
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const float* __restrict__ logits, int vocab,
                                                                const float* __restrict__ temperature,
                                                                const int32_t* __restrict__ top_k,
                                                                const float* __restrict__ top_p,
                                                                const float* __restrict__ u,
                                                                int32_t* __restrict__ out) {
  __shared__ float red[33];
  __shared__ float sval[kSampleThreads / 32];
  __shared__ int sidx[kSampleThreads / 32];
  __shared__ float chunk_prefix[kSampleThreads + 1];
  __shared__ int result;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // ---- max and argmax (lowest index wins)
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float x = row[i];
    if (x > best) {
      best = x;
      bi = i;
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
  if (lane == 0) {
    sval[warp] = best;
    sidx[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? sval[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (lane == 0) {
      sval[0] = best;
      sidx[0] = bi == 0x7fffffff ? 0 : bi;
    }
  }
  __syncthreads();
  const float t = temperature[r];
  if (t <= 0.f) {
    if (threadIdx.x == 0) out[r] = sidx[0];
    return;
  }
  RowView v{row, vocab, sval[0], 1.f / fmaxf(t, 1e-6f)};

  // ---- thresholds by bisection on the bit pattern of e in (0, 1]
  float th = 0.f;  // keep everything
  float count, mass;
  const int k = top_k[r];
  if (k > 0 && k < vocab) {
    uint32_t lo = 0u, hi = 0x3f800000u;  // count(e >= lo) >= k holds for lo = 0; e <= 1
    while (lo < hi) {
      const uint32_t mid = lo + (hi - lo + 1u) / 2u;
      count_mass(v, __uint_as_float(mid), red, count, mass);
      if (count >= (float)k) lo = mid; else hi = mid - 1u;
    }
    th = __uint_as_float(lo);
  }
  const float p = top_p[r];
  if (p < 1.f) {
    count_mass(v, th, red, count, mass);
    const float need = fmaxf(p, 1e-6f) * mass;
    uint32_t lo = __float_as_uint(th), hi = 0x3f800000u;
    while (lo < hi) {
      const uint32_t mid = lo + (hi - lo + 1u) / 2u;
      count_mass(v, __uint_as_float(mid), red, count, mass);
      if (mass >= need) lo = mid; else hi = mid - 1u;
    }
    th = __uint_as_float(lo);
  }

  // ---- inverse CDF in index order over the kept entries
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int i0 = min(vocab, (int)threadIdx.x * per), i1 = min(vocab, i0 + per);
  float cs = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float x = v.e(i);
    if (x >= th) cs += x;
  }
  chunk_prefix[threadIdx.x + 1] = cs;
  if (threadIdx.x == 0) {
    chunk_prefix[0] = 0.f;
    result = -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // sequential prefix over 1024 chunk sums: fixed order
    float run = 0.f;
    for (int i = 1; i <= (int)blockDim.x; ++i) {
      run += chunk_prefix[i];
      chunk_prefix[i] = run;
    }
  }
  __syncthreads();
  const float total = chunk_prefix[blockDim.x];
  const float target = u[r] * total;
  const float before = chunk_prefix[threadIdx.x], after = chunk_prefix[threadIdx.x + 1];
  if (before <= target && target < after) {
    float run = before;
    int last = -1, hit = -1;
    for (int i = i0; i < i1 && hit < 0; ++i) {
      const float x = v.e(i);
      if (x >= th) {
        run += x;
        last = i;
        if (run > target) hit = i;
      }
    }
    result = hit >= 0 ? hit : last;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = result >= 0 ? result : sidx[0];
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_sample(const float* logits, int n_rows, int vocab, const float* temperature, const int32_t* top_k,
                          const float* top_p, const float* u, int32_t* out, void* stream) {
  FTK_REQUIRE(n_rows >= 0 && vocab >= 1, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
  if (n_rows == 0) return 0;
  FTK_REQUIRE(logits && temperature && top_k && top_p && u && out, "sample: null pointer");
  sample_kernel<<<n_rows, kSampleThreads, 0, (cudaStream_t)stream>>>(logits, vocab, temperature, top_k, top_p, u, out);
  FTK_LAUNCH_CHECK("sample");
  return 0;
}
