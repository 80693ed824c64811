// Sampling from float32 logits.  A row is cut into chunks, one thread block each; the block that
// finishes a row last puts the chunks together and draws.
//
// temperature <= 0: argmax, lowest index on a tie (python/freetoken/engine/sample.py:78-79).
// Otherwise (sample.py:63-73, python/freetoken/kernel/triton/sampling.py:123-143,342-425,576-618):
// e_i = exp((logit_i - max) / T); top-k keeps e_i >= the k-th largest value; top-p then keeps
// e_i >= th for the largest th whose kept mass reaches top_p of the mass left by top-k; the drawn
// token is the first index whose running kept mass exceeds u times the kept mass.  The thresholds
// are found by bisection on the bit pattern of e (monotonic for positive floats), so no sort is
// needed; every sum is taken in a fixed order.  The uniform number u comes from the host (a
// counter-based generator keyed by seed, request and step), so a draw does not depend on what else
// is in the batch.
//
// Phase 1 (every block): the chunk's maximum, its lowest index, and, for a row that samples, the
// chunk's mass relative to its own maximum.  Phase 2 (the row's last block): the row's maximum from
// the chunk maxima; greedy rows are done.  Without top-k / top-p the chunk masses, brought to the
// row's maximum, say which chunk holds the drawn token, and only that chunk is walked.  With top-k
// or top-p the block bisects over the whole row.
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

constexpr int kSampleMaxChunks = 32;
constexpr int kSampleMaxRows = 2048;  // rows per launch (the host loops beyond)
__device__ float4 g_sample_part[kSampleMaxRows * kSampleMaxChunks];  // (max, index bits, mass, -)
__device__ unsigned int g_sample_arrivals[kSampleMaxRows];

// (max, lowest index of it) over the block; the result is in sval[0] / sidx[0] after the call.
__device__ __forceinline__ void block_argmax(float best, int bi, float* sval, int* sidx) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) {
      best = ob;
      bi = oi;
    }
  }
  __syncthreads();
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
      sidx[0] = bi;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const float* __restrict__ logits, int vocab,
                                                                const float* __restrict__ temperature,
                                                                const int32_t* __restrict__ top_k,
                                                                const float* __restrict__ top_p,
                                                                const float* __restrict__ u,
                                                                int32_t* __restrict__ out, int chunk) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[33];
  __shared__ float sval[kSampleThreads / 32];
  __shared__ int sidx[kSampleThreads / 32];
  __shared__ float chunk_prefix[kSampleThreads + 1];
  __shared__ int result;
  __shared__ bool last;
  const int r = blockIdx.y, c = blockIdx.x, n_chunks = gridDim.x;
  const float* row = logits + (size_t)r * vocab;
  const float t = temperature[r];
  const float inv_t = 1.f / fmaxf(t, 1e-6f);

  // ---- phase 1: this chunk's max, argmax (lowest index wins) and mass
  const int c0 = c * chunk, c1 = min(vocab, c0 + chunk);  // chunk is a multiple of 4
  float best = -INFINITY;
  int bi = 0x7fffffff;
  const bool vec = (vocab & 3) == 0;
  if (vec) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i = (c0 >> 2) + threadIdx.x; i < (c1 >> 2); i += blockDim.x) {
      const float4 x = __ldg(row4 + i);
      if (x.x > best) { best = x.x; bi = 4 * i; }
      if (x.y > best) { best = x.y; bi = 4 * i + 1; }
      if (x.z > best) { best = x.z; bi = 4 * i + 2; }
      if (x.w > best) { best = x.w; bi = 4 * i + 3; }
    }
  } else {
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
      const float x = row[i];
      if (x > best) { best = x; bi = i; }
    }
  }
  block_argmax(best, bi, sval, sidx);
  const float lmax = sval[0];
  const int lidx = sidx[0];
  float lsum = 0.f;
  if (t > 0.f) {  // the chunk was just read: this pass hits the cache
    float m = 0.f;
    if (lmax > -INFINITY)
      for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) m += expf((row[i] - lmax) * inv_t);
    lsum = block_sum(m, red);
  }
  if (threadIdx.x == 0) {
    g_sample_part[r * kSampleMaxChunks + c] = make_float4(lmax, __int_as_float(lidx), lsum, 0.f);
    __threadfence();
    last = atomicAdd(&g_sample_arrivals[r], 1u) == (unsigned)n_chunks - 1u;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();

  // ---- phase 2: the row, by its last block
  if (threadIdx.x == 0) {
    g_sample_arrivals[r] = 0;  // ready for the next launch
    float gb = -INFINITY;
    int gi = 0x7fffffff;
    for (int j = 0; j < n_chunks; ++j) {  // ascending chunks: the first of equal maxima stays
      const float4 pj = __ldcg(&g_sample_part[r * kSampleMaxChunks + j]);
      if (pj.x > gb) {
        gb = pj.x;
        gi = __float_as_int(pj.y);
      }
    }
    sval[0] = gb;
    sidx[0] = gi == 0x7fffffff ? 0 : gi;
  }
  __syncthreads();
  if (t <= 0.f) {
    if (threadIdx.x == 0) out[r] = sidx[0];
    return;
  }
  RowView v{row, vocab, sval[0], inv_t};
  const int k = top_k[r];
  const float p = top_p[r];
  int w0 = 0, w1 = vocab;      // the index range that is walked for the draw
  float mass_before = 0.f;     // kept mass in front of it
  float total_known = -1.f;    // kept mass of the whole row, where phase 1 gave it
  if (!(k > 0 && k < vocab) && !(p < 1.f)) {
    // everything is kept: the chunk masses say where the drawn token lies
    if (threadIdx.x == 0) {
      float run = 0.f;
      for (int j = 0; j < n_chunks; ++j) {
        const float4 pj = __ldcg(&g_sample_part[r * kSampleMaxChunks + j]);
        const float mj = pj.x > -INFINITY ? pj.z * expf((pj.x - v.mx) * inv_t) : 0.f;
        chunk_prefix[j] = run;
        run += mj;
      }
      chunk_prefix[n_chunks] = run;
      const float target = u[r] * run;
      int pick = n_chunks - 1;
      for (int j = 0; j < n_chunks; ++j)
        if (target < chunk_prefix[j + 1]) {
          pick = j;
          break;
        }
      sidx[1] = pick;
      sval[1] = chunk_prefix[pick];
      sval[2] = run;
    }
    __syncthreads();
    w0 = sidx[1] * chunk;
    w1 = min(vocab, w0 + chunk);
    mass_before = sval[1];
    total_known = sval[2];
    __syncthreads();
  }

  // ---- thresholds by bisection on the bit pattern of e in (0, 1]
  float th = 0.f;  // keep everything
  float count, mass;
  if (k > 0 && k < vocab) {
    uint32_t lo = 0u, hi = 0x3f800000u;  // count(e >= lo) >= k holds for lo = 0; e <= 1
    while (lo < hi) {
      const uint32_t mid = lo + (hi - lo + 1u) / 2u;
      count_mass(v, __uint_as_float(mid), red, count, mass);
      if (count >= (float)k) lo = mid; else hi = mid - 1u;
    }
    th = __uint_as_float(lo);
  }
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

  // ---- inverse CDF in index order over the kept entries of [w0, w1)
  const int per = (w1 - w0 + blockDim.x - 1) / blockDim.x;
  const int i0 = min(w1, w0 + (int)threadIdx.x * per), i1 = min(w1, i0 + per);
  float cs = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float x = v.e(i);
    if (x >= th) cs += x;
  }
  chunk_prefix[threadIdx.x + 1] = cs;
  if (threadIdx.x == 0) {
    chunk_prefix[0] = mass_before;
    result = -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // sequential prefix over the threads' sums: fixed order
    float run = mass_before;
    for (int i = 1; i <= (int)blockDim.x; ++i) {
      run += chunk_prefix[i];
      chunk_prefix[i] = run;
    }
  }
  __syncthreads();
  const float total = total_known >= 0.f ? total_known : chunk_prefix[blockDim.x];
  const float target = u[r] * total;
  const float before = chunk_prefix[threadIdx.x], after = chunk_prefix[threadIdx.x + 1];
  if (target >= chunk_prefix[blockDim.x]) {
    // rounding put the target at or past the end of the range: its last kept entry
    int lastk = -1;
    for (int i = i0; i < i1; ++i)
      if (v.e(i) >= th) lastk = i;
    if (lastk >= 0) atomicMax(&result, lastk);
  } else if ((before <= target && target < after) || (threadIdx.x == 0 && target < before)) {
    float run = before;  // one thread gets here
    int lastk = -1, hit = -1;
    for (int i = i0; i < i1 && hit < 0; ++i) {
      const float x = v.e(i);
      if (x >= th) {
        run += x;
        lastk = i;
        if (run > target) hit = i;
      }
    }
    result = hit >= 0 ? hit : lastk;
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
  // chunks per row: enough blocks to fill the GPU, none shorter than 4096 entries
  int chunks = 296 / (n_rows < kSampleMaxRows ? n_rows : kSampleMaxRows);
  const int most = (vocab + 4095) / 4096;
  if (chunks > most) chunks = most;
  if (chunks > kSampleMaxChunks) chunks = kSampleMaxChunks;
  if (chunks < 1) chunks = 1;
  int chunk = ((vocab + chunks - 1) / chunks + 3) & ~3;
  chunks = (vocab + chunk - 1) / chunk;
  for (int r0 = 0; r0 < n_rows; r0 += kSampleMaxRows) {
    const int n = n_rows - r0 < kSampleMaxRows ? n_rows - r0 : kSampleMaxRows;
    FTK_LAUNCH(sample_kernel, dim3(chunks, n), kSampleThreads, 0, (cudaStream_t)stream, logits + (size_t)r0 * vocab, vocab,
               temperature + r0, top_k + r0, top_p + r0, u + r0, out + r0, chunk);
    FTK_LAUNCH_CHECK("sample");
  }
  return 0;
}
