// Per-head RMSNorm + partial NeoX rotation + scatter into pages, one pass over the projected heads.
//
// Stands for three reference kernels and three copies: the strided per-head norm
// (python/freetoken/kernel/triton/norm.py:42-75), the rope kernel
// (python/freetoken/kernel/triton/rope.py:28-91), the KV store
// (python/freetoken/kernel/csrc/jit/store.cu:27-53) and the .contiguous() of q, k and v
// (python/freetoken/models/minimax_m3/attention.py:87-89).
//
// One warp handles one (token, head).  The head vector is normed in registers, parked in shared
// memory so that a lane can read its rotation partner, rotated with the cos/sin row of the token's
// position, and written to its destination: a dense [T, heads, D] tensor (queries) or the row of a
// paged slab [pages, heads, page_size, D] that the token's slot names (keys, values).
#include "common.cuh"

namespace ftk {

constexpr int kMaxSections = 4;
constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHeadDim = 256;

struct Sections {
  FtkSection s[kMaxSections];
  int n;
  int total_heads;
};

template <typename T>
__global__ void norm_rope_store_kernel(const T* __restrict__ x, int n_tokens, int row_elems, int head_dim,
                                       int rotary_dim, const int32_t* __restrict__ positions,
                                       const float* __restrict__ rope_table, int max_pos, float eps, int gemma,
                                       Sections sec) {
  pdl_wait();
  pdl_trigger();
  __shared__ float park[kWarpsPerBlock][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int hs = blockIdx.x * kWarpsPerBlock + warp;  // head index among the sections' heads
  if (hs >= sec.total_heads) return;
  // which section, which head inside it
  int si = 0, hl = hs;
  while (si < sec.n - 1 && hl >= sec.s[si].n_heads) {
    hl -= sec.s[si].n_heads;
    ++si;
  }
  const FtkSection& S = sec.s[si];
  long long slot = 0;
  if (S.slab) {
    slot = S.slot_map[t];
    if (slot < 0 || slot >= (long long)S.num_pages * S.page_size) return;  // not stored
  }
  const T* src = x + (size_t)t * row_elems + (size_t)(S.first_head + hl) * head_dim;
  constexpr int kPer = kMaxHeadDim / 32;
  float v[kPer];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int d = lane + 32 * i;
    v[i] = d < head_dim ? to_float(src[d]) : 0.f;
    ss += v[i] * v[i];
  }
  if (S.norm_weight) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)head_dim + eps);
    const float one = gemma ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) v[i] = v[i] * inv * (S.norm_weight[d] + one);
    }
  }
  if (S.rotate && rotary_dim > 0) {
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) park[warp][d] = v[i];
    }
    __syncwarp();
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = rope_table + (size_t)pos * rotary_dim;
    const int half = rotary_dim >> 1;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int d = lane + 32 * i;
      if (d < half) {
        v[i] = park[warp][d] * cs[d] - park[warp][d + half] * cs[half + d];
      } else if (d < rotary_dim) {
        v[i] = park[warp][d] * cs[d - half] + park[warp][d - half] * cs[d];
      }
    }
  }
  T* dst;
  if (S.slab) {
    const long long page = slot / S.page_size, off = slot % S.page_size;
    dst = (T*)S.slab + (((size_t)page * S.n_heads + hl) * S.page_size + off) * head_dim;
  } else {
    dst = (T*)S.dense_out + ((size_t)t * S.n_heads + hl) * head_dim;
  }
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) dst[d] = from_float<T>(v[i]);
  }
}

// The same for bfloat16 heads of 64, 128 or 256 elements with 16-byte accesses: a head is spread over
// LPH = head_dim / 8 lanes (8 consecutive elements each), a warp takes 32 / LPH heads at once, and a
// lane gets its rotation partners from the lane half a rotary span away (rotary_dim a multiple of 16).
// (Measured at 2,048 tokens of 64 heads: 25.6 microseconds.  A block per token whose warps walk the token's
// heads with eight loads in flight per lane and the token's table rows read once took 30 to 37; four
// tokens per thread took 29.)
template <int LPH>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
norm_rope_store_vec_kernel(const __nv_bfloat16* __restrict__ x, int n_tokens, int row_elems, int rotary_dim,
                           const int32_t* __restrict__ positions, const float* __restrict__ rope_table, int max_pos,
                           float eps, int gemma, Sections sec) {
  pdl_wait();
  pdl_trigger();
  constexpr int kHeadDim = LPH * 8;
  constexpr int kHeadsPerWarp = 32 / LPH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int sub = lane / LPH, l = lane % LPH;
  const int hs = (blockIdx.x * kWarpsPerBlock + warp) * kHeadsPerWarp + sub;
  const bool live = hs < sec.total_heads;
  int si = 0, hl = live ? hs : 0;
  while (si < sec.n - 1 && hl >= sec.s[si].n_heads) {
    hl -= sec.s[si].n_heads;
    ++si;
  }
  const FtkSection& S = sec.s[si];
  long long slot = 0;
  bool store = live;
  if (S.slab) {
    slot = S.slot_map[t];
    if (slot < 0 || slot >= (long long)S.num_pages * S.page_size) store = false;  // not stored
  }
  const __nv_bfloat16* src = x + (size_t)t * row_elems + (size_t)(S.first_head + hl) * kHeadDim + l * 8;
  // everything this thread reads is asked for before the first use: the row, the norm weight, and the
  // two runs of eight table entries of its rotation (cos | sin halves of the position's row)
  const int half = rotary_dim >> 1;
  const bool rot = S.rotate && rotary_dim > 0;
  const bool low = l * 8 < half, in = l * 8 < rotary_dim;
  float w[8], ca[8], cb[8];
  if (S.norm_weight) {
    *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(S.norm_weight + l * 8);
    *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(S.norm_weight + l * 8 + 4);
  }
  if (rot && in) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = rope_table + (size_t)pos * rotary_dim;
    const int d0 = l * 8;
    const float* a = low ? cs + d0 : cs + d0 - half;  // cos of this element's pair
    const float* b = low ? cs + half + d0 : cs + d0;  // sin of this element's pair
    *reinterpret_cast<float4*>(ca) = *reinterpret_cast<const float4*>(a);
    *reinterpret_cast<float4*>(ca + 4) = *reinterpret_cast<const float4*>(a + 4);
    *reinterpret_cast<float4*>(cb) = *reinterpret_cast<const float4*>(b);
    *reinterpret_cast<float4*>(cb + 4) = *reinterpret_cast<const float4*>(b + 4);
  }
  float v[8];
  {
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (live) raw = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h2[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  }
  {
    // the heads of a warp may lie in different sections (with and without a norm): every lane runs
    // the shuffles, the ones with a norm use the result
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (S.norm_weight) {
      const float inv = rsqrtf(ss / (float)kHeadDim + eps);
      const float one = gemma ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = v[j] * inv * (w[j] + one);
    }
  }
  {
    // rotation partners: the lane half a rotary span away, on either side
    const int hop = half >> 3;  // lanes per half span
    float partner[8];
    if (hop > 0 && (hop & (hop - 1)) == 0) {  // a power of two: the partner is the lane with that bit flipped
#pragma unroll
      for (int j = 0; j < 8; ++j) partner[j] = __shfl_xor_sync(0xffffffffu, v[j], hop & 31);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float up = __shfl_down_sync(0xffffffffu, v[j], hop & 31);
        const float dn = __shfl_up_sync(0xffffffffu, v[j], hop & 31);
        partner[j] = low ? up : dn;
      }
    }
    if (rot && in) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = low ? v[j] * ca[j] - partner[j] * cb[j] : v[j] * ca[j] + partner[j] * cb[j];
    }
  }
  if (!store) return;
  __nv_bfloat16* dst;
  if (S.slab) {
    // (slots are 32-bit numbers: the 64-bit division costs several times the 32-bit one)
    const unsigned int us = (unsigned int)slot, ps = (unsigned int)S.page_size;
    const unsigned int page = us / ps, off = us % ps;
    dst = (__nv_bfloat16*)S.slab + (((size_t)page * S.n_heads + hl) * S.page_size + off) * kHeadDim;
  } else {
    dst = (__nv_bfloat16*)S.dense_out + ((size_t)t * S.n_heads + hl) * kHeadDim;
  }
  uint4 pk;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
  for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  *reinterpret_cast<uint4*>(dst + l * 8) = pk;
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_norm_rope_store(const void* x, int dtype, int n_tokens, int row_elems, int head_dim,
                                   int rotary_dim, const int32_t* positions, const float* rope_table,
                                   int max_pos, float eps, int gemma, int n_sections,
                                   const FtkSection* sections, void* stream) {
  FTK_REQUIRE(dtype_ok(dtype), "norm_rope_store: bad dtype %d", dtype);
  FTK_REQUIRE(n_sections >= 1 && n_sections <= kMaxSections, "norm_rope_store: %d sections (1..%d allowed)",
              n_sections, kMaxSections);
  FTK_REQUIRE(head_dim >= 1 && head_dim <= kMaxHeadDim, "norm_rope_store: head_dim=%d exceeds %d", head_dim,
              kMaxHeadDim);
  FTK_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
              "norm_rope_store: rotary_dim=%d must be even and <= head_dim=%d", rotary_dim, head_dim);
  FTK_REQUIRE(n_tokens >= 0 && n_tokens <= 65535 * 1024, "norm_rope_store: bad token count %d", n_tokens);
  if (n_tokens == 0) return 0;
  FTK_REQUIRE(x && sections, "norm_rope_store: null pointer");
  Sections sec;
  sec.n = n_sections;
  sec.total_heads = 0;
  bool any_rot = false;
  for (int i = 0; i < n_sections; ++i) {
    sec.s[i] = sections[i];
    const FtkSection& S = sections[i];
    FTK_REQUIRE(S.n_heads >= 1 && S.first_head >= 0 && (size_t)(S.first_head + S.n_heads) * head_dim <= (size_t)row_elems,
                "norm_rope_store: section %d names heads outside the row", i);
    FTK_REQUIRE((S.dense_out != nullptr) != (S.slab != nullptr),
                "norm_rope_store: section %d needs exactly one destination", i);
    if (S.slab) FTK_REQUIRE(S.slot_map && S.page_size >= 1 && S.num_pages >= 1, "norm_rope_store: section %d has a bad slab", i);
    any_rot = any_rot || S.rotate;
    sec.total_heads += S.n_heads;
  }
  if (any_rot && rotary_dim > 0)
    FTK_REQUIRE(positions && rope_table && max_pos >= 1, "norm_rope_store: rotation needs positions and a table");
  cudaStream_t s = (cudaStream_t)stream;
  // 16-byte accesses: bfloat16 heads of 64 / 128 / 256, rotation spans of whole lanes, aligned tensors
  bool vec = dtype == FTK_BF16 && (head_dim == 64 || head_dim == 128 || head_dim == 256) && rotary_dim % 16 == 0 &&
             row_elems % 8 == 0 && ((uintptr_t)x & 15) == 0;
  for (int i = 0; i < n_sections && vec; ++i) {
    const FtkSection& S = sections[i];
    if (((uintptr_t)S.dense_out & 15) || ((uintptr_t)S.slab & 15) || ((uintptr_t)S.norm_weight & 15)) vec = false;
  }
  const int bx = (sec.total_heads + kWarpsPerBlock - 1) / kWarpsPerBlock;
  for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
    const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
    Sections part = sec;
    for (int i = 0; i < n_sections; ++i) {
      if (part.s[i].dense_out)
        part.s[i].dense_out = (char*)part.s[i].dense_out + (size_t)t0 * part.s[i].n_heads * head_dim * dtype_size(dtype);
      if (part.s[i].slot_map) part.s[i].slot_map += t0;
    }
    dim3 grid(bx, nt);
    if (vec) {
      note_variant("head norm + rotation + cache write: a warp per head, 16-byte accesses");
      const int lph = head_dim / 8, per_block = kWarpsPerBlock * (32 / lph);
      dim3 vgrid((sec.total_heads + per_block - 1) / per_block, nt);
      const __nv_bfloat16* xs = (const __nv_bfloat16*)x + (size_t)t0 * row_elems;
      const int32_t* ps = positions ? positions + t0 : nullptr;
      if (lph == 8)
        FTK_LAUNCH(norm_rope_store_vec_kernel<8>, vgrid, kWarpsPerBlock * 32, 0, s, xs, nt, row_elems, rotary_dim, ps,
                   rope_table, max_pos, eps, gemma, part);
      else if (lph == 16)
        FTK_LAUNCH(norm_rope_store_vec_kernel<16>, vgrid, kWarpsPerBlock * 32, 0, s, xs, nt, row_elems, rotary_dim, ps,
                   rope_table, max_pos, eps, gemma, part);
      else
        FTK_LAUNCH(norm_rope_store_vec_kernel<32>, vgrid, kWarpsPerBlock * 32, 0, s, xs, nt, row_elems, rotary_dim, ps,
                   rope_table, max_pos, eps, gemma, part);
    } else if (dtype == FTK_F32)
      (note_variant("head norm + rotation + cache write: a warp per head"),
       FTK_LAUNCH(norm_rope_store_kernel<float>, grid, kWarpsPerBlock * 32, 0, s, 
          (const float*)x + (size_t)t0 * row_elems, nt, row_elems, head_dim, rotary_dim,
          positions ? positions + t0 : nullptr, rope_table, max_pos, eps, gemma, part));
    else
      FTK_LAUNCH(norm_rope_store_kernel<__nv_bfloat16>, grid, kWarpsPerBlock * 32, 0, s, 
          (const __nv_bfloat16*)x + (size_t)t0 * row_elems, nt, row_elems, head_dim, rotary_dim,
          positions ? positions + t0 : nullptr, rope_table, max_pos, eps, gemma, part);
  }
  FTK_LAUNCH_CHECK("norm_rope_store");
  return 0;
}
