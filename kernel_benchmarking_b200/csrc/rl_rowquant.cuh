// Row passes of the FP8-weight path: y = rmsnorm(x) * gamma @ (Wq * w_scale)^T with e4m3 weights and
// per-token e4m3 activations.
//
// Per-token quantisation needs the whole row before the first MMA (its absolute maximum), so the
// path has two kernels:
//   rowquant_kernel   one CTA per token row: sum of squares and amax of x*gamma in fp32, then
//                     q = e4m3(x*gamma * 448/amax) and row_scale = rsqrt(mean x^2 + eps) * amax/448.
//                     q does not depend on 1/rms, so one pass over x yields both; the row stays in
//                     registers between the two steps (x is read from memory once).
//   the CTA-pair GEMM (rl_prefill_pair.cuh, FP8 configuration): 256 x 256 tiles, k-blocks of 128 e4m3
//                     elements, kind::f8f6f4 MMAs with both operands from shared memory, two accumulators;
//                     epilogue y = acc * row_scale[m] * w_scale[n] -> bf16 -> TMA store.
#pragma once
#include <cuda_fp8.h>

#include "rl_prefill.cuh"

namespace rl {

// ---------------------------------------------------------------- row statistics + quantisation
struct RowQuantParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* gamma;  // [K] or nullptr
  uint8_t* q;                  // [M, ldq] e4m3 codes
  float* row_scale;            // [M]
  int M, K;
  long long ldx, ldq;
  float eps;
};

__device__ __forceinline__ float block_reduce_128(float v, bool is_max, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
#pragma unroll
  for (int w = 1; w < 4; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
  return r;
}

// Chunks of 8 bf16 (16 bytes) a thread keeps in registers between the statistics and the quantisation:
// rows of up to 128 threads x 8 chunks x 8 = 8192 elements are read from memory once, longer rows re-read
// the part beyond that.
constexpr int RQ_CACHED_CHUNKS = 8;

__device__ __forceinline__ void rowquant_stats(const uint4& u, const uint4& g, float& ssq, float& amax) {
  const uint32_t xs[4] = {u.x, u.y, u.z, u.w}, gs[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float x0 = bf16lo(xs[i]), x1 = bf16hi(xs[i]);
    ssq = fmaf(x0, x0, ssq);
    ssq = fmaf(x1, x1, ssq);
    amax = fmaxf(amax, fmaxf(fabsf(x0 * bf16lo(gs[i])), fabsf(x1 * bf16hi(gs[i]))));
  }
}
__device__ __forceinline__ uint2 rowquant_codes(const uint4& u, const uint4& g, float qs) {
  const uint32_t xs[4] = {u.x, u.y, u.z, u.w}, gs[4] = {g.x, g.y, g.z, g.w};
  uint32_t packed[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float a0 = bf16lo(xs[2 * i]) * bf16lo(gs[2 * i]) * qs, a1 = bf16hi(xs[2 * i]) * bf16hi(gs[2 * i]) * qs;
    const float a2 = bf16lo(xs[2 * i + 1]) * bf16lo(gs[2 * i + 1]) * qs,
                a3 = bf16hi(xs[2 * i + 1]) * bf16hi(gs[2 * i + 1]) * qs;
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a0, a1), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a2, a3), __NV_SATFINITE, __NV_E4M3);
    packed[i] = lo | (hi << 16);
  }
  return make_uint2(packed[0], packed[1]);
}

__global__ void __launch_bounds__(128) rowquant_kernel(const RowQuantParams p) {
  __shared__ float scratch[4];
  launch_dependents();  // lets the GEMM behind this kernel run its prologue; it waits before its first load
  const int m = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx);
  const uint4* gr = reinterpret_cast<const uint4*>(p.gamma);
  const int chunks = p.K >> 3;  // 8 bf16 per 16-byte chunk
  const uint4 ones = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);  // bf16 ones
  float ssq = 0.f, amax = 0.f;
  uint4 xc[RQ_CACHED_CHUNKS];
#pragma unroll
  for (int i = 0; i < RQ_CACHED_CHUNKS; ++i) {  // all of a thread's loads in flight together
    const int c = threadIdx.x + 128 * i;
    xc[i] = (c < chunks) ? xr[c] : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < RQ_CACHED_CHUNKS; ++i) {
    const int c = threadIdx.x + 128 * i;
    if (c < chunks) rowquant_stats(xc[i], gr != nullptr ? __ldg(gr + c) : ones, ssq, amax);
  }
  for (int c = threadIdx.x + 128 * RQ_CACHED_CHUNKS; c < chunks; c += 128)
    rowquant_stats(xr[c], gr != nullptr ? __ldg(gr + c) : ones, ssq, amax);
  ssq = block_reduce_128(ssq, false, scratch);
  amax = fmaxf(block_reduce_128(amax, true, scratch), 1e-30f);
  const float qs = 448.0f / amax;
  uint2* qr = reinterpret_cast<uint2*>(p.q + (size_t)m * p.ldq);
#pragma unroll
  for (int i = 0; i < RQ_CACHED_CHUNKS; ++i) {
    const int c = threadIdx.x + 128 * i;
    if (c < chunks) qr[c] = rowquant_codes(xc[i], gr != nullptr ? __ldg(gr + c) : ones, qs);
  }
  for (int c = threadIdx.x + 128 * RQ_CACHED_CHUNKS; c < chunks; c += 128)
    qr[c] = rowquant_codes(xr[c], gr != nullptr ? __ldg(gr + c) : ones, qs);
  if (threadIdx.x == 0) p.row_scale[m] = (1.0f / sqrtf(ssq / (float)p.K + p.eps)) * (amax / 448.0f);
}

// The statistics pass of rowquant_kernel on its own: inv_rms[m] = rsqrt(mean_k x^2 + eps) and, when asked for,
// amax[m] = max_k |x * gamma| (the fp32 product of the two bf16 values, which is exact).
__global__ void __launch_bounds__(128) rowstats_amax_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ gamma,
                                                            float* __restrict__ inv_rms, float* __restrict__ amax_out,
                                                            int M, int K, long long ldx, float eps) {
  __shared__ float scratch[4];
  const int m = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)m * ldx);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  const int chunks = K >> 3;
  float ssq = 0.f, amax = 0.f;
  for (int c = threadIdx.x; c < chunks; c += 128) {
    const uint4 u = xr[c];
    uint4 g = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);  // bf16 ones
    if (gr != nullptr) g = __ldg(gr + c);
    const uint32_t xs[4] = {u.x, u.y, u.z, u.w}, gs[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x0 = bf16lo(xs[i]), x1 = bf16hi(xs[i]);
      ssq = fmaf(x0, x0, ssq);
      ssq = fmaf(x1, x1, ssq);
      amax = fmaxf(amax, fmaxf(fabsf(x0 * bf16lo(gs[i])), fabsf(x1 * bf16hi(gs[i]))));
    }
  }
  ssq = block_reduce_128(ssq, false, scratch);
  amax = block_reduce_128(amax, true, scratch);
  if (threadIdx.x == 0) {
    inv_rms[m] = 1.0f / sqrtf(ssq / (float)K + eps);
    if (amax_out != nullptr) amax_out[m] = amax;
  }
}

}  // namespace rl
