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

// Chunks of 8 bf16 (16 bytes) a thread keeps between the statistics and the quantisation, as the fp32 products
// x * gamma.  The CTA is sized to the row (128 threads up to K = 4096, 256 up to 8192, 512 beyond), so rows of up
// to 512 threads x 4 chunks x 8 = 16384 elements are read from memory once and multiplied once; longer rows
// re-read the part beyond that.  Four chunks per thread keep the kernel at 8 CTAs of 128 threads per SM, which it
// needs to cover DRAM latency.
constexpr int RQ_CACHED_CHUNKS = 4;

// packed fp32 pair multiply (sm_100): {a.x * b.x, a.y * b.y}, each rounded to nearest like a scalar multiply
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 r;
  asm("{\n\t.reg .b64 va, vb, vc;\n\t"
      "mov.b64 va, {%2, %3};\n\tmov.b64 vb, {%4, %5};\n\t"
      "mul.rn.f32x2 vc, va, vb;\n\t"
      "mov.b64 {%0, %1}, vc;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return r;
}

// One chunk: the eight products x * gamma (exact in fp32), their absolute maximum and the sum of squares of x.
__device__ __forceinline__ void rowquant_products(const uint4& u, const uint4& g, float2 (&prod)[4], float2& ssq,
                                                  float& amax) {
  const uint32_t xs[4] = {u.x, u.y, u.z, u.w}, gs[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 xv = make_float2(bf16lo(xs[i]), bf16hi(xs[i]));
    ffma2_sq(ssq, xv.x, xv.y);
    prod[i] = fmul2(xv, make_float2(bf16lo(gs[i]), bf16hi(gs[i])));
    amax = fmaxf(amax, fmaxf(fabsf(prod[i].x), fabsf(prod[i].y)));
  }
}
// e4m3 codes of eight products scaled by qs = 448 / amax (one rounding of the product, one of the code)
__device__ __forceinline__ uint2 rowquant_codes(const float2 (&prod)[4], float qs) {
  const float2 q2 = make_float2(qs, qs);
  uint32_t c[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = __nv_cvt_float2_to_fp8x2(fmul2(prod[i], q2), __NV_SATFINITE, __NV_E4M3);
  return make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
}

template <int NT>
__global__ void __launch_bounds__(NT, 1024 / NT) rowquant_kernel(const RowQuantParams p) {
  __shared__ float2 scratch[NT / 32];
  launch_dependents();  // lets the GEMM behind this kernel run its prologue; it waits before its first load
  // launched with programmatic stream serialisation itself: behind a kernel that lets its dependents start early
  // (this library's small-M kernel does) the CTAs are already resident when that kernel ends, which takes this
  // kernel's launch latency out of a chain of decode steps.  Nothing is read before everything in front is complete.
  grid_dependency_wait();
  const int m = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx);
  const uint4* gr = reinterpret_cast<const uint4*>(p.gamma);
  const int chunks = p.K >> 3;  // 8 bf16 per 16-byte chunk
  const uint4 ones = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);  // bf16 ones
  float2 ssq2 = make_float2(0.f, 0.f);
  float amax = 0.f;
  uint4 xc[RQ_CACHED_CHUNKS];
  float2 prod[RQ_CACHED_CHUNKS][4];
#pragma unroll
  for (int i = 0; i < RQ_CACHED_CHUNKS; ++i) {  // all of a thread's loads in flight together
    const int c = threadIdx.x + NT * i;
    xc[i] = (c < chunks) ? xr[c] : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < RQ_CACHED_CHUNKS; ++i) {
    const int c = threadIdx.x + NT * i;
    rowquant_products(xc[i], (gr != nullptr && c < chunks) ? __ldg(gr + c) : ones, prod[i], ssq2, amax);  // zeros beyond the row
  }
  for (int c = threadIdx.x + NT * RQ_CACHED_CHUNKS; c < chunks; c += NT) {
    float2 pr[4];
    rowquant_products(xr[c], gr != nullptr ? __ldg(gr + c) : ones, pr, ssq2, amax);
  }
  // both reductions at once: warp butterflies, then the four warps' results through shared memory
  float ssq = ssq2.x + ssq2.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  }
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = make_float2(ssq, amax);
  __syncthreads();
  ssq = 0.f;
  amax = 1e-30f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) {
    ssq += scratch[w].x;
    amax = fmaxf(amax, scratch[w].y);
  }
  const float qs = 448.0f / amax;
  uint2* qr = reinterpret_cast<uint2*>(p.q + (size_t)m * p.ldq);
#pragma unroll
  for (int i = 0; i < RQ_CACHED_CHUNKS; ++i) {
    const int c = threadIdx.x + NT * i;
    if (c < chunks) qr[c] = rowquant_codes(prod[i], qs);
  }
  for (int c = threadIdx.x + NT * RQ_CACHED_CHUNKS; c < chunks; c += NT) {
    float2 pr[4];
    float2 s_unused = make_float2(0.f, 0.f);
    float a_unused = 0.f;
    rowquant_products(xr[c], gr != nullptr ? __ldg(gr + c) : ones, pr, s_unused, a_unused);
    qr[c] = rowquant_codes(pr, qs);
  }
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
