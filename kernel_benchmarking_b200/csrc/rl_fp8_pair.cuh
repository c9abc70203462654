// FP8-weight path: y = rmsnorm(x) * gamma @ (Wq * w_scale)^T with e4m3 weights and per-token e4m3
// activations.
//
// Per-token quantisation needs the whole row before the first MMA (its absolute maximum), so the
// path has two kernels:
//   rowquant_kernel   one CTA per token row: sum of squares and amax of x*gamma in fp32, then
//                     q = e4m3(x*gamma * 448/amax) and row_scale = rsqrt(mean x^2 + eps) * amax/448.
//                     q does not depend on 1/rms, so one pass over x yields both.
//   fp8_pair_kernel   CTA pairs (cta_group::2), 256 x 256 tiles, k-blocks of 128 e4m3 elements,
//                     kind::f8f6f4 MMAs with both operands from shared memory, two accumulators in
//                     TMEM so the epilogue overlaps the next tile; epilogue y = acc * row_scale[m] *
//                     w_scale[n] -> bf16 -> TMA store.
// Per k-block and SM the GEMM moves 32 KB into shared memory and reads 48 KB of operands for twice
// the math of a bf16 k-block, which is where its speed-up over the bf16 kernel comes from.
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

__global__ void __launch_bounds__(128) rowquant_kernel(const RowQuantParams p) {
  __shared__ float scratch[4];
  launch_dependents();  // lets the GEMM behind this kernel run its prologue; it waits before its first load
  const int m = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx);
  const uint4* gr = reinterpret_cast<const uint4*>(p.gamma);
  const int chunks = p.K >> 3;  // 8 bf16 per 16-byte chunk
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
  amax = fmaxf(block_reduce_128(amax, true, scratch), 1e-30f);
  const float qs = 448.0f / amax;
  uint2* qr = reinterpret_cast<uint2*>(p.q + (size_t)m * p.ldq);
  for (int c = threadIdx.x; c < chunks; c += 128) {
    const uint4 u = xr[c];
    uint4 g = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    if (gr != nullptr) g = __ldg(gr + c);
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
    qr[c] = make_uint2(packed[0], packed[1]);
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

// ---------------------------------------------------------------- FP8 pair GEMM
struct Fp8GemmParams {
  int M, N, K;
  const float* row_scale;  // [M]
  const float* w_scale;    // [N]
  int m_tiles, n_tiles, group_m;
  int* status;
};

template <int STAGES_>
struct Fp8PairCfg {
  static constexpr int BN = 256, STAGES = STAGES_;
  static constexpr int THREADS = 64 + 128;
  static constexpr int A_BYTES = 128 * 128;  // 128 rows x 128 e4m3
  static constexpr int B_BYTES = 128 * 128;  // this CTA's half of the W tile
  static constexpr int EPI_BYTES = 128 * 64 * 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_EPI = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_WS = OFF_EPI + 2 * EPI_BYTES;  // [2][256] w_scale slice of the tile being drained
  static constexpr int OFF_BAR = OFF_WS + 2 * 256 * 4;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 64;
  static constexpr int TMEM_COLS = 512;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::THREADS, 1)
fp8_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_y, const Fp8GemmParams p) {
  constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  if (sbase & 1023u) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, (int)DEV_BAD_SMEM_ALIGNMENT);
    return;
  }
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  auto bar_ready = [&](int s) { return bar0 + 8u * s; };            // rank 0 only: 2 arrivals + tx of both CTAs
  auto bar_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };  // local, MMA commit multicast
  auto bar_tfull = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto bar_tempty = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };  // rank 0 only, 8 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_MISC);
  volatile int* epi_go = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC + 8);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(smem + Cfg::OFF_MISC + 16);
  float* wsc = reinterpret_cast<float*>(smem + Cfg::OFF_WS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
  const int KB = (p.K + 127) >> 7;
  const int total_tiles = p.m_tiles * p.n_tiles;
  PrefillParams tp{};  // tile order shared with the bf16 kernels
  tp.m_tiles = p.m_tiles; tp.n_tiles = p.n_tiles; tp.group_m = p.group_m;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_ready(s), 2);
      mbar_init(bar_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull(a), 1);
      mbar_init(bar_tempty(a), 8);
    }
    ctl->abort = 0;
    ctl->status = p.status;
    ctl->limit_ns = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, own halves)
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    const uint32_t lead_ready0 = mapa_shared(bar_ready(0), 0);
    grid_dependency_wait();  // the quantised activations come from the kernel launched just before
    for (int t = pair; ok && t < total_tiles; t += n_pairs) {
      int mt, nt;
      prefill_tile_coords(t, tp, mt, nt);
      for (int kb = 0; kb < KB; ++kb) {
        if (!mbar_wait_warp(bar_empty(s), ph ^ 1, ctl, 0, STAGES + s, kb)) { ok = false; break; }
        if (elect_one()) {
          const uint32_t lead_ready = lead_ready0 + 8u * s;
          mbar_expect_tx_cluster(lead_ready, Cfg::A_BYTES + Cfg::B_BYTES);
          tma_load_2d_pair(sbase + Cfg::OFF_A + s * Cfg::A_BYTES, &tm_a, lead_ready, kb * 128, mt * 256 + (int)rank * 128);
          tma_load_2d_pair(sbase + Cfg::OFF_B + s * Cfg::B_BYTES, &tm_w, lead_ready, kb * 128, nt * BN + (int)rank * 128);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer (rank 0 only)
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc(256, BN, 0, 0);  // e4m3 x e4m3, fp32 accumulate
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      const uint64_t adesc0 = make_sw128_kmajor_desc(sbase + Cfg::OFF_A);
      const uint64_t bdesc0 = make_sw128_kmajor_desc(sbase + Cfg::OFF_B);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int t = pair; ok && t < total_tiles; t += n_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait_warp(bar_tempty(acc), aph ^ 1u, ctl, 1, 2 * STAGES + 2 + acc, it)) break;
        const uint32_t d = tmem_base + acc * BN;
        uint32_t ready_now = mbar_test_wait(bar_ready(s), ph);
        for (int kb = 0; kb < KB; ++kb) {
          if (!ready_now) {
            if (!mbar_wait(bar_ready(s), ph, ctl, 1, s, kb)) { ok = false; break; }
          }
          tc_fence_after();
          const int sn = (s + 1 == STAGES) ? 0 : s + 1;
          const uint32_t phn = (s + 1 == STAGES) ? (ph ^ 1u) : ph;
          ready_now = mbar_test_wait(bar_ready(sn), phn);
          umma_kblock_f8_ss_pair(d, adesc0 + (uint64_t)(s * (Cfg::A_BYTES >> 4)),
                                 bdesc0 + (uint64_t)(s * (Cfg::B_BYTES >> 4)), idesc, (uint32_t)(kb != 0), bar_empty(s),
                                 leader);
          s = sn;
          ph = phn;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) umma_commit_pair_pred(bar_tfull(acc), leader);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t swz = (uint32_t)(row & 7);
    const int epi_tid = threadIdx.x - 64;
    const uint32_t lead_tempty0 = mapa_shared(bar_tempty(0), 0);
    const uint64_t pol_y = l2_policy_evict_first();
    bool ok = true;
    int it = 0;
    uint32_t chunk_no = 0;
    for (int t = pair; ok && t < total_tiles; t += n_pairs, ++it) {
      int mt, nt;
      prefill_tile_coords(t, tp, mt, nt);
      const int acc = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      // stage this tile's 256 per-channel scales while the accumulator is still filling
      {
        const int n = nt * BN + epi_tid;
        wsc[acc * 256 + epi_tid] = (n < p.N) ? __ldg(p.w_scale + n) : 0.f;
        wsc[acc * 256 + 128 + epi_tid] = (n + 128 < p.N) ? __ldg(p.w_scale + n + 128) : 0.f;
      }
      grid_dependency_wait();
      const int m = mt * 256 + (int)rank * 128 + row;
      const float rsc = (m < p.M) ? __ldg(p.row_scale + m) : 0.f;
      mbar_wait(bar_tfull(acc), aph, ctl, 3, 2 * STAGES + acc, it);
      named_bar_sync(3, 128);
      if (epi_tid == 0) *epi_go = ctl->abort ? 0 : 1;
      named_bar_sync(4, 128);
      ok = (*epi_go != 0);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c, ++chunk_no) {
        uint8_t* stage = smem + Cfg::OFF_EPI + (chunk_no & 1) * Cfg::EPI_BYTES;
        if (epi_tid == 0) tma_store_wait_read<1>();
        named_bar_sync(1, 128);
        uint32_t v0[32], v1[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * 64, v0);
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * 64 + 32, v1);
        tmem_wait_ld();
        if (c == BN / 64 - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * acc);
        }
        const float* wc = wsc + acc * 256 + c * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 w0 = *reinterpret_cast<const float4*>(wc + 8 * j), w1 = *reinterpret_cast<const float4*>(wc + 8 * j + 4);
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(v0[8 * j + 0]) * rsc * w0.x, __uint_as_float(v0[8 * j + 1]) * rsc * w0.y);
          o.y = pack_bf16x2(__uint_as_float(v0[8 * j + 2]) * rsc * w0.z, __uint_as_float(v0[8 * j + 3]) * rsc * w0.w);
          o.z = pack_bf16x2(__uint_as_float(v0[8 * j + 4]) * rsc * w1.x, __uint_as_float(v0[8 * j + 5]) * rsc * w1.y);
          o.w = pack_bf16x2(__uint_as_float(v0[8 * j + 6]) * rsc * w1.z, __uint_as_float(v0[8 * j + 7]) * rsc * w1.w);
          *reinterpret_cast<uint4*>(stage + row * 128 + (((uint32_t)j ^ swz) << 4)) = o;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 w0 = *reinterpret_cast<const float4*>(wc + 32 + 8 * j),
                       w1 = *reinterpret_cast<const float4*>(wc + 32 + 8 * j + 4);
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(v1[8 * j + 0]) * rsc * w0.x, __uint_as_float(v1[8 * j + 1]) * rsc * w0.y);
          o.y = pack_bf16x2(__uint_as_float(v1[8 * j + 2]) * rsc * w0.z, __uint_as_float(v1[8 * j + 3]) * rsc * w0.w);
          o.z = pack_bf16x2(__uint_as_float(v1[8 * j + 4]) * rsc * w1.x, __uint_as_float(v1[8 * j + 5]) * rsc * w1.y);
          o.w = pack_bf16x2(__uint_as_float(v1[8 * j + 6]) * rsc * w1.z, __uint_as_float(v1[8 * j + 7]) * rsc * w1.w);
          *reinterpret_cast<uint4*>(stage + row * 128 + (((uint32_t)(4 + j) ^ swz) << 4)) = o;
        }
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        if (epi_tid == 0) {
          const int n0 = nt * BN + c * 64;
          if (n0 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage), n0, mt * 256 + (int)rank * 128, pol_y);
          tma_store_commit();
        }
      }
    }
    if (epi_tid == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (ctl->abort) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace rl
