// Fused RMSNorm -> Linear for M >= 128 tokens (tensor-core bound).
//
//   y[m, n] = rsqrt(mean_k x[m,k]^2 + eps) * sum_k (x[m,k] * gamma[k]) * W[n,k]
//
// One persistent CTA per SM walks 128 x BN output tiles.  Warp roles:
//   warp 0      TMA producer: x tile [128 x 64], W tile [BN x 64], gamma slice, per k-block
//   warp 1      UMMA issuer (tcgen05.mma, fp32 accumulators in TMEM, two buffers)
//   TG x 4 warps transform (k-blocks dealt round-robin to TG groups): each thread owns one token row of the landed x tile,
//               accumulates its sum of squares in fp32 and folds gamma into the
//               tile - back into shared memory (A_SS_FOLD) or into tensor memory
//               as the UMMA A operand (A_TS_FOLD)
//   last 4 warps epilogue: tcgen05.ld, multiply each row by its 1/rms, bf16,
//               swizzled staging tile, TMA store
// The reference's fused kernels use the same algebra - accumulate x@W^T and
// sum(x^2) together, scale in the epilogue (python/bench_kernels/helion/
// rmsnorm_linear.py:20-34, res/c2_kernels/rmsnorm_linear_4096x4096x4096.py:57-77).
#pragma once
#include "rl_ptx.cuh"

namespace rl {

enum AMode : int { A_SS_DIRECT = 0, A_SS_FOLD = 1, A_TS_FOLD = 2 };

struct PrefillParams {
  int M, N, K;
  float eps;
  const __nv_bfloat16* gamma;  // [K] or nullptr (only with A_SS_DIRECT / treated as ones)
  int m_tiles, n_tiles, group_m;
  int* status;  // RL_STATUS_INTS ints or nullptr
  const float* row_rstd;  // [M] 1/rms per token from rowstats_kernel (kernels built with PRESTATS), else nullptr;
                          // FP8 pair kernel: the per-token scale rsqrt(mean x^2 + eps) * amax / 448 from rowquant_kernel
  const float* w_scale;   // FP8 pair kernel: [N] per-output-channel weight scales
  // Pair kernels: the last `tail_tiles` tiles are each cut along K into `tail_split` (2, 3 or 4) slices computed by
  // different CTA pairs (0 = off).  tail_counters: 2 per (tail tile, CTA rank), zero between launches;
  // tail_partials: one 128-row x 256-column fp32 block per (tail tile, slice, CTA rank).
  int tail_tiles, tail_split;
  unsigned* tail_counters;
  float* tail_partials;
  int extra_kb;  // pair kernels: k-blocks appended from a second pair of operand matrices (0 or 1)
  int x_from_prepass;  // pair kernels: the activation matrix is written by the kernel launched just before (rowscale_kernel)
  // Pair kernels: best-effort alignment of the resident pairs at tile boundaries (nullptr = off).  round_words[pair]
  // holds (round_epoch << 12) | the index of the tile that pair has started (0xfff once it has none left); a pair
  // about to start its i-th tile gives the others up to round_wait_ns to get there.  Timing only: nothing depends on it.
  unsigned* round_words;
  unsigned round_epoch;    // 20 bits, different for every launch
  unsigned round_wait_ns;
};

// Row statistics on their own: rstd[m] = rsqrt(mean_k x[m,k]^2 + eps).  One warp per token row, 16-byte
// loads, butterfly reduction.  Used by the PRESTATS kernels, where every column tile would otherwise
// recompute the same sums of squares (N/256 times per row).
__global__ void __launch_bounds__(128) rowstats_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ rstd,
                                                       int M, int K, long long ldx, float eps) {
  launch_dependents();  // the GEMM behind this kernel may start loading tiles; it waits before it reads rstd
  const int m = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (m >= M) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)m * ldx);
  const int chunks = K >> 3;
  float2 acc = make_float2(0.f, 0.f);
  int c = lane;
  for (; c + 96 < chunks; c += 128) {  // four independent 16-byte loads in flight per lane
    uint4 u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) u[i] = xr[c + 32 * i];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ffma2_sq(acc, bf16lo(u[i].x), bf16hi(u[i].x));
      ffma2_sq(acc, bf16lo(u[i].y), bf16hi(u[i].y));
      ffma2_sq(acc, bf16lo(u[i].z), bf16hi(u[i].z));
      ffma2_sq(acc, bf16lo(u[i].w), bf16hi(u[i].w));
    }
  }
  for (; c < chunks; c += 32) {
    const uint4 u = xr[c];
    ffma2_sq(acc, bf16lo(u.x), bf16hi(u.x));
    ffma2_sq(acc, bf16lo(u.y), bf16hi(u.y));
    ffma2_sq(acc, bf16lo(u.z), bf16hi(u.z));
    ffma2_sq(acc, bf16lo(u.w), bf16hi(u.w));
  }
  float s = acc.x + acc.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) rstd[m] = 1.0f / sqrtf(s / (float)K + eps);
}

// Row statistics and the gamma fold in one pass over x: rstd[m] as above and xs[m, k] = bf16(x[m, k] * gamma[k]), the
// product rounded once to bf16 exactly as the GEMM kernels' transform warps round it.  For wide layers: each
// activation is then folded once here instead of once per 256-channel column tile in the main loop, and the GEMM
// runs without transform warps (x straight from shared memory, two accumulators).  One warp per token row.
__global__ void __launch_bounds__(128) rowscale_kernel(const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ gamma,
                                                       __nv_bfloat16* __restrict__ xs, float* __restrict__ rstd, int M,
                                                       int K, long long ldx, long long ldxs, float eps) {
  launch_dependents();  // the GEMM behind this kernel sets itself up meanwhile; it waits before its first load
  const int m = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (m >= M) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)m * ldx);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  uint4* out = reinterpret_cast<uint4*>(xs + (size_t)m * ldxs);
  const int chunks = K >> 3;
  float2 acc = make_float2(0.f, 0.f);
  auto one = [&](const uint4 u, const uint4 g, int c) {
    ffma2_sq(acc, bf16lo(u.x), bf16hi(u.x));
    ffma2_sq(acc, bf16lo(u.y), bf16hi(u.y));
    ffma2_sq(acc, bf16lo(u.z), bf16hi(u.z));
    ffma2_sq(acc, bf16lo(u.w), bf16hi(u.w));
    out[c] = make_uint4(mul_bf16x2(u.x, g.x), mul_bf16x2(u.y, g.y), mul_bf16x2(u.z, g.z), mul_bf16x2(u.w, g.w));
  };
  int c = lane;
  for (; c + 96 < chunks; c += 128) {  // four independent 16-byte loads of x (and of gamma, from L1) in flight per lane
    uint4 u[4], g[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) u[i] = xr[c + 32 * i];
#pragma unroll
    for (int i = 0; i < 4; ++i) g[i] = __ldg(gr + c + 32 * i);
#pragma unroll
    for (int i = 0; i < 4; ++i) one(u[i], g[i], c + 32 * i);
  }
  for (; c < chunks; c += 32) one(xr[c], __ldg(gr + c), c);
  float s = acc.x + acc.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) rstd[m] = 1.0f / sqrtf(s / (float)K + eps);
}

template <int BN_, int STAGES_, int AMODE_, int TG_ = 2>
struct PrefillCfg {
  static constexpr int BM = 128, BK = 64, BN = BN_, STAGES = STAGES_, AMODE = AMODE_;
  static constexpr int TG = TG_;                       // transform groups of 4 warps; group g takes k-blocks j = g (mod TG)
  static constexpr int THREADS = 64 + 128 * TG + 128;  // producer, MMA, TG x 4 transform warps, 4 epilogue warps
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int G_BYTES = BK * 2;
  static constexpr int EPI_BYTES = 128 * 64 * 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_EPI = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_G = OFF_EPI + 2 * EPI_BYTES;
  static constexpr int OFF_RS = OFF_G + STAGES * G_BYTES;
  static constexpr int OFF_BAR = OFF_RS + TG * 2 * 128 * 4;
  static constexpr int NUM_BARS = 3 * STAGES + 6;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;  // + alignment slack
  static constexpr int TMEM_COLS = 512;
  static constexpr int A_COL0 = 2 * BN;  // TMEM columns of the A stages (A_TS_FOLD)
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN");
  // A ring slot must always be served by the same transform group: a group that skipped a slot's
  // previous phase could mistake that phase for the one it is waiting for (parity waits alias).
  static_assert(STAGES % TG == 0, "STAGES must be a multiple of TG");
  static_assert(AMODE != A_TS_FOLD || 2 * BN + STAGES * 32 <= 512, "TMEM budget");
  static_assert(2 * BN <= 512, "TMEM budget");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(B_BYTES % 1024 == 0, "B stage alignment");
};

__device__ __forceinline__ void prefill_tile_coords(int t, const PrefillParams& p, int& mt, int& nt) {
  // Groups of `group_m` row-tiles are swept across all column tiles before the
  // next group starts, so one group of x rows stays in L2 while W streams past.
  const int per_group = p.group_m * p.n_tiles;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int m_first = g * p.group_m;
  const int gm = min(p.group_m, p.m_tiles - m_first);
  nt = r / gm;
  mt = m_first + (r - nt * gm);
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_y, const PrefillParams p) {
  constexpr int BN = Cfg::BN, STAGES = Cfg::STAGES, AMODE = Cfg::AMODE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_xf = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
  auto bar_tfull = [&](int a) { return bar0 + 8u * (3 * STAGES + a); };
  auto bar_tempty = [&](int a) { return bar0 + 8u * (3 * STAGES + 2 + a); };
  auto bar_rs = [&](int a) { return bar0 + 8u * (3 * STAGES + 4 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_MISC);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(smem + Cfg::OFF_MISC + 16);
  float* rs = reinterpret_cast<float*>(smem + Cfg::OFF_RS);
  volatile int* epi_go = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (p.K + 63) >> 6;
  const int total_tiles = p.m_tiles * p.n_tiles;
  const bool has_gamma = (p.gamma != nullptr);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_xf(s), 4);
      mbar_init(bar_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull(a), 1);
      mbar_init(bar_tempty(a), 4);
      mbar_init(bar_rs(a), 4 * Cfg::TG);
    }
    ctl->abort = 0;
    ctl->status = p.status;
    ctl->limit_ns = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_x);
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        int mt, nt;
        prefill_tile_coords(t, p, mt, nt);
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait_warp(bar_empty(s), ph ^ 1, ctl, 0, 2 * STAGES + s, kb)) { ok = false; break; }
          if (elect_one()) {
            const int kvalid = min(64, p.K - kb * 64);
            const uint32_t gbytes = (has_gamma && AMODE != A_SS_DIRECT) ? (uint32_t)kvalid * 2u : 0u;
            mbar_expect_tx(bar_full(s), Cfg::A_BYTES + Cfg::B_BYTES + gbytes);
            tma_load_2d(sbase + Cfg::OFF_A + s * Cfg::A_BYTES, &tm_x, bar_full(s), kb * 64, mt * 128);
            tma_load_2d(sbase + Cfg::OFF_B + s * Cfg::B_BYTES, &tm_w, bar_full(s), kb * 64, nt * BN);
            if (gbytes) bulk_load_1d(sbase + Cfg::OFF_G + s * Cfg::G_BYTES, p.gamma + kb * 64, gbytes, bar_full(s));
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    {
      constexpr uint32_t idesc = make_idesc(128, BN, 1, 1);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait_warp(bar_tempty(acc), aph ^ 1, ctl, 1, 3 * STAGES + 2 + acc, it)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait_warp(bar_full(s), ph, ctl, 1, s, kb)) { ok = false; break; }
          if (AMODE != A_SS_DIRECT) {
            if (!mbar_wait_warp(bar_xf(s), ph, ctl, 1, STAGES + s, kb)) { ok = false; break; }
          }
          tc_fence_after();
          const uint64_t bdesc = make_sw128_kmajor_desc(sbase + Cfg::OFF_B + s * Cfg::B_BYTES);
          const uint64_t adesc = make_sw128_kmajor_desc(sbase + Cfg::OFF_A + s * Cfg::A_BYTES);
          const uint32_t a_t = tmem_base + Cfg::A_COL0 + s * 32;
          if (AMODE == A_SS_DIRECT) {
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < 4; ++k) umma_ss(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
            }
            __syncwarp();
            // the row-statistics warps must be done reading the x tile before its slot is recycled
            if (!mbar_wait_warp(bar_xf(s), ph, ctl, 1, STAGES + s, kb)) { ok = false; break; }
            if (elect_one()) umma_commit(bar_empty(s));
          } else if (elect_one()) {
            if (AMODE == A_TS_FOLD) {
#pragma unroll
              for (int k = 0; k < 4; ++k) umma_ts(d, a_t + k * 8, bdesc + 2 * k, idesc, (kb | k) != 0);
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) umma_ss(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
            }
            umma_commit(bar_empty(s));
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok && elect_one()) umma_commit(bar_tfull(acc));
        __syncwarp();
      }
    }
  } else if (warp < 2 + 4 * Cfg::TG) {
    // ------------------------------------------------------------ transform: sum of squares + gamma fold
    constexpr int TG = Cfg::TG;
    const int grp = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t swz = (uint32_t)(row & 7);
    bool ok = true;
    int it = 0;
    int j_base = 0;  // index of this tile's first k-block in the CTA's running count (ring slot = j % STAGES)
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it, j_base += KB) {
      const int acc = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      float ss = 0.f;
      for (int kb = (grp - j_base % TG + TG) % TG; kb < KB; kb += TG) {
        const int j = j_base + kb;
        const int s = j % STAGES;
        const uint32_t ph = (uint32_t)(j / STAGES) & 1u;
        ok = mbar_wait(bar_full(s), ph, ctl, 2, s, kb);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        uint8_t* a_row = smem + Cfg::OFF_A + s * Cfg::A_BYTES + row * 128;
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 u = *reinterpret_cast<const uint4*>(a_row + ((c ^ swz) << 4));
          v[4 * c + 0] = u.x; v[4 * c + 1] = u.y; v[4 * c + 2] = u.z; v[4 * c + 3] = u.w;
        }
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const float lo = bf16lo(v[jj]), hi = bf16hi(v[jj]);
          s0 = fmaf(lo, lo, s0);
          s1 = fmaf(hi, hi, s1);
        }
        ss += s0 + s1;
        if (AMODE != A_SS_DIRECT) {
          if (has_gamma) {
            const uint4* g = reinterpret_cast<const uint4*>(smem + Cfg::OFF_G + s * Cfg::G_BYTES);
            const int kvalid = p.K - kb * 64;  // >= 64 except in a ragged last block
            if (kvalid >= 64) {
              // the eight gamma loads back to back, no branch between them (a branch per load exposes each latency)
              uint4 gv[8];
#pragma unroll
              for (int c = 0; c < 8; ++c) gv[c] = g[c];
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                v[4 * c + 0] = mul_bf16x2(v[4 * c + 0], gv[c].x);
                v[4 * c + 1] = mul_bf16x2(v[4 * c + 1], gv[c].y);
                v[4 * c + 2] = mul_bf16x2(v[4 * c + 2], gv[c].z);
                v[4 * c + 3] = mul_bf16x2(v[4 * c + 3], gv[c].w);
              }
            } else {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                if (c * 8 < kvalid) {
                  const uint4 gv = g[c];
                  v[4 * c + 0] = mul_bf16x2(v[4 * c + 0], gv.x);
                  v[4 * c + 1] = mul_bf16x2(v[4 * c + 1], gv.y);
                  v[4 * c + 2] = mul_bf16x2(v[4 * c + 2], gv.z);
                  v[4 * c + 3] = mul_bf16x2(v[4 * c + 3], gv.w);
                } else {
                  v[4 * c + 0] = v[4 * c + 1] = v[4 * c + 2] = v[4 * c + 3] = 0u;
                }
              }
            }
          }
          if (AMODE == A_SS_FOLD) {
            if (has_gamma) {
#pragma unroll
              for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(a_row + ((c ^ swz) << 4)) =
                    make_uint4(v[4 * c + 0], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
              fence_proxy_async_smem();
            }
          } else {
            __syncwarp();
            tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + Cfg::A_COL0 + s * 32, v);
            tmem_wait_st();
            tc_fence_before();
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_xf(s));
      }
      if (!ok) break;
      // rs[.][acc] was last read by the epilogue of the tile two iterations back
      ok = mbar_wait(bar_tempty(acc), aph ^ 1, ctl, 2, 3 * STAGES + 2 + acc, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      rs[(grp * 2 + acc) * 128 + row] = ss;  // this group's share of the row's sum of squares
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_rs(acc));
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t swz = (uint32_t)(row & 7);
    const int epi_tid = threadIdx.x - (64 + 128 * Cfg::TG);
    bool ok = true;
    int it = 0;
    uint32_t chunk_no = 0;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++it) {
      int mt, nt;
      prefill_tile_coords(t, p, mt, nt);
      const int acc = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      mbar_wait(bar_tfull(acc), aph, ctl, 3, 3 * STAGES + acc, it) &&
          mbar_wait(bar_rs(acc), aph, ctl, 3, 3 * STAGES + 4 + acc, it);
      // The four epilogue warps meet at named barriers below, which have no time
      // limit: they must agree on whether to go on, so one thread decides for all.
      named_bar_sync(3, 128);
      if (epi_tid == 0) *epi_go = ctl->abort ? 0 : 1;
      named_bar_sync(4, 128);
      ok = (*epi_go != 0);
      if (!ok) break;
      tc_fence_after();
      float ssum = 0.f;
#pragma unroll
      for (int g = 0; g < Cfg::TG; ++g) ssum += rs[(g * 2 + acc) * 128 + row];
      const float r = 1.0f / sqrtf(ssum / (float)p.K + p.eps);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c, ++chunk_no) {
        uint8_t* stage = smem + Cfg::OFF_EPI + (chunk_no & 1) * Cfg::EPI_BYTES;
        // the store that last read this staging buffer was issued two chunks ago
        if (epi_tid == 0) tma_store_wait_read<1>();
        named_bar_sync(1, 128);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * 64 + h * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * j + 0]) * r, __uint_as_float(v[8 * j + 1]) * r);
            o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]) * r, __uint_as_float(v[8 * j + 3]) * r);
            o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]) * r, __uint_as_float(v[8 * j + 5]) * r);
            o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]) * r, __uint_as_float(v[8 * j + 7]) * r);
            *reinterpret_cast<uint4*>(stage + row * 128 + (((uint32_t)(h * 4 + j) ^ swz) << 4)) = o;
          }
        }
        if (c == BN / 64 - 1) {
          // accumulator fully read: hand the TMEM buffer (and rs[acc]) back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty(acc));
        }
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        if (epi_tid == 0) {
          const int n0 = nt * BN + c * 64;
          if (n0 < p.N) tma_store_2d(&tm_y, smem_u32(stage), n0, mt * 128);
          tma_store_commit();
        }
      }
    }
    if (epi_tid == 0) tma_store_wait_all<0>();
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (ctl->abort) {
    // a wait ran out: give copies and MMAs still in flight time to land before the CTA's memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace rl
