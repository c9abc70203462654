// Fused RMSNorm -> Linear for M <= 64 tokens (HBM-bound on W).
//
// Operands are swapped so that the 128-wide UMMA M dimension runs over output
// channels: A = W tile [128 channels x 64], B = (x*gamma) tile [MPAD tokens x 64],
// D[channel, token] in TMEM.  Work is counted in (channel-tile, k-block) units and
// every SM pulls the same share of W through a deep TMA ring.  With T channel
// tiles on G CTAs each CTA owns floor(T / G) tiles whole; the k-loops of the
// remaining T mod G tiles are dealt out stream-K style, CTA c taking one contiguous
// run of their units.  A CTA does its share of the split tiles first and its own
// tiles last, so the exchange between CTAs happens early, hidden behind the rest
// of the stream, and the kernel ends on an epilogue that needs nobody else.
// A split tile is finished by the last CTA to arrive: every contributor writes
// its fp32 partial tile and its partial sum of squares to the workspace and bumps
// the tile's counter; whoever sees the final count adds the partials in contributor
// order (so the result does not depend on arrival order), applies 1/rms per token
// and stores y.  No CTA ever waits for another.  Counters are left at zero for
// the next launch.
//
// Warp roles: 0 TMA producer, 1 UMMA issuer, then TW transform warps (sum of squares via
// warp shuffles + gamma fold in shared memory), then 4 epilogue warps.
//
// Ring depth, measured on 28672 x 4096 with 16 tokens: 8 stages stream 2-3 % faster than 12 (less to
// fill and drain per launch), 6 are 1 % slower than 8, 4 are 10 % slower.  A configuration sized for
// two CTAs per SM (6 stages, 2 transform warps, 256 threads), so that the next launch's CTAs could
// set up on the free half while this launch drains, measured the same as with one CTA per SM.
#pragma once
#include "rl_ptx.cuh"

namespace rl {

struct DecodeParams {
  int M, N, K;
  float eps;
  const __nv_bfloat16* gamma;  // [K] or nullptr
  __nv_bfloat16* y;
  long long ldy;
  int n_tiles, KB;
  int sk_tiles;      // tiles [0, sk_tiles) are split along K over all CTAs (stream-K); the rest are owned whole
  int units_total;   // sk_tiles * KB: the units of the split part
  int whole_per_cta; // tiles sk_tiles + cta + i * grid, i < whole_per_cta, belong to CTA `cta`
  int* status;
  int* counters;        // [n_tiles], zero between launches
  float* partials;      // [grid][2][MPAD][128]
  float* ssq_partials;  // [grid][2][MPAD]
  // FP8 configuration: x is the e4m3 activation matrix from rowquant_kernel, W the e4m3 weights
  const float* row_scale;  // [M] rsqrt(mean x^2 + eps) * amax / 448 per token
  const float* w_scale;    // [N] per-output-channel weight scales
};

template <int MPAD_, int STAGES_, int TW_ = 4, int MINB_ = 1, bool FP8_ = false>
struct DecodeCfg {
  static constexpr int MPAD = MPAD_, STAGES = STAGES_;
  // FP8: e4m3 weights and per-token e4m3 activations (quantised beforehand by rowquant_kernel), kind::f8f6f4
  // MMAs; a k-block is 128 elements (the same 128 bytes per tile row), gamma and the row statistics are already
  // inside the activations and their per-token scale, so the transform warps only pass the tiles on, and the
  // epilogue multiplies by row_scale[m] * w_scale[n].  Half the weight bytes of the bf16 kernel per launch.
  static constexpr bool FP8 = FP8_;
  static constexpr int KBW = FP8_ ? 128 : 64;  // elements per k-block
  static constexpr int TW = TW_;      // transform warps; units are dealt to them round-robin
  static constexpr int MINB = MINB_;  // CTAs per SM the kernel is compiled (and sized) for
  static constexpr int THREADS = 64 + 32 * TW + 128;
  static constexpr int W_BYTES = 128 * 64 * 2;
  static constexpr int X_BYTES = MPAD * 64 * 2;
  static constexpr int G_BYTES = 128;
  static constexpr int OFF_W = 0;
  static constexpr int OFF_X = OFF_W + STAGES * W_BYTES;
  static constexpr int OFF_G = OFF_X + STAGES * X_BYTES;
  static constexpr int OFF_SSQ = OFF_G + STAGES * G_BYTES;
  static constexpr int OFF_RVEC = OFF_SSQ + TW * 2 * MPAD * 4;
  static constexpr int OFF_BAR = OFF_RVEC + MPAD * 4;
  static constexpr int NUM_BARS = 3 * STAGES + 6;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;
  static constexpr int TMEM_COLS = (2 * MPAD < 32) ? 32 : 2 * MPAD;
  static constexpr int NCH = MPAD / 4;  // 16-byte chunks of the x tile per lane of the warp that transforms a unit
  static_assert(MPAD == 16 || MPAD == 32 || MPAD == 64, "MPAD");
  static_assert(X_BYTES % 1024 == 0, "x stage alignment");
  // units are dealt to the transform warps round-robin; a ring slot must always belong to the same
  // warp, or a warp that skipped a slot's previous phase could mistake it for its own (parity aliasing)
  static_assert(TW >= 1 && TW <= 4 && STAGES % TW == 0, "STAGES must be a multiple of the transform warps");
  // (the four epilogue warps follow the transform warps: any four consecutive warps cover the four lane quarters of tensor memory)
  static_assert(SMEM_BYTES * MINB + 1024 * MINB <= 233472, "shared memory budget for MINB CTAs per SM");
};

// Balanced contiguous split of `total` units over `G` CTAs.
__host__ __device__ __forceinline__ int sk_begin(int c, int total, int G) {
  const int q = total / G, rem = total % G;
  return c * q + (c < rem ? c : rem);
}
__host__ __device__ __forceinline__ int sk_cta_of_unit(int u, int total, int G) {
  const int q = total / G, rem = total % G;
  const int cut = rem * (q + 1);
  return (u < cut) ? u / (q + 1) : rem + (u - cut) / q;
}

// A CTA's work as a list of segments (a tile's k-range, or part of it).  First its contiguous run of the
// split part's units, cut at channel-tile boundaries and rotated by one - last piece first - so that the
// pieces at both ends of the run (the ones shared with other CTAs) are done early; then the tiles it owns whole.
struct DecodeSegments {
  int u_begin, u_end, KB, first_tile, nseg_sk, nseg, whole0, whole_stride;
  __device__ __forceinline__ DecodeSegments(int b, int e, int kb, int whole_first, int whole_count, int stride)
      : u_begin(b), u_end(e), KB(kb), whole0(whole_first), whole_stride(stride) {
    first_tile = b / kb;
    nseg_sk = (e > b) ? (e - 1) / kb - first_tile + 1 : 0;
    nseg = nseg_sk + whole_count;
  }
  __device__ __forceinline__ int units() const { return (u_end - u_begin) + (nseg - nseg_sk) * KB; }
  // i-th segment in processing order -> natural index within the split run (-1 for an owned tile), channel
  // tile, first k-block, unit count
  __device__ __forceinline__ void get(int i, int& nat, int& tile, int& kb0, int& n_units) const {
    if (i >= nseg_sk) {
      nat = -1;
      tile = whole0 + (i - nseg_sk) * whole_stride;
      kb0 = 0;
      n_units = KB;
      return;
    }
    nat = (nseg_sk >= 2) ? (i == 0 ? nseg_sk - 1 : i - 1) : i;
    tile = first_tile + nat;
    const int s = max(u_begin, tile * KB), e = min(u_end, (tile + 1) * KB);
    kb0 = s - tile * KB;
    n_units = e - s;
  }
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::MINB)
decode_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
              const DecodeParams p) {
  constexpr int MPAD = Cfg::MPAD, STAGES = Cfg::STAGES, NCH = Cfg::NCH, TW = Cfg::TW, KBW = Cfg::KBW;
  constexpr bool FP8 = Cfg::FP8;
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
  volatile int* epi_go = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC + 8);
  volatile int* epi_last = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC + 12);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(smem + Cfg::OFF_MISC + 16);
  float* ssq = reinterpret_cast<float*>(smem + Cfg::OFF_SSQ);    // [TW warps][2][MPAD] partial sums of squares
  float* rvec = reinterpret_cast<float*>(smem + Cfg::OFF_RVEC);  // [MPAD] 1/rms per token of the tile being finished

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.KB;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int u_begin = sk_begin(cta, p.units_total, G);
  const int u_end = sk_begin(cta + 1, p.units_total, G);
  const bool has_gamma = !FP8 && (p.gamma != nullptr);
  const DecodeSegments segs(u_begin, u_end, KB, p.sk_tiles + cta, p.whole_per_cta, G);

  // one unit's loads: W tile (streamed once: evict-first), x tile (re-read by every CTA: evict-last), gamma slice
  auto issue_unit = [&](int s, int tile, int kb, uint64_t pol_w, uint64_t pol_x) {
    const int kvalid = min(64, p.K - kb * 64);
    const uint32_t gbytes = has_gamma ? (uint32_t)kvalid * 2u : 0u;
    mbar_expect_tx(bar_full(s), Cfg::W_BYTES + Cfg::X_BYTES + gbytes);
    tma_load_2d_hint(sbase + Cfg::OFF_W + s * Cfg::W_BYTES, &tm_w, bar_full(s), kb * KBW, tile * 128, pol_w);
    tma_load_2d_hint(sbase + Cfg::OFF_X + s * Cfg::X_BYTES, &tm_x, bar_full(s), kb * KBW, 0, pol_x);
    if (gbytes) bulk_load_1d(sbase + Cfg::OFF_G + s * Cfg::G_BYTES, p.gamma + kb * 64, gbytes, bar_full(s));
  };
  const int n_pre = min(STAGES, segs.units());  // units whose loads go out before the CTA-wide sync

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_xf(s), 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull(a), 1);
      mbar_init(bar_tempty(a), 4);
      mbar_init(bar_rs(a), TW);
    }
    ctl->abort = 0;
    ctl->status = p.status;
    ctl->limit_ns = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
    launch_dependents();
    grid_dependency_wait();
    // fill the ring right away: the first loads need neither tensor memory nor the other warps
    const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
    int issued = 0;
    for (int i = 0; i < segs.nseg && issued < n_pre; ++i) {
      int nat, tile, kb0, n_units;
      segs.get(i, nat, tile, kb0, n_units);
      for (int k = 0; k < n_units && issued < n_pre; ++k, ++issued) issue_unit(issued, tile, kb0 + k, pol_w, pol_x);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  grid_dependency_wait();  // every thread: nothing below may touch global memory before the previous grid is done
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (units after the pre-filled ones)
    {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      int s = (n_pre == STAGES) ? 0 : n_pre;
      uint32_t ph = (n_pre == STAGES) ? 1u : 0u;
      int j = 0;
      bool ok = true;
      for (int i = 0; ok && i < segs.nseg; ++i) {
        int nat, tile, kb0, n_units;
        segs.get(i, nat, tile, kb0, n_units);
        for (int k = 0; k < n_units; ++k, ++j) {
          if (j < n_pre) continue;  // went out before the CTA-wide sync
          if (!mbar_wait_warp(bar_empty(s), ph ^ 1, ctl, 0, 2 * STAGES + s, j)) { ok = false; break; }
          if (elect_one()) issue_unit(s, tile, kb0 + k, pol_w, pol_x);
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    {
      constexpr uint32_t idesc = FP8 ? make_idesc(128, MPAD, 0, 0) : make_idesc(128, MPAD, 1, 1);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int u = 0;  // running unit count (for error records only)
      for (int seg = 0; ok && seg < segs.nseg; ++seg) {
        int nat, tile, kb0, n_units;
        segs.get(seg, nat, tile, kb0, n_units);
        const int acc = seg & 1;
        const uint32_t aph = (seg >> 1) & 1;
        if (!mbar_wait_warp(bar_tempty(acc), aph ^ 1, ctl, 1, 3 * STAGES + 2 + acc, seg)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * MPAD;
        for (int i = 0; i < n_units; ++i) {
          if (!mbar_wait_warp(bar_full(s), ph, ctl, 1, s, u + i)) { ok = false; break; }
          if (!mbar_wait_warp(bar_xf(s), ph, ctl, 1, STAGES + s, u + i)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_sw128_kmajor_desc(sbase + Cfg::OFF_W + s * Cfg::W_BYTES);
          const uint64_t bdesc = make_sw128_kmajor_desc(sbase + Cfg::OFF_X + s * Cfg::X_BYTES);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (FP8) umma_f8_ss(d, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0);
              else umma_ss(d, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0);
            }
            umma_commit(bar_empty(s));
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok && elect_one()) umma_commit(bar_tfull(acc));
        __syncwarp();
        u += n_units;
      }
    }
  } else if (warp < 2 + TW) {
    // ------------------------------------------------------------ transform
    // The x tile of one unit is small (MPAD x 128 bytes), so one warp handles a whole unit and
    // the TW warps take units round-robin: TW units are in flight in this role at once.
    const int tw = warp - 2;     // 0..TW-1
    const int c = lane & 7;      // 16-byte chunk within the 128-byte row
    bool ok = true;
    int u = 0;  // running unit count of the CTA = ring position of the segment's first unit
    for (int seg = 0; ok && seg < segs.nseg; ++seg) {
      int nat, tile, kb0, n_units;
      segs.get(seg, nat, tile, kb0, n_units);
      const int acc = seg & 1;
      const uint32_t aph = (seg >> 1) & 1;
      float ss[NCH];
#pragma unroll
      for (int i = 0; i < NCH; ++i) ss[i] = 0.f;
      const int j0 = u;
      for (int i = ((tw - j0) % TW + TW) % TW; i < n_units; i += TW) {
        const int j = j0 + i;
        const int s = j % STAGES;
        const uint32_t ph = (uint32_t)(j / STAGES) & 1u;
        ok = mbar_wait(bar_full(s), ph, ctl, 2, s, u + i);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (FP8) {  // nothing to fold and nothing to sum: hand the tile on
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_xf(s));
          continue;
        }
        uint8_t* xt = smem + Cfg::OFF_X + s * Cfg::X_BYTES;
        const int kvalid = p.K - (kb0 + i) * 64;
        uint4 gv = make_uint4(0, 0, 0, 0);
        const bool cvalid = (c * 8 < kvalid);
        if (has_gamma && cvalid) gv = reinterpret_cast<const uint4*>(smem + Cfg::OFF_G + s * Cfg::G_BYTES)[c];
#pragma unroll
        for (int jj = 0; jj < NCH; ++jj) {
          const int row = (lane >> 3) + jj * 4;
          uint4* ptr = reinterpret_cast<uint4*>(xt + row * 128 + ((c ^ (row & 7)) << 4));
          uint4 v = *ptr;
          float a = ss[jj];
          a = fmaf(bf16lo(v.x), bf16lo(v.x), a); a = fmaf(bf16hi(v.x), bf16hi(v.x), a);
          a = fmaf(bf16lo(v.y), bf16lo(v.y), a); a = fmaf(bf16hi(v.y), bf16hi(v.y), a);
          a = fmaf(bf16lo(v.z), bf16lo(v.z), a); a = fmaf(bf16hi(v.z), bf16hi(v.z), a);
          a = fmaf(bf16lo(v.w), bf16lo(v.w), a); a = fmaf(bf16hi(v.w), bf16hi(v.w), a);
          ss[jj] = a;
          if (has_gamma) {
            if (cvalid) {
              v.x = mul_bf16x2(v.x, gv.x); v.y = mul_bf16x2(v.y, gv.y);
              v.z = mul_bf16x2(v.z, gv.z); v.w = mul_bf16x2(v.w, gv.w);
            } else {
              v = make_uint4(0, 0, 0, 0);
            }
            *ptr = v;
          }
        }
        if (has_gamma) fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_xf(s));
      }
      if (!ok) break;
      // each token row is spread over 8 neighbouring lanes: butterfly-reduce
#pragma unroll
      for (int jj = 0; jj < NCH; ++jj) {
        float a = ss[jj];
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        a += __shfl_xor_sync(0xffffffffu, a, 4);
        ss[jj] = a;
      }
      ok = mbar_wait(bar_tempty(acc), aph ^ 1, ctl, 2, 3 * STAGES + 2 + acc, seg);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (c == 0) {
#pragma unroll
        for (int jj = 0; jj < NCH; ++jj) ssq[(tw * 2 + acc) * MPAD + (lane >> 3) + jj * 4] = ss[jj];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_rs(acc));
      u += n_units;
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    const int epi_tid = threadIdx.x - (64 + 32 * TW);
    const float inv_k = 1.0f / (float)p.K;
    for (int seg = 0; seg < segs.nseg; ++seg) {
      int nat, tile, kb0, n_units;
      segs.get(seg, nat, tile, kb0, n_units);
      const int acc = seg & 1;
      const uint32_t aph = (seg >> 1) & 1;
      mbar_wait(bar_tfull(acc), aph, ctl, 3, 3 * STAGES + acc, seg) &&
          mbar_wait(bar_rs(acc), aph, ctl, 3, 3 * STAGES + 4 + acc, seg);
      // named barriers have no time limit: one thread decides for the whole group
      named_bar_sync(3, 128);
      if (epi_tid == 0) *epi_go = ctl->abort ? 0 : 1;
      named_bar_sync(4, 128);
      if (*epi_go == 0) break;
      tc_fence_after();

      float a[MPAD];
#pragma unroll
      for (int h = 0; h < MPAD / 16; ++h) {
        uint32_t v[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + acc * MPAD + h * 16, v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) a[h * 16 + j] = __uint_as_float(v[j]);
      }
      const int n = tile * 128 + n_local;
      const bool whole = (n_units == KB);
      [[maybe_unused]] float wsn = 1.0f;  // FP8: this thread's channel scale
      if (FP8) wsn = (n < p.N) ? __ldg(p.w_scale + n) : 0.f;
      // one thread per token adds up the transform warps' shares of the sum of squares
      float tot = 0.f;
      if (epi_tid < MPAD) {
#pragma unroll
        for (int w = 0; w < TW; ++w) tot += ssq[(w * 2 + acc) * MPAD + epi_tid];
      }
      bool finish = whole;
      if (whole) {
        if (epi_tid < MPAD)
          rvec[epi_tid] = FP8 ? ((epi_tid < p.M) ? __ldg(p.row_scale + epi_tid) : 0.f) : 1.0f / sqrtf(tot * inv_k + p.eps);
        named_bar_sync(1, 128);
      } else {
        const int slot = (nat == 0) ? 0 : 1;  // slot 0: the tile this CTA's run starts in
        float* part = p.partials + (size_t)(cta * 2 + slot) * MPAD * 128;
#pragma unroll
        for (int m = 0; m < MPAD; ++m) part[m * 128 + n_local] = a[m];
        if (!FP8 && epi_tid < MPAD) p.ssq_partials[(cta * 2 + slot) * MPAD + epi_tid] = tot;
        __threadfence();
        named_bar_sync(1, 128);
        const int first = sk_cta_of_unit(tile * KB, p.units_total, G);
        const int last = sk_cta_of_unit(tile * KB + KB - 1, p.units_total, G);
        if (epi_tid == 0) {
          const int old = atomicAdd(p.counters + tile, 1);
          const int is_last = (old == last - first);
          if (is_last) p.counters[tile] = 0;  // ready for the next launch
          *epi_last = is_last;
          __threadfence();
        }
        named_bar_sync(2, 128);
        finish = (*epi_last != 0);
        if (finish) {
          // last to arrive: add the contributors' partial tiles in contributor order
#pragma unroll
          for (int m = 0; m < MPAD; ++m) a[m] = 0.f;
          float s2 = 0.f;
          for (int cc = first; cc <= last; ++cc) {
            const int cslot = (sk_begin(cc, p.units_total, G) / KB == tile) ? 0 : 1;
            const float* cpart = p.partials + (size_t)(cc * 2 + cslot) * MPAD * 128;
            float ld[MPAD];
#pragma unroll
            for (int m = 0; m < MPAD; ++m) ld[m] = __ldcg(cpart + m * 128 + n_local);
            if (!FP8 && epi_tid < MPAD) s2 += __ldcg(p.ssq_partials + (cc * 2 + cslot) * MPAD + epi_tid);
#pragma unroll
            for (int m = 0; m < MPAD; ++m) a[m] += ld[m];
          }
          if (epi_tid < MPAD)
            rvec[epi_tid] = FP8 ? ((epi_tid < p.M) ? __ldg(p.row_scale + epi_tid) : 0.f) : 1.0f / sqrtf(s2 * inv_k + p.eps);
          named_bar_sync(5, 128);
        }
      }
      if (finish) {
        if (n < p.N) {
#pragma unroll
          for (int m = 0; m < MPAD; ++m)
            if (m < p.M) p.y[(size_t)m * p.ldy + n] = __float2bfloat16_rn(FP8 ? a[m] * rvec[m] * wsn : a[m] * rvec[m]);
        }
      }
      // accumulator and ssq[acc] fully consumed
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty(acc));
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (ctl->abort) {
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
