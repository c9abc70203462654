// Fused RMSNorm -> Linear for large M on CTA pairs (cluster of 2, tcgen05 cta_group::2).
//
// A pair of CTAs on neighbouring SMs computes one 256 x BN output tile.  Each CTA loads only
// its own halves - x rows [128 x 64] and W rows [BN/2 x 64] per k-block, no multicast - and
// the pair's MMA (M = 256, N = BN, issued by one lane of the rank-0 CTA) reads both W halves
// from the two CTAs' shared memory, so every byte brought in from L2 feeds twice the math of
// a single-CTA tile.  (Elements per k-block: 64 bf16, or 128 e4m3 in the FP8 configuration -
// 128 bytes per tile row either way.)
//
// A_TS_FOLD: the gamma-folded activation tile is the MMA's A operand in tensor memory.  The
//   transform warps read the landed x tile from shared memory, multiply by gamma (and, without
//   the row-statistics pre-pass, accumulate each row's sum of squares) and tcgen05.st the
//   result into a ring of ASLOTS A slots that sits behind the accumulators.
// A_SS_DIRECT (gamma == nullptr - the reference operator -, gamma already folded into a copy of x by the
//   pre-pass, the plain GEMM, LoRA, FP8): the MMA reads x straight from shared memory.  With 1/rms from the pre-pass (PRESTATS) there is no
//   transform stage at all: TG = 0, the CTA is producer + MMA issuer + four epilogue warps, and the
//   x tile completes on the same barrier as the W tile.  Without the pre-pass the transform warps
//   accumulate the sums of squares.
// TMEM per CTA: NACC accumulators of BN columns, then ASLOTS x 32 columns of A ring.
//
// Barriers (shared memory, identical offsets in both CTAs):
//   fullA[s]    local        x tile + gamma slice landed              producer -> own transform warps
//   ready[s]    rank 0 only  both W halves landed (2 arrivals + tx) and both CTAs' transform warps
//                            done with slot s (8 arrivals): the one wait per k-block of the MMA loop
//                            (no transform stage: 2 arrivals + the tx of both x and both W halves)
//   empty[s]    local        MMAs that read slot s are done            MMA commit (multicast) -> producers,
//                                                                      and -> transform warps (A slot reuse)
//   tfull[a]    local        accumulator a complete                    MMA commit (multicast) -> epilogues
//   tempty[a]   rank 0 only  both epilogues drained accumulator a (8 arrivals) -> MMA warp
//   rsfull[a]   local        row sums of squares written               transform -> own epilogue
//   rsfree[a]   local        row sums consumed                         epilogue -> own transform warps
#pragma once
#include "rl_prefill.cuh"

namespace rl {

template <int BN_, int NACC_, int STAGES_, int ASLOTS_, int TG_, int AMODE_, bool PRESTATS_ = false, bool SWIGLU_ = false,
          bool FP8_ = false>
struct PairCfg {
  static constexpr int BN = BN_, NACC = NACC_, STAGES = STAGES_, ASLOTS = ASLOTS_, TG = TG_, AMODE = AMODE_;
  // PRESTATS: 1/rms per token comes from rowstats_kernel; the transform warps only fold gamma
  static constexpr bool PRESTATS = PRESTATS_;
  // SWIGLU: W is [2 n, K] = gate rows then up rows (python/baselines/rmsnorm_swiglu.py:36-42).  The rank-0 CTA
  // loads gate channels, the rank-1 CTA the matching up channels, so accumulator columns [0,128) and
  // [128,256) hold gate and up of the same 128 output channels and the epilogue emits silu(gate) * up.
  static constexpr bool SWIGLU = SWIGLU_;
  // (BN = 512: the tile's first 256 accumulator columns are gate, the second 256 up, of the same 256 output channels)
  static_assert(!SWIGLU_ || BN_ == 256 || BN_ == 512, "SwiGLU epilogue: gate and up halves of 128 or 256 columns");
  // FP8: both operands are e4m3 (activations quantised per token by rowquant_kernel, weights with per-channel
  // scales), k-blocks of 128 elements (the same 128 bytes per tile row), kind::f8f6f4 MMAs, and the epilogue
  // multiplies by row_scale[m] * w_scale[n].
  static constexpr bool FP8 = FP8_;
  static constexpr int KBW = FP8_ ? 128 : 64;  // elements per k-block
  // WIDE (BN = 512): one tile is two MMA-wide column halves that share the activation tile - every x byte brought
  // in from L2 feeds twice the math (the measured upper bound of that saving at the power cap: +7 to +9 %).  The
  // tile's accumulator is all of tensor memory, so the drain of one tile cannot run under the main loop of the next
  // as with two 256-column accumulators; the two halves are released separately instead (the barriers that count
  // accumulators count halves here), and the next tile's first k-block starts on the first half while the second
  // is still draining.  Each CTA's W stage is two boxes of 128 rows, one per half.
  static constexpr bool WIDE = (BN_ == 512);
  static constexpr int MMA_N = WIDE ? 256 : BN_;
  static_assert(!WIDE || (NACC_ == 2 && AMODE_ == A_SS_DIRECT && PRESTATS_ && !FP8_),
                "512-column tiles: transform-free bf16, two separately released halves");
  // XFORM: the kernel has transform warps (they fold gamma and / or accumulate the sums of squares).  Without
  // them (x straight from shared memory, 1/rms from the pre-pass) both operand tiles complete directly on the
  // barrier the MMA warp waits on and the CTA is producer + MMA + epilogue only.
  static constexpr bool XFORM = (AMODE_ == A_TS_FOLD) || !PRESTATS_;
  static_assert(XFORM ? (TG_ > 0) : (TG_ == 0), "transform groups exactly where there is transform work");
  static_assert(!FP8_ || (!XFORM && !SWIGLU_ && BN_ == 256), "FP8: operands straight from shared memory");
  static constexpr int THREADS = 64 + 128 * TG + 128;
  static constexpr int A_BYTES = 128 * 64 * 2;
  static constexpr int B_BYTES = (BN / 2) * 64 * 2;  // this CTA's half of the W tile
  static constexpr int G_BYTES = 128;
  static constexpr int EPI_BYTES = 128 * 64 * 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_EPI = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_G = OFF_EPI + 2 * EPI_BYTES;
  static constexpr int OFF_RS = OFF_G + (AMODE_ == A_TS_FOLD ? STAGES * G_BYTES : 0);
  static constexpr int OFF_WS = OFF_RS + (PRESTATS_ ? 0 : TG * NACC * 128 * 4);  // FP8: [2][256] w_scale of the tiles being drained
  static constexpr int OFF_BAR = OFF_WS + (FP8_ ? 2 * 256 * 4 : 0);
  static constexpr int NUM_BARS = 3 * STAGES + 4 * NACC;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 64;  // no alignment slack: the kernel checks the base instead
  static constexpr int TMEM_COLS = 512;
  static constexpr int ACC_COLS = WIDE ? BN : NACC * BN;
  static constexpr int A_COL0 = ACC_COLS;
  static_assert(AMODE == A_TS_FOLD || AMODE == A_SS_DIRECT, "pair kernel: TS fold or SS direct");
  static_assert(BN % 64 == 0 && (BN <= 256 || BN == 512), "BN");
  static_assert(B_BYTES % 1024 == 0, "W stage alignment");
  static_assert(NACC == 1 || NACC == 2, "NACC");
  // a ring slot is always served by the same transform group (parity waits alias otherwise), and a
  // group that waits for the MMA which last read its A slot must itself be the one feeding that MMA
  static_assert(TG == 0 || (STAGES % (TG ? TG : 1) == 0 && (AMODE != A_TS_FOLD || (STAGES - ASLOTS) % (TG ? TG : 1) == 0)),
                "ring / group layout");
  static_assert(AMODE != A_TS_FOLD || (ASLOTS <= STAGES && NACC * BN + 32 * ASLOTS <= 512), "TMEM budget");
  static_assert(ACC_COLS <= 512, "TMEM budget");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// One work item of a CTA pair: a whole tile (slice < 0, k-blocks [0, KB)), or one k-slice of a tail tile.
//
// Tiles are dealt round-robin, tile t to pair t % n_pairs.  The main loop runs at the same ~650 cycles per
// k-block whatever the tile's width (measured: 256 x 64 strips gained nothing), so the way to spread the tiles
// of a partly filled last round over the idle pairs is along K: with tail_split = S each
// of the last `tail_tiles` tiles is cut into S k-slices that S different pairs compute at the same time (pair
// u takes slice u % S of tail tile u / S); the S partial accumulators meet in the epilogue.
struct PairItem {
  int t, kb0, kb1, slice;
};
template <bool TAIL>
__device__ __forceinline__ bool pair_item(const PrefillParams& p, int pair, int n_pairs, int total_tiles, int KB, int i,
                                          PairItem& w) {
  w.t = pair + i * n_pairs;
  w.kb0 = 0;
  w.kb1 = KB;
  w.slice = -1;
  if (!TAIL || p.tail_split <= 1) return w.t < total_tiles;
  const int t_main = total_tiles - p.tail_tiles;  // a multiple of n_pairs (or 0)
  if (w.t < t_main) return true;
  const int u = w.t - t_main;
  if (u >= p.tail_tiles * p.tail_split) return false;
  const int S = p.tail_split;
  w.t = t_main + u / S;
  w.slice = u % S;
  w.kb0 = (int)(((long long)w.slice * KB) / S);
  w.kb1 = (int)(((long long)(w.slice + 1) * KB) / S);
  return true;
}

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::THREADS, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                    const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_x2,
                    const __grid_constant__ CUtensorMap tm_w2, const PrefillParams p) {
  constexpr int BN = Cfg::BN, NACC = Cfg::NACC, STAGES = Cfg::STAGES, ASLOTS = Cfg::ASLOTS, TG = Cfg::TG;
  constexpr bool TS = (Cfg::AMODE == A_TS_FOLD);
  constexpr bool PRESTATS = Cfg::PRESTATS;
  constexpr bool SWIGLU = Cfg::SWIGLU;
  constexpr bool FP8 = Cfg::FP8, XFORM = Cfg::XFORM, WIDE = Cfg::WIDE;
  constexpr int KBW = Cfg::KBW;
  // k-split tail tiles: 1/rms must come from outside (a slice sees only part of a row) and the epilogue is plain
  constexpr bool TAIL = PRESTATS && !SWIGLU && (BN == 256 || BN == 512);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  if (sbase & 1023u) {
    // swizzled tiles need a 1024-byte aligned base; every thread of both CTAs sees the same value
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, (int)DEV_BAD_SMEM_ALIGNMENT);
    return;
  }
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  auto bar_fullA = [&](int s) { return bar0 + 8u * s; };
  auto bar_ready = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto bar_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
  auto bar_tfull = [&](int a) { return bar0 + 8u * (3 * STAGES + a); };
  auto bar_tempty = [&](int a) { return bar0 + 8u * (3 * STAGES + NACC + a); };
  auto bar_rsfull = [&](int a) { return bar0 + 8u * (3 * STAGES + 2 * NACC + a); };
  auto bar_rsfree = [&](int a) { return bar0 + 8u * (3 * STAGES + 3 * NACC + a); };
  const uint32_t bar_tail = sbase + Cfg::OFF_MISC + 48u;  // partial blocks of a k-split tile landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_MISC);
  volatile int* epi_go = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC + 8);
  CtaCtl* ctl = reinterpret_cast<CtaCtl*>(smem + Cfg::OFF_MISC + 16);
  float* rs = reinterpret_cast<float*>(smem + Cfg::OFF_RS);  // [TG][NACC][128] partial sums of squares
  [[maybe_unused]] float* wsc = reinterpret_cast<float*>(smem + Cfg::OFF_WS);  // FP8: [2][256] per-channel scales

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 issues the MMAs
  const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
  // p.extra_kb k-blocks are appended to every tile's k-loop with their operands taken from a second pair of
  // matrices (tm_x2 [M, L], tm_w2 [N, L], columns beyond L zero-filled by TMA): y = x W^T + x2 W2^T, the low-rank
  // update of a LoRA layer riding in the same accumulator.  Only the producer knows the difference.
  const int KB_main = (p.K + KBW - 1) / KBW;
  const int KB = KB_main + p.extra_kb;
  const int total_tiles = p.m_tiles * p.n_tiles;  // 256 x BN tiles
  const bool has_gamma = (p.gamma != nullptr);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_fullA(s), 1);
      mbar_init(bar_ready(s), XFORM ? 2 + 8 : 2);
      mbar_init(bar_empty(s), 1);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(bar_tfull(a), 1);
      mbar_init(bar_tempty(a), 8);
      mbar_init(bar_rsfull(a), XFORM ? 4 * TG : 1);
      mbar_init(bar_rsfree(a), 4);
    }
    mbar_init(bar_tail, 1);
    ctl->abort = 0;
    ctl->status = p.status;
    ctl->limit_ns = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_x);
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_y);
    if (p.extra_kb) {
      prefetch_tmap(&tm_x2);
      prefetch_tmap(&tm_w2);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, own halves)
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    const uint32_t lead_ready0 = mapa_shared(bar_ready(0), 0);
    PairItem w;
    // FP8, or gamma folded by the pre-pass: the activations are written by the kernel launched just before this one
    if (FP8 || p.x_from_prepass) grid_dependency_wait();
    for (int i = 0; ok && pair_item<TAIL>(p, pair, n_pairs, total_tiles, KB, i, w); ++i) {
      int mt, nt;
      prefill_tile_coords(w.t, p, mt, nt);
      if (p.round_words != nullptr && rank == 0 && i >= 1 && w.slice < 0) {
        // Best-effort alignment.  Pairs that share an operand panel fetch each k-block of it from DRAM once only while
        // they walk it together; left alone they drift apart over a long sweep (16384 x 28672 x 8192: 11.6 GB read,
        // 5.8 GB with this).  Say that this pair starts its i-th tile, then give the others a moment to get there;
        // whoever is not there by then is not waited for.
        const unsigned want = (p.round_epoch << 12) | (unsigned)i;
        if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.round_words + pair), "r"(want) : "memory");
        const uint64_t t0 = global_timer_ns();
        while (true) {
          bool mine = true;
          for (int j = lane; j < n_pairs; j += 32) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.round_words + j) : "memory");
            mine = mine && ((v >> 12) == p.round_epoch) && ((v & 0xfffu) >= (unsigned)i);
          }
          if (__all_sync(0xffffffffu, mine)) break;
          if (__any_sync(0xffffffffu, global_timer_ns() - t0 > (uint64_t)p.round_wait_ns)) break;
          __nanosleep(100);
        }
      }
      for (int kb = w.kb0; kb < w.kb1; ++kb) {
        if (!mbar_wait_warp(bar_empty(s), ph ^ 1, ctl, 0, 2 * STAGES + s, kb)) { ok = false; break; }
        if (elect_one()) {
          const bool extra = (kb >= KB_main);
          const int kcol = extra ? (kb - KB_main) * KBW : kb * KBW;
          const uint32_t lead_ready = lead_ready0 + 8u * s;
          if (XFORM) {
            const int kvalid = min(64, p.K - kb * 64);
            const uint32_t gbytes = (TS && has_gamma && !extra) ? (uint32_t)kvalid * 2u : 0u;
            mbar_expect_tx(bar_fullA(s), Cfg::A_BYTES + gbytes);
            tma_load_2d(sbase + Cfg::OFF_A + s * Cfg::A_BYTES, extra ? &tm_x2 : &tm_x, bar_fullA(s), kcol,
                        mt * 256 + (int)rank * 128);
            if (gbytes) bulk_load_1d(sbase + Cfg::OFF_G + s * Cfg::G_BYTES, p.gamma + kb * 64, gbytes, bar_fullA(s));
            mbar_expect_tx_cluster(lead_ready, Cfg::B_BYTES);
          } else {
            // no transform stage: the x tile is counted on the MMA warp's barrier as well
            mbar_expect_tx_cluster(lead_ready, Cfg::A_BYTES + Cfg::B_BYTES);
            tma_load_2d_pair(sbase + Cfg::OFF_A + s * Cfg::A_BYTES, extra ? &tm_x2 : &tm_x, lead_ready, kcol,
                             mt * 256 + (int)rank * 128);
          }
          if (WIDE) {
            // two boxes of 128 weight rows: this CTA's share of the tile's first and second 256 columns
            // (SwiGLU: the first half is this CTA's 128 gate channels of the tile's 256, the second the matching up channels)
            tma_load_2d_pair(sbase + Cfg::OFF_B + s * Cfg::B_BYTES, &tm_w, lead_ready, kcol,
                             SWIGLU ? nt * 256 + (int)rank * 128 : nt * BN + (int)rank * 128);
            tma_load_2d_pair(sbase + Cfg::OFF_B + s * Cfg::B_BYTES + Cfg::B_BYTES / 2, &tm_w, lead_ready, kcol,
                             SWIGLU ? p.N + nt * 256 + (int)rank * 128 : nt * BN + 256 + (int)rank * 128);
          } else {
            tma_load_2d_pair(sbase + Cfg::OFF_B + s * Cfg::B_BYTES, extra ? &tm_w2 : &tm_w, lead_ready, kcol,
                             SWIGLU ? (int)rank * p.N + nt * 128 : nt * BN + (int)rank * (BN / 2));
          }
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
    if (p.round_words != nullptr && rank == 0 && lane == 0)
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.round_words + pair), "r"((p.round_epoch << 12) | 0xfffu) : "memory");
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer (rank 0 only)
    if (rank == 0) {
      constexpr uint32_t idesc = FP8 ? make_idesc(256, Cfg::MMA_N, 0, 0) : make_idesc(256, Cfg::MMA_N, 1, 1);
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      const uint64_t bdesc0 = make_sw128_kmajor_desc(sbase + Cfg::OFF_B);
      const uint64_t adesc0 = make_sw128_kmajor_desc(sbase + Cfg::OFF_A);
      int s = 0, aslot = 0;
      uint32_t ph = 0;
      bool ok = true;
      PairItem w;
      for (int it = 0; ok && pair_item<TAIL>(p, pair, n_pairs, total_tiles, KB, it, w); ++it) {
        // (WIDE: every tile uses both column halves, barrier set 0 for the first and 1 for the second)
        const int acc = WIDE ? 0 : ((NACC == 2) ? (it & 1) : 0);
        const uint32_t aph = (NACC == 2 && !WIDE) ? ((it >> 1) & 1) : (it & 1);
        if (!mbar_wait_warp(bar_tempty(acc), aph ^ 1u, ctl, 1, 3 * STAGES + NACC + acc, it)) break;
        const uint32_t d = tmem_base + acc * BN;
        // The issue loop sets the tensor cores' pace: one barrier wait per k-block, the poll for the
        // next slot started before this slot's MMAs are issued, and one predicated issue block.
        uint32_t ready_now = mbar_test_wait(bar_ready(s), ph);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!ready_now) {
            if (!mbar_wait(bar_ready(s), ph, ctl, 1, STAGES + s, kb)) { ok = false; break; }
          }
          tc_fence_after();
          const int sn = (s + 1 == STAGES) ? 0 : s + 1;
          const uint32_t phn = (s + 1 == STAGES) ? (ph ^ 1u) : ph;
          ready_now = mbar_test_wait(bar_ready(sn), phn);  // next k-block (or the next tile's first)
          if (TS) {
            umma_kblock_ts_pair(d, tmem_base + Cfg::A_COL0 + aslot * 32, bdesc0 + (uint64_t)(s * (Cfg::B_BYTES >> 4)),
                                idesc, (uint32_t)(kb != w.kb0), bar_empty(s), leader);
          } else if (FP8) {
            umma_kblock_f8_ss_pair(d, adesc0 + (uint64_t)(s * (Cfg::A_BYTES >> 4)),
                                   bdesc0 + (uint64_t)(s * (Cfg::B_BYTES >> 4)), idesc, (uint32_t)(kb != w.kb0),
                                   bar_empty(s), leader);
          } else if (WIDE) {
            const uint64_t ad = adesc0 + (uint64_t)(s * (Cfg::A_BYTES >> 4));
            const uint64_t bd = bdesc0 + (uint64_t)(s * (Cfg::B_BYTES >> 4));
            umma_kblock_ss_pair_nocommit(d, ad, bd, idesc, (uint32_t)(kb != w.kb0), leader);
            if (kb == w.kb0) {
              // the second half may still be draining the tile before: its MMAs wait for that, the first half's
              // are already running
              if (!mbar_wait_warp(bar_tempty(1), aph ^ 1u, ctl, 1, 3 * STAGES + NACC + 1, it)) { ok = false; break; }
              tc_fence_after();
            }
            umma_kblock_ss_pair_nocommit(d + 256, ad, bd + (uint64_t)((Cfg::B_BYTES / 2) >> 4), idesc,
                                         (uint32_t)(kb != w.kb0), leader);
            umma_commit_pair_pred(bar_empty(s), leader);
          } else {
            umma_kblock_ss_pair(d, adesc0 + (uint64_t)(s * (Cfg::A_BYTES >> 4)),
                                bdesc0 + (uint64_t)(s * (Cfg::B_BYTES >> 4)), idesc, (uint32_t)(kb != w.kb0), bar_empty(s),
                                leader);
          }
          s = sn;
          ph = phn;
          if (++aslot == ASLOTS) aslot = 0;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) umma_commit_pair_pred(bar_tfull(acc), leader);
      }
    }
    __syncwarp();
  } else if (XFORM && warp < 2 + 4 * TG) {
    // ------------------------------------------------------------ transform (both CTAs)
    constexpr int TGd = TG ? TG : 1;  // (TG == 0 only in configurations without this role)
    const int grp = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t swz = (uint32_t)(row & 7);
    const uint32_t lead_ready0 = mapa_shared(bar_ready(0), 0);
    bool ok = true;
    int j_base = 0;  // k-blocks this pair has been through: ring slot and phase follow from it
    PairItem w;
    for (int it = 0; ok && pair_item<TAIL>(p, pair, n_pairs, total_tiles, KB, it, w); ++it, j_base += w.kb1 - w.kb0) {
      const int acc = (NACC == 2) ? (it & 1) : 0;
      const uint32_t aph = (NACC == 2) ? ((it >> 1) & 1) : (it & 1);
      float2 ss2 = make_float2(0.f, 0.f);
      for (int kb = w.kb0 + (grp - j_base % TGd + TGd) % TGd; kb < w.kb1; kb += TGd) {
        const int j = j_base + kb - w.kb0;
        const int s = j % STAGES;
        const uint32_t ph = (uint32_t)(j / STAGES) & 1u;
        ok = mbar_wait(bar_fullA(s), ph, ctl, 2, s, kb);
        if (TS && ASLOTS < STAGES && j >= ASLOTS) {
          // the MMA that last read this A slot (k-block j - ASLOTS) must be done
          const int jo = j - ASLOTS;
          ok = ok && mbar_wait(bar_empty(jo % STAGES), (uint32_t)(jo / STAGES) & 1u, ctl, 2, 2 * STAGES + jo % STAGES, kb);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint8_t* a_row = smem + Cfg::OFF_A + s * Cfg::A_BYTES + row * 128;
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 u = *reinterpret_cast<const uint4*>(a_row + ((c ^ swz) << 4));
          v[4 * c + 0] = u.x; v[4 * c + 1] = u.y; v[4 * c + 2] = u.z; v[4 * c + 3] = u.w;
        }
        if (!PRESTATS) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) ffma2_sq(ss2, bf16lo(v[jj]), bf16hi(v[jj]));
        }
        if (TS) {
          if (has_gamma) {
            const uint4* g = reinterpret_cast<const uint4*>(smem + Cfg::OFF_G + s * Cfg::G_BYTES);
            const int kvalid = p.K - kb * 64;
            if (kvalid >= 64) {
              // whole k-block: the eight gamma loads issued back to back with no branch between them (a branch
              // per load left each load's latency exposed: 640 cycles per k-block instead of about 100)
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
              // last, partial k-block (K not a multiple of 64): the gamma slice ends at K; x beyond K is zero-filled
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
          __syncwarp();
          tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + Cfg::A_COL0 + (j % ASLOTS) * 32, v);
          tmem_wait_st();
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_ready0 + 8u * s);
      }
      if (!ok) break;
      if (!PRESTATS) {
        ok = mbar_wait(bar_rsfree(acc), aph ^ 1u, ctl, 2, 3 * STAGES + 3 * NACC + acc, it);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        rs[(grp * NACC + acc) * 128 + row] = ss2.x + ss2.y;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rsfull(acc));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t swz = (uint32_t)(row & 7);
    const int epi_tid = threadIdx.x - (64 + 128 * TG);
    const uint32_t lead_tempty0 = mapa_shared(bar_tempty(0), 0);
    const uint64_t pol_y = l2_policy_evict_first();
    bool ok = true;
    uint32_t chunk_no = 0;
    PairItem w;
    for (int it = 0; ok && pair_item<TAIL>(p, pair, n_pairs, total_tiles, KB, it, w); ++it) {
      int mt, nt;
      prefill_tile_coords(w.t, p, mt, nt);
      const int acc = WIDE ? 0 : ((NACC == 2) ? (it & 1) : 0);
      const uint32_t aph = (NACC == 2 && !WIDE) ? ((it >> 1) & 1) : (it & 1);
      [[maybe_unused]] const float* wc_tile = wsc + (it & 1) * 256;
      if (FP8) {
        // stage this tile's 256 per-channel scales while the accumulator is still filling; the buffer of the
        // tile before last is free: every epilogue thread has passed this iteration's predecessor's barriers
        const int n = nt * BN + epi_tid;
        wsc[(it & 1) * 256 + epi_tid] = (n < p.N) ? __ldg(p.w_scale + n) : 0.f;
        wsc[(it & 1) * 256 + 128 + epi_tid] = (n + 128 < p.N) ? __ldg(p.w_scale + n + 128) : 0.f;
      }
      float r_pre = 0.f;
      if (PRESTATS) {
        // launched with programmatic stream serialisation right behind rowstats_kernel: everything up to
        // here overlapped it; its results are needed (and guaranteed visible) only from this point on
        grid_dependency_wait();
        const int m = mt * 256 + (int)rank * 128 + row;
        r_pre = (p.row_rstd == nullptr) ? 1.0f : ((m < p.M) ? __ldg(p.row_rstd + m) : 0.f);
      }
      mbar_wait_long(bar_tfull(acc), aph, ctl, 3, 3 * STAGES + acc, it) &&
          (PRESTATS || mbar_wait(bar_rsfull(acc), aph, ctl, 3, 3 * STAGES + 2 * NACC + acc, it));
      // named barriers have no time limit: one thread decides for the four warps whether to go on
      named_bar_sync(3, 128);
      if (epi_tid == 0) *epi_go = ctl->abort ? 0 : 1;
      named_bar_sync(4, 128);
      ok = (*epi_go != 0);
      if (!ok) break;
      tc_fence_after();
      float r = r_pre;
      if (!PRESTATS) {
        float ssum = 0.f;
#pragma unroll
        for (int g = 0; g < TG; ++g) ssum += rs[(g * NACC + acc) * 128 + row];
        r = 1.0f / sqrtf(ssum / (float)p.K + p.eps);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rsfree(acc));
      }
      // convert 32 accumulator columns to bf16: 16 packed words
      // (col = first of the 32 columns within the tile; FP8 also applies the per-channel weight scales)
      auto cvt32 = [&](const uint32_t (&v)[32], uint32_t (&o)[16], [[maybe_unused]] int col) {
        if constexpr (FP8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 ws4 = *reinterpret_cast<const float4*>(wc_tile + col + 4 * j);
            o[2 * j] = pack_bf16x2(__uint_as_float(v[4 * j]) * r * ws4.x, __uint_as_float(v[4 * j + 1]) * r * ws4.y);
            o[2 * j + 1] = pack_bf16x2(__uint_as_float(v[4 * j + 2]) * r * ws4.z, __uint_as_float(v[4 * j + 3]) * r * ws4.w);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            o[j] = pack_bf16x2(__uint_as_float(v[2 * j]) * r, __uint_as_float(v[2 * j + 1]) * r);
        }
      };
      // write 64 columns (two 16-word halves) of this thread's row into a swizzled staging tile
      auto sts64 = [&](uint8_t* stage, const uint32_t (&lo)[16], const uint32_t (&hi)[16]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          *reinterpret_cast<uint4*>(stage + row * 128 + (((uint32_t)j ^ swz) << 4)) =
              make_uint4(lo[4 * j], lo[4 * j + 1], lo[4 * j + 2], lo[4 * j + 3]);
          *reinterpret_cast<uint4*>(stage + row * 128 + (((uint32_t)(4 + j) ^ swz) << 4)) =
              make_uint4(hi[4 * j], hi[4 * j + 1], hi[4 * j + 2], hi[4 * j + 3]);
        }
      };
      const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      bool tail_done = false;
      if constexpr (TAIL) {
        if (w.slice >= 0) {
          // ---- one k-slice of a tail tile (always this pair's last item).  The S contributors of a tile each
          // finish 1/S of its columns: a CTA writes the fp32 partials of the other contributors' columns to the
          // workspace, announces it, waits until all S have (they run at the same time: the grid is no larger
          // than the device holds), pulls the S - 1 other partials of its own columns through the idle operand
          // ring and adds them to its own in slice order, so the result does not depend on who came first.
          tail_done = true;
          const int S = p.tail_split;                     // 2, 3 or 4
          // the tile's four 64-column chunks are dealt to the S contributors as evenly as they go (S = 3: 1, 1, 2)
          const int c_lo = (w.slice * (BN / 64)) / S;
          const int nch = ((w.slice + 1) * (BN / 64)) / S - c_lo;
          const int tl = w.t - (total_tiles - p.tail_tiles);
          unsigned* cnt = p.tail_counters + 2 * (tl * 2 + (int)rank);  // [0] partials written, [1] waits passed
          constexpr int SLOT_F4 = 128 * BN / 4;                        // float4 per (tile, slice, rank) block
          constexpr uint32_t PART_BYTES = 64 * 128 * 4;                // 64 columns of a block: contiguous
          // (S - 1) x the chunks a contributor finishes: at most 4 of a 256-column tile's four chunks, 6 of a
          // 512-column tile's eight (S = 2: 4, S = 3: 2 x 3, S = 4: 3 x 2)
          constexpr uint32_t PART_BUFS = (BN == 512) ? 6 : 4;
          static_assert(PART_BUFS * PART_BYTES <= (uint32_t)Cfg::OFF_EPI, "partial buffers fit in the operand ring");
          // block layout [column / 4][row] float4: a warp's 32 rows of one column group are 512 contiguous bytes
          float4* slot0 = reinterpret_cast<float4*>(p.tail_partials) + (size_t)(tl * S * 2 + (int)rank) * SLOT_F4;
          float4* mine = slot0 + (size_t)w.slice * 2 * SLOT_F4;
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            if (c >= c_lo && c < c_lo + nch) continue;    // my own columns stay in tensor memory
            uint32_t v0[32], v1[32];
            tmem_ld32(trow + c * 64, v0);
            tmem_ld32(trow + c * 64 + 32, v1);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              mine[(c * 16 + j) * 128 + row] =
                  make_float4(__uint_as_float(v0[4 * j]), __uint_as_float(v0[4 * j + 1]), __uint_as_float(v0[4 * j + 2]),
                              __uint_as_float(v0[4 * j + 3]));
              mine[(c * 16 + 8 + j) * 128 + row] =
                  make_float4(__uint_as_float(v1[4 * j]), __uint_as_float(v1[4 * j + 1]), __uint_as_float(v1[4 * j + 2]),
                              __uint_as_float(v1[4 * j + 3]));
            }
          }
          __threadfence();
          named_bar_sync(1, 128);
          if (epi_tid == 0) {
            atomicAdd(cnt, 1u);
            const bool good = global_count_wait(cnt, (unsigned)S, ctl, 3, 100 + tl, it);
            if (good) {
              __threadfence();
              asm volatile("fence.proxy.async.global;" ::: "memory");  // the bulk copies below read what others wrote
              // the other contributors' partials of my columns: one bulk copy of 32 KB per (slice, chunk)
              mbar_expect_tx(bar_tail, (uint32_t)((S - 1) * nch) * PART_BYTES);
              int b = 0;
              for (int sl = 0; sl < S; ++sl) {
                if (sl == w.slice) continue;
                for (int c = 0; c < nch; ++c, ++b)
                  bulk_load_1d(sbase + (uint32_t)b * PART_BYTES,
                               slot0 + (size_t)sl * 2 * SLOT_F4 + (size_t)(c_lo + c) * 16 * 128, PART_BYTES, bar_tail);
              }
              // the last of the S to get here puts the pair of counters back to zero for the next launch
              if (atomicAdd(cnt + 1, 1u) == (unsigned)(S - 1)) {
                cnt[0] = 0u;
                cnt[1] = 0u;
              }
            }
            *epi_go = good ? 1 : 0;
            tma_store_wait_read<0>();  // earlier tiles' stores are done with the staging tiles
          }
          named_bar_sync(2, 128);
          ok = (*epi_go != 0);
          if (!ok) break;
          ok = mbar_wait(bar_tail, 0u, ctl, 3, 200 + tl, it);
          named_bar_sync(3, 128);
          if (epi_tid == 0) *epi_go = ctl->abort ? 0 : 1;
          named_bar_sync(4, 128);
          ok = (*epi_go != 0);
          if (!ok) break;
          const int m0 = mt * 256 + (int)rank * 128;
#pragma unroll 1
          for (int c = 0; c < nch; ++c) {
            uint8_t* stage = smem + Cfg::OFF_EPI + (c & 1) * Cfg::EPI_BYTES;
            uint32_t o[2][16];
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {  // 16 columns at a time keeps the register count of the hot loops
              uint32_t own[16];
              tmem_ld16(trow + (c_lo + c) * 64 + qq * 16, own);
              float a[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) a[j] = 0.f;
              tmem_wait_ld();
              int b = 0;
#pragma unroll 1
              for (int sl = 0; sl < S; ++sl) {  // slice order, this CTA's own slice in its place
                if (sl == w.slice) {
#pragma unroll
                  for (int j = 0; j < 16; ++j) a[j] += __uint_as_float(own[j]);
                } else {
                  const float4* ps = reinterpret_cast<const float4*>(smem + (size_t)(b * nch + c) * PART_BYTES) +
                                     (qq * 4) * 128 + row;
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float4 d4 = ps[j * 128];
                    a[4 * j] += d4.x; a[4 * j + 1] += d4.y; a[4 * j + 2] += d4.z; a[4 * j + 3] += d4.w;
                  }
                  ++b;
                }
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float s0 = r, s1 = r;
                if constexpr (FP8) {
                  const float2 ws2 = *reinterpret_cast<const float2*>(wc_tile + (c_lo + c) * 64 + qq * 16 + 2 * j);
                  s0 *= ws2.x;
                  s1 *= ws2.y;
                }
                o[qq >> 1][(qq & 1) * 8 + j] = pack_bf16x2(a[2 * j] * s0, a[2 * j + 1] * s1);
              }
            }
            sts64(stage, o[0], o[1]);
            fence_proxy_async_smem();
            named_bar_sync(2, 128);
            if (epi_tid == 0) {
              const int n0 = nt * BN + (c_lo + c) * 64;
              if (n0 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage), n0, m0, pol_y);
              tma_store_commit();
            }
          }
        }
      }
      if (tail_done) {
        // the slice's columns were finished above
      } else if constexpr (SWIGLU && WIDE) {
        // p.N = n output channels; this tile covers channels nt*256 .. +255: gate in columns [0,256), up in [256,512).
        // Four chunks of 64 output channels through the two staging tiles; both halves are free after the last read.
        const int m0 = mt * 256 + (int)rank * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c, ++chunk_no) {
          uint8_t* stage = smem + Cfg::OFF_EPI + (chunk_no & 1) * Cfg::EPI_BYTES;
          if (epi_tid == 0) tma_store_wait_read<1>();
          named_bar_sync(1, 128);
          uint32_t lo[16], hi[16];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t vg[32], vu[32];
            tmem_ld32(trow + c * 64 + h * 32, vg);
            tmem_ld32(trow + 256 + c * 64 + h * 32, vu);
            tmem_wait_ld();
            uint32_t (&o)[16] = (h == 0) ? lo : hi;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g0 = __uint_as_float(vg[2 * j]) * r, g1 = __uint_as_float(vg[2 * j + 1]) * r;
              const float u0 = __uint_as_float(vu[2 * j]) * r, u1 = __uint_as_float(vu[2 * j + 1]) * r;
              o[j] = pack_bf16x2(__fdividef(g0, 1.0f + __expf(-g0)) * u0, __fdividef(g1, 1.0f + __expf(-g1)) * u1);
            }
          }
          if (c == 3) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive_cluster(lead_tempty0);
              mbar_arrive_cluster(lead_tempty0 + 8u);
            }
          }
          sts64(stage, lo, hi);
          fence_proxy_async_smem();
          named_bar_sync(2, 128);
          if (epi_tid == 0) {
            const int n0 = nt * 256 + c * 64;
            if (n0 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage), n0, m0, pol_y);
            tma_store_commit();
          }
        }
      } else if constexpr (SWIGLU) {
        // p.N = n output channels; this tile covers channels nt*128 .. +127: gate in columns [0,128), up in [128,256)
        uint8_t* stage0 = smem + Cfg::OFF_EPI;
        uint8_t* stage1 = smem + Cfg::OFF_EPI + Cfg::EPI_BYTES;
        if (epi_tid == 0) tma_store_wait_read<0>();
        named_bar_sync(1, 128);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t lo[16], hi[16];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t vg[32], vu[32];
            tmem_ld32(trow + c * 64 + h * 32, vg);
            tmem_ld32(trow + 128 + c * 64 + h * 32, vu);
            tmem_wait_ld();
            uint32_t (&o)[16] = (h == 0) ? lo : hi;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g0 = __uint_as_float(vg[2 * j]) * r, g1 = __uint_as_float(vg[2 * j + 1]) * r;
              const float u0 = __uint_as_float(vu[2 * j]) * r, u1 = __uint_as_float(vu[2 * j + 1]) * r;
              // silu(g) = g / (1 + e^-g) with the fast exponential and division: the result is rounded to bf16
              // (8 bits of mantissa) right after, and an IEEE division per output would dominate this epilogue
              o[j] = pack_bf16x2(__fdividef(g0, 1.0f + __expf(-g0)) * u0, __fdividef(g1, 1.0f + __expf(-g1)) * u1);
            }
          }
          if (c == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * acc);
          }
          sts64(c == 0 ? stage0 : stage1, lo, hi);
        }
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        if (epi_tid == 0) {
          const int m0 = mt * 256 + (int)rank * 128;
          if (nt * 128 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage0), nt * 128, m0, pol_y);
          if (nt * 128 + 64 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage1), nt * 128 + 64, m0, pol_y);
          tma_store_commit();
        }
      } else if constexpr (NACC == 1 && BN == 256) {
        // One accumulator: the next tile's first MMA waits for this drain, so tensor memory is emptied as
        // fast as possible - columns 0..127 straight into the two staging tiles, columns 128..255 into
        // registers as packed bf16 - and released before any store is issued.
        uint8_t* stage0 = smem + Cfg::OFF_EPI;
        uint8_t* stage1 = smem + Cfg::OFF_EPI + Cfg::EPI_BYTES;
        if (epi_tid == 0) tma_store_wait_read<0>();  // the previous tile's stores are done reading the staging tiles
        named_bar_sync(1, 128);
        uint32_t pk[4][16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v0[32], v1[32];
          tmem_ld32(trow + c * 64, v0);
          tmem_ld32(trow + c * 64 + 32, v1);
          tmem_wait_ld();
          if (c < 2) {
            uint32_t lo[16], hi[16];
            cvt32(v0, lo, c * 64);
            cvt32(v1, hi, c * 64 + 32);
            sts64(c == 0 ? stage0 : stage1, lo, hi);
          } else {
            cvt32(v0, pk[2 * (c - 2)], c * 64);
            cvt32(v1, pk[2 * (c - 2) + 1], c * 64 + 32);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * acc);
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        const int m0 = mt * 256 + (int)rank * 128;
        if (epi_tid == 0) {
          if (nt * BN < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage0), nt * BN, m0, pol_y);
          if (nt * BN + 64 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage1), nt * BN + 64, m0, pol_y);
          tma_store_commit();
          tma_store_wait_read<0>();
        }
        named_bar_sync(1, 128);
        sts64(stage0, pk[0], pk[1]);
        sts64(stage1, pk[2], pk[3]);
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        if (epi_tid == 0) {
          if (nt * BN + 128 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage0), nt * BN + 128, m0, pol_y);
          if (nt * BN + 192 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage1), nt * BN + 192, m0, pol_y);
          tma_store_commit();
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c, ++chunk_no) {
          uint8_t* stage = smem + Cfg::OFF_EPI + (chunk_no & 1) * Cfg::EPI_BYTES;
          if (epi_tid == 0) tma_store_wait_read<1>();
          named_bar_sync(1, 128);
          uint32_t v0[32], v1[32];
          tmem_ld32(trow + c * 64, v0);
          tmem_ld32(trow + c * 64 + 32, v1);
          tmem_wait_ld();
          if (c == BN / 64 - 1 || (WIDE && c == 3)) {
            // accumulator (WIDE: this half of it) drained into registers: the pair's MMA warp may start on it again
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * (WIDE ? (c > 3 ? 1 : 0) : acc));
          }
          uint32_t lo[16], hi[16];
          cvt32(v0, lo, c * 64);
          cvt32(v1, hi, c * 64 + 32);
          sts64(stage, lo, hi);
          fence_proxy_async_smem();
          named_bar_sync(2, 128);
          if (epi_tid == 0) {
            const int n0 = nt * BN + c * 64;
            if (n0 < p.N) tma_store_2d_hint(&tm_y, smem_u32(stage), n0, mt * 256 + (int)rank * 128, pol_y);
            tma_store_commit();
          }
        }
      }
    }
    if (epi_tid == 0) tma_store_wait_all<0>();
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (ctl->abort) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();  // neither CTA frees tensor memory or exits while its peer may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace rl
