// C ABI of librmsnorm_linear: argument checks, TMA descriptors, kernel choice.
// Declarations and the reference interfaces they replace: include/rmsnorm_linear.h
#include "../../include/rmsnorm_linear.h"

#include <algorithm>
#include <atomic>
#include <mutex>

#include "rl_decode.cuh"
#include "rl_rowquant.cuh"
#include "rl_prefill.cuh"
#include "rl_prefill_pair.cuh"

namespace {

using namespace rl;

constexpr int RL_MAX_CTAS = 160;      // upper bound on the persistent grid (B200: 148 SMs)
constexpr size_t STATUS_BYTES = 256;  // RL_STATUS_INTS ints
// The tile counters must be zero between launches and kernels leave them so, but only if
// every shape finds them at the same place: the counter region has a fixed capacity and
// position, whatever M, N and K are.  Partial tiles behind it need no clean state.
constexpr int RL_MAX_DECODE_TILES = 16384;  // N <= 2,097,152 output channels
constexpr size_t COUNTER_BYTES = (size_t)RL_MAX_DECODE_TILES * 4;

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int cuda_err(cudaError_t e) { return RL_ERR_CUDA - (int)e; }

// ---- driver entry point for cuTensorMapEncodeTiled (no link-time libcuda dependency)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return (EncodeTiledFn)f;
  }();
  return fn;
}

// Row-major 2-D tensor [outer, inner] of 1- or 2-byte elements, 128-byte-swizzled boxes.
// Encoding a descriptor costs a few microseconds of host time, which shows at decode sizes (a 40 us
// kernel): the last few descriptors are kept per host thread, keyed by everything that defines them.
struct MapKey {
  const void* ptr;
  uint64_t inner, outer, stride;
  uint32_t box_inner, box_outer;
  int dt, dev;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && stride == o.stride && box_inner == o.box_inner &&
           box_outer == o.box_outer && dt == o.dt && dev == o.dev;
  }
};
int make_map(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* ptr, uint64_t inner,
             uint64_t outer, uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer) {
  constexpr int SLOTS = 16;
  thread_local MapKey keys[SLOTS];
  thread_local CUtensorMap maps[SLOTS];
  thread_local bool used[SLOTS] = {false};
  thread_local int next = 0;
  int dev = 0;
  (void)cudaGetDevice(&dev);
  const MapKey key{ptr, inner, outer, row_stride_elems, box_inner, box_outer, (int)dt, dev};
  for (int i = 0; i < SLOTS; ++i)
    if (used[i] && keys[i] == key) {
      *map = maps[i];
      return RL_OK;
    }
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return RL_ERR_TENSOR_MAP;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return RL_ERR_TENSOR_MAP;
  keys[next] = key;
  maps[next] = *map;
  used[next] = true;
  next = (next + 1) % SLOTS;
  return RL_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel and device instead of on every call.
template <class KernelFn>
cudaError_t set_smem_once(KernelFn fn, int bytes, bool max_carveout = false) {
  // keyed by the kernel's address: every instantiation with the same signature shares this function
  static std::mutex mu;
  static const void* seen[64][64];
  static int n_seen[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  dev &= 63;
  const void* key = reinterpret_cast<const void*>(fn);
  std::lock_guard<std::mutex> lk(mu);
  for (int i = 0; i < n_seen[dev]; ++i)
    if (seen[dev][i] == key) return cudaSuccess;
  e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  // a kernel sized for several CTAs per SM needs the whole shared-memory carve-out to get them
  if (e == cudaSuccess && max_carveout)
    e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess && n_seen[dev] < 64) seen[dev][n_seen[dev]++] = key;
  return e;
}

struct DeviceInfo {
  int sms = 0;
  int cc_major = 0;
  bool ok = false;
};
int device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_err(e);
  if (dev < 0 || dev >= 64) return RL_ERR_UNSUPPORTED_ARCH;
  std::lock_guard<std::mutex> lk(mu);
  if (!cache[dev].ok) {
    if ((e = cudaDeviceGetAttribute(&cache[dev].sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
      return cuda_err(e);
    if ((e = cudaDeviceGetAttribute(&cache[dev].cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
      return cuda_err(e);
    cache[dev].ok = true;
  }
  *out = cache[dev];
  return RL_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// fp32 partial blocks of k-split tail tiles: one 128 x 256 block per CTA of the persistent grid
constexpr size_t TAIL_SLOT_BYTES = (size_t)128 * 512 * 4;  // (the 512-column tiles' blocks; 256-column tiles use half)
constexpr size_t TAIL_BYTES = (size_t)RL_MAX_CTAS * TAIL_SLOT_BYTES;

// Wide layers fold gamma into a copy of x once, in the row-statistics pre-pass, instead of in every column tile's
// main loop (rowscale_kernel): the fold is then done once per activation, not N / 256 times, and the GEMM runs
// without transform warps and with two accumulators.  The copy costs one more pass over x that the GEMM has to
// wait for (4 M K bytes of DRAM traffic plus a few microseconds of exposed launch and wait), whatever N.  Measured,
// gamma folded in the main loop against in the pre-pass, same bits out.  By width at M >= 2048: N = 1536 5 %
// slower, 4096 equal, 6144 2-3 % faster, 8192 to 57344 4-6 % faster (bursts and seconds-long loops alike).  By
// size at N >= 6144: 128 x 6144 x 4096 and 256 x 8192 x 4096 8-10 % slower (a 30 us GEMM behind a 4 us wait),
// 512 x 14336 x 4096 and 1024 x 6144 x 4096 equal, 2048 x 8192 x 2048 5 % faster.
constexpr int RL_PRESCALE_MIN_N = 6144;
constexpr long long RL_PRESCALE_MIN_MNK = 30000000000ll;   // M N K: a GEMM of about 50 us
inline bool prescale_pays(int M, int N, int K) {
  return N >= RL_PRESCALE_MIN_N && (long long)M * N * K >= RL_PRESCALE_MIN_MNK;
}

#ifndef RL_ROUND_WAIT_NS
#define RL_ROUND_WAIT_NS 50000u
#endif
#ifndef RL_ALIGN_MIN_ROUNDS
#define RL_ALIGN_MIN_ROUNDS 32
#endif
constexpr size_t SYNC_BYTES = 1024;  // RL_MAX_CTAS / 2 progress words, rounded up
struct WsLayout {
  size_t counters_off, ssq_off, partials_off, total;
  size_t rstd_off, tail_off, min_total;  // M > 64 only
  size_t sync_off;                       // M > 64: one progress word per CTA pair (alignment at tile boundaries)
  size_t tail_total;                     // M > 64: end of the k-split partial blocks
  size_t xs_off, xs_bytes;               // M > 64, wide layers: the gamma-folded copy of x [M, K] (0 bytes otherwise)
};
WsLayout ws_layout(int M, int N, int K = 0) {
  WsLayout w{};
  if (M > 64) {
    // status block, the counter region every shape keeps at the same place (zero between launches), 1/rms per
    // token for the PRESTATS kernels, the partial blocks of k-split tail tiles, then (wide layers) the folded copy
    // of x.  A workspace that ends before the partial blocks (min_total) still works: the tail tiles are then
    // computed whole; one that ends before the copy (tail_total) still works: gamma is folded in the main loop.
    w.counters_off = STATUS_BYTES;
    w.rstd_off = STATUS_BYTES + COUNTER_BYTES;
    w.sync_off = w.rstd_off + align_up((size_t)M * 4, 256);
    w.tail_off = w.sync_off + SYNC_BYTES;
    w.min_total = w.tail_off;
    w.tail_total = w.tail_off + TAIL_BYTES;
    w.xs_off = w.tail_total;
    w.xs_bytes = (K > 0 && prescale_pays(M, N, K)) ? align_up((size_t)M * (size_t)K * 2, 256) : 0;
    w.total = w.xs_off + w.xs_bytes;
    return w;
  }
  const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  (void)N;
  w.counters_off = STATUS_BYTES;
  w.ssq_off = w.counters_off + COUNTER_BYTES;
  w.partials_off = w.ssq_off + align_up((size_t)RL_MAX_CTAS * 2 * mpad * 4, 256);
  w.total = w.partials_off + (size_t)RL_MAX_CTAS * 2 * mpad * 128 * 4;
  return w;
}

// The CTA-pair configurations the entry points use: <BN, accumulators, ring stages, A slots in tensor memory,
// transform groups, A operand mode, 1/rms from the pre-pass, SwiGLU epilogue, FP8 operands>.
using PairFold = PairCfg<256, 1, 6, 6, 2, A_TS_FOLD, true>;        // gamma folded through tensor memory; k-split tail
using PairFoldFused = PairCfg<256, 1, 6, 6, 2, A_TS_FOLD>;         // the same with the sums of squares in the transform
using PairFoldN192 = PairCfg<192, 2, 6, 4, 2, A_TS_FOLD>;
using PairDirectFused = PairCfg<256, 2, 6, 1, 2, A_SS_DIRECT>;     // no gamma: x straight from shared memory
using PairDirect = PairCfg<256, 2, 6, 1, 0, A_SS_DIRECT, true>;    // ... with 1/rms from the pre-pass (or no norm at all)
using PairWide = PairCfg<512, 2, 4, 1, 0, A_SS_DIRECT, true>;      // the same on 256 x 512 tiles: half the x bytes per FLOP
using PairSwigluWide = PairCfg<512, 2, 4, 1, 0, A_SS_DIRECT, true, true>;  // 256 output channels per tile: 256 gate + 256 up columns
using PairSwiglu = PairCfg<256, 1, 6, 6, 2, A_TS_FOLD, true, true>;
using PairSwigluDirect = PairCfg<256, 2, 6, 1, 0, A_SS_DIRECT, true, true>;  // no gamma, or gamma folded by the pre-pass
using PairFp8 = PairCfg<256, 2, 6, 1, 0, A_SS_DIRECT, true, false, true>;

template <class Cfg>
int launch_prefill(const void* x, const __nv_bfloat16* gamma, const void* W, void* y, int M, int N, int K,
                   int64_t ldx, int64_t ldw, int64_t ldy, float eps, int* status, int sms, cudaStream_t st) {
  CUtensorMap tx, tw, ty;
  int rc;
  if ((rc = make_map(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, K, M, ldx, 64, 128))) return rc;
  if ((rc = make_map(&tw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, K, N, ldw, 64, Cfg::BN))) return rc;
  if ((rc = make_map(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, N, M, ldy, 64, 128))) return rc;
  PrefillParams p{};
  p.M = M; p.N = N; p.K = K; p.eps = eps;
  p.gamma = gamma;
  p.m_tiles = (M + 127) / 128;
  p.n_tiles = (N + Cfg::BN - 1) / Cfg::BN;
  p.group_m = 16;
  p.status = status;
  const long long tiles = (long long)p.m_tiles * p.n_tiles;
  const int grid = (int)(tiles < sms ? tiles : sms);
  cudaError_t e = set_smem_once(prefill_kernel<Cfg>, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return cuda_err(e);
  prefill_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(tx, tw, ty, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? RL_OK : cuda_err(e);
}

// How many CTA pairs of this kernel the device holds at once (the two CTAs of a pair sit on neighbouring SMs of
// one TPC, so this can be fewer than SMs / 2).  Asked once per device and kernel.
template <class Cfg>
int max_cta_pairs(int sms, int* out) {
  static int cache[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int n = cache[dev & 63];
  if (n == 0) {
    cudaError_t e = set_smem_once(prefill_pair_kernel<Cfg>, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return cuda_err(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sms / 2));
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    e = cudaOccupancyMaxActiveClusters(&n, prefill_pair_kernel<Cfg>, &cfg);
    if (e != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = sms / 2; }
    cache[dev & 63] = n;
  }
  *out = n;
  return RL_OK;
}

// What to do with the last, partly filled round of tiles.  `tiles` tiles are dealt to `max_pairs` CTA pairs; r =
// tiles % max_pairs of them form the last round, which costs a whole tile's time however few they are.  Cut
// along K into S slices, r * S pairs share that work and then spend a few microseconds exchanging partial
// sums; worth it when the slices are long enough (KB k-blocks of 64 in the whole K).
struct TailPlan {
  int tiles, split;
};
TailPlan plan_tail(long long tiles, int max_pairs, int KB) {
  const int r = (int)(tiles % max_pairs);
  if (r == 0) return TailPlan{0, 0};
  // the exchange costs about as much as 15 k-blocks of the main loop (measured: ~5 us); split only when each pair
  // is spared clearly more than that: KB (1 - 1/S) >= 20
  if ((long long)r * 4 <= max_pairs && r * 4 * 2 <= RL_MAX_CTAS && KB >= 32) return TailPlan{r, 4};
  if ((long long)r * 3 <= max_pairs && r * 3 * 2 <= RL_MAX_CTAS && KB >= 32) return TailPlan{r, 3};
  if ((long long)r * 2 <= max_pairs && r * 2 * 2 <= RL_MAX_CTAS && KB >= 40) return TailPlan{r, 2};
  return TailPlan{0, 0};
}

// 256 x 512 tiles (PairWide) halve the activation bytes every pair pulls in and issue eight MMAs per barrier wait
// instead of four: measured 6-10 % more work per unit of time than 256 x 256 tiles, tile for tile.  There are half as
// many of them, so their last, partly filled round weighs twice as much.  Both widths are costed in units of one
// narrow tile's time - whole rounds, plus the last round: nothing, a k-split's 1/S and the exchange (about 15
// k-blocks), or a whole round when it cannot be split - and the wide tiles run where theirs, at 93 % per column,
// comes to at least 2 % less.
inline double rounds_cost(long long tiles, int pairs, int KB) {
  const TailPlan tp = plan_tail(tiles, pairs, KB);
  const double last = (tiles % pairs == 0) ? 0.0 : (tp.split > 1 ? 1.0 / tp.split + 15.0 / KB : 1.0);
  return (double)(tiles / pairs) + last;
}
inline bool wide_tiles_pay(int M, int N, int K, int pairs) {
  if (K < 4096 || pairs <= 0) return false;
  const long long m_tiles = (M + 255) / 256;
  const long long tiles512 = m_tiles * ((N + 511) / 512), tiles256 = m_tiles * ((N + 255) / 256);
  if (tiles512 < 3LL * pairs) return false;
  const int KB = (K + 63) / 64;
  return 2.0 * 0.93 * rounds_cost(tiles512, pairs, KB) < 0.98 * rounds_cost(tiles256, pairs, KB);
}

// Row tiles (of 256 tokens) per sweep group.  Tiles are walked group by group, a group's row tiles against every
// column tile, so the x rows of one group stay in L2 while W streams past; W is read from DRAM once per group.
// Two limits.  The group's x rows must fit a budget well inside the 126 MB L2 (the W tiles in flight and the y
// tiles on their way out share it).  And the 74 pairs running at a time should cover a patch of tiles that is not
// too far from square: a taller group makes them touch more distinct operand tiles at once.  Measured: on
// 16384 x 7168 x 8192 groups of 10 beat groups of 8 by 2 %; groups of 8, 10 and 16 time the same on the 4096- and
// 8192-token shapes while 16 halves the weight re-reads; groups of 32 ran the e4m3 kernel 5-6 % slower on
// narrow weights although W then streamed from DRAM only once.
constexpr int RL_GROUP_BUDGET_MB = 40;
constexpr int RL_GROUP_MAX = 16;
int pick_group_m(int m_tiles, long long row_tile_bytes) {
  long long g = ((long long)RL_GROUP_BUDGET_MB << 20) / (row_tile_bytes > 0 ? row_tile_bytes : 1);
  if (g > RL_GROUP_MAX) g = RL_GROUP_MAX;
  if (g < 4) g = 4;
  if (g > m_tiles) g = m_tiles;
  const long long groups = (m_tiles + g - 1) / g;  // even the groups out
  return (int)((m_tiles + groups - 1) / groups);
}

// Everything a launch of the CTA-pair kernel needs besides its configuration.
struct PairArgs {
  const void* x = nullptr;             // [M, K] bf16 (FP8: e4m3 activations from rowquant_kernel)
  const __nv_bfloat16* gamma = nullptr;
  const void* W = nullptr;             // [N, K] (SwiGLU: [2N, K])
  void* y = nullptr;
  int M = 0, N = 0, K = 0;
  int64_t ldx = 0, ldw = 0, ldy = 0;
  float eps = 0.f;
  int* status = nullptr;               // start of the workspace, or nullptr
  size_t ws_bytes = 0;
  size_t tail_off = 0, ws_total = 0;   // where the partial blocks of k-split tiles live, and the size that holds them
  size_t sync_off = 0;                 // where the pairs' progress words live (0 = none)
  int sms = 0;
  void* xs = nullptr;                  // gamma-folded copy of x [M, K] for the pre-pass to write (wide layers), or nullptr
  cudaStream_t st = nullptr;
  bool no_norm = false;                // plain GEMM: no row statistics at all
  bool split_tail = true;
  const void* x2 = nullptr;            // LoRA: second operand pair [M, L] / [N, L]
  const void* w2 = nullptr;
  int L = 0;
  int64_t ldx2 = 0, ldw2 = 0;
  const float* row_scale = nullptr;    // FP8: per-token scale (already computed on `st`)
  const float* w_scale = nullptr;      // FP8: per-channel weight scales
};

template <class Cfg>
int launch_prefill_pair(const PairArgs& a) {
  CUtensorMap tx, tw, ty, tx2, tw2;
  int rc;
  const int M = a.M, N = a.N, K = a.K;
  const CUtensorMapDataType dt = Cfg::FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int eb = Cfg::FP8 ? 1 : 2;
  // gamma folded by the pre-pass into a dense copy of x: the GEMM reads the copy and sees no gamma
  const bool prescale = (a.xs != nullptr);
  if (prescale && !(Cfg::AMODE == A_SS_DIRECT && Cfg::PRESTATS && !Cfg::FP8 && a.gamma != nullptr &&
                    !a.no_norm && a.x2 == nullptr))
    return RL_ERR_BAD_VARIANT;
  if ((rc = make_map(&tx, dt, eb, prescale ? a.xs : a.x, K, M, prescale ? (int64_t)K : a.ldx, Cfg::KBW, 128))) return rc;
  if ((rc = make_map(&tw, dt, eb, a.W, K, Cfg::SWIGLU ? 2 * (uint64_t)N : (uint64_t)N, a.ldw, Cfg::KBW,
                     Cfg::WIDE ? 128 : Cfg::BN / 2)))
    return rc;
  if ((rc = make_map(&ty, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y, N, M, a.ldy, 64, 128))) return rc;
  if (Cfg::AMODE == A_SS_DIRECT && a.gamma != nullptr && !prescale) return RL_ERR_BAD_VARIANT;
  tx2 = tx;
  tw2 = tw;
  if (a.x2 != nullptr) {
    // second operand pair [M, L] / [N, L]: same boxes as the first, columns L..63 come back as zeros
    if (Cfg::AMODE != A_SS_DIRECT || Cfg::SWIGLU || Cfg::FP8 || Cfg::WIDE || a.L <= 0 || a.L > 64) return RL_ERR_BAD_VARIANT;
    if ((rc = make_map(&tx2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.x2, a.L, M, a.ldx2, 64, 128))) return rc;
    if ((rc = make_map(&tw2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.w2, a.L, (uint64_t)N, a.ldw2, 64, Cfg::BN / 2))) return rc;
  }
  PrefillParams p{};
  p.M = M; p.N = N; p.K = K; p.eps = a.eps;
  p.gamma = prescale ? nullptr : a.gamma;
  p.x_from_prepass = prescale ? 1 : 0;
  p.m_tiles = (M + 255) / 256;
  // SwiGLU: N = output channels, W has 2N rows; a tile covers half as many output channels as it has accumulator columns
  p.n_tiles = Cfg::SWIGLU ? (N + Cfg::BN / 2 - 1) / (Cfg::BN / 2) : (N + Cfg::BN - 1) / Cfg::BN;
  p.group_m = pick_group_m(p.m_tiles, (long long)256 * K * eb);
  p.status = a.status;
  p.extra_kb = (a.x2 != nullptr) ? 1 : 0;
  p.w_scale = a.w_scale;
  if (Cfg::FP8) {
    if (a.row_scale == nullptr || a.w_scale == nullptr) return RL_ERR_NULL_POINTER;
    p.row_rstd = a.row_scale;
  } else if (Cfg::PRESTATS && !a.no_norm) {
    if (a.status == nullptr) return RL_ERR_WORKSPACE;
    float* rstd = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a.status) + ws_layout(M > 65 ? M : 65, N).rstd_off);
    if (prescale)
      rowscale_kernel<<<(M + 3) / 4, 128, 0, a.st>>>(reinterpret_cast<const __nv_bfloat16*>(a.x), a.gamma,
                                                     reinterpret_cast<__nv_bfloat16*>(a.xs), rstd, M, K, a.ldx, K, a.eps);
    else
      rowstats_kernel<<<(M + 3) / 4, 128, 0, a.st>>>(reinterpret_cast<const __nv_bfloat16*>(a.x), rstd, M, K, a.ldx, a.eps);
    p.row_rstd = rstd;
  }
  cudaError_t e = set_smem_once(prefill_pair_kernel<Cfg>, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return cuda_err(e);
  int max_pairs = 0;
  if ((rc = max_cta_pairs<Cfg>(a.sms, &max_pairs))) return rc;
  const long long tiles = (long long)p.m_tiles * p.n_tiles;
  int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
  if (Cfg::PRESTATS && !Cfg::SWIGLU && (Cfg::BN == 256 || Cfg::BN == 512) && a.split_tail && a.status != nullptr) {
    const TailPlan tp = plan_tail(tiles, max_pairs, (K + Cfg::KBW - 1) / Cfg::KBW + p.extra_kb);
    if (tp.split > 1 && a.ws_total > 0 && a.ws_bytes >= a.ws_total) {
      p.tail_tiles = tp.tiles;
      p.tail_split = tp.split;
      p.tail_counters = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(a.status) + STATUS_BYTES);
      p.tail_partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a.status) + a.tail_off);
      if (tiles < max_pairs) pairs = tp.tiles * tp.split;  // fewer tiles than pairs: every tile is cut
    }
  }
  // Long sweeps of wide tiles (a workspace given, and the caller has not asked for kernels whose CTAs never wait):
  // the pairs re-align at tile boundaries, best effort, RL_ROUND_WAIT_NS at most per tile.  Measured: it halves
  // the DRAM reads of 16384 x 28672 x 8192 (48 rounds: 11.6 -> 5.8 GB, 1321 -> 1352 TFLOP/s sustained) and changes
  // nothing at 12 rounds (24 rounds: +1 % sustained at K = 8192, -0.7 % at K = 4096); on the 256 x 256 kernels, whose few rounds end in a k-split, it cost 2-6 % in bursts
  // (pairs that start every tile together hit L2 together), so they run free.
  if (Cfg::WIDE && a.sync_off != 0 && a.split_tail && a.status != nullptr && a.ws_bytes >= a.sync_off + SYNC_BYTES &&
      tiles >= (long long)RL_ALIGN_MIN_ROUNDS * pairs && tiles / pairs < 4000) {
    static std::atomic<unsigned> epoch_counter{0};
    p.round_words = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(a.status) + a.sync_off);
    p.round_epoch = (++epoch_counter) & 0xfffffu;
    p.round_wait_ns = RL_ROUND_WAIT_NS;
  }
  if (Cfg::PRESTATS && p.row_rstd != nullptr) {
    // behind rowstats_kernel (FP8: rowquant_kernel) with programmatic stream serialisation: the GEMM sets up
    // and, in the bf16 case, streams its tiles while the row statistics are still being computed, and waits only
    // where it first reads them.  Only in that case: rowstats_kernel and rowscale_kernel are normal launches, so
    // everything earlier in the stream (whoever wrote x and W) is complete before they start, and the producer
    // warp may load the caller's operands without waiting (rowquant_kernel is itself a programmatic dependent that
    // waits before it reads anything, and the FP8 producer waits for it before its first load, which amounts to
    // the same).  With the norm switched off nothing is launched in front, and the
    // kernel must not become a programmatic dependent of whatever the caller ran before it: it is launched
    // normally below.
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(2 * pairs));
    lc.blockDim = dim3(Cfg::THREADS);
    lc.dynamicSmemBytes = Cfg::SMEM_BYTES;
    lc.stream = a.st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    e = cudaLaunchKernelEx(&lc, prefill_pair_kernel<Cfg>, tx, tw, ty, tx2, tw2, p);
    return e == cudaSuccess ? RL_OK : cuda_err(e);
  }
  prefill_pair_kernel<Cfg><<<2 * pairs, Cfg::THREADS, Cfg::SMEM_BYTES, a.st>>>(tx, tw, ty, tx2, tw2, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? RL_OK : cuda_err(e);
}

// The 16-token configuration of the small-M kernel: <tokens, ring stages, transform warps, CTAs per SM>.
#ifndef RL_DEC16_STAGES
#define RL_DEC16_STAGES 8
#define RL_DEC16_TW 4
#define RL_DEC16_MINB 1
#endif
using DecodeCfg16 = DecodeCfg<16, RL_DEC16_STAGES, RL_DEC16_TW, RL_DEC16_MINB>;

// x / W: bf16, or (FP8 configuration) the e4m3 activations from rowquant_kernel and the e4m3 weights, with the
// per-token and per-channel scales the epilogue applies.
template <class Cfg>
int launch_decode(const void* x, const __nv_bfloat16* gamma, const void* W, void* y, int M, int N, int K,
                  int64_t ldx, int64_t ldw, int64_t ldy, float eps, uint8_t* ws, const WsLayout& wl, int sms,
                  cudaStream_t st, const float* row_scale = nullptr, const float* w_scale = nullptr) {
  CUtensorMap tw, tx;
  int rc;
  const CUtensorMapDataType dt = Cfg::FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int eb = Cfg::FP8 ? 1 : 2;
  if (Cfg::FP8 && (!row_scale || !w_scale)) return RL_ERR_NULL_POINTER;
  if ((rc = make_map(&tw, dt, eb, W, K, N, ldw, Cfg::KBW, 128))) return rc;
  if ((rc = make_map(&tx, dt, eb, x, K, M, ldx, Cfg::KBW, Cfg::MPAD))) return rc;
  DecodeParams p{};
  p.M = M; p.N = N; p.K = K; p.eps = eps;
  p.gamma = gamma;
  p.row_scale = row_scale;
  p.w_scale = w_scale;
  p.y = reinterpret_cast<__nv_bfloat16*>(y);
  p.ldy = ldy;
  p.n_tiles = (N + 127) / 128;
  if (p.n_tiles > RL_MAX_DECODE_TILES) return RL_ERR_BAD_SHAPE;
  p.KB = (K + Cfg::KBW - 1) / Cfg::KBW;
  const long long units = (long long)p.n_tiles * p.KB;
  if (units > 0x7fffffffLL) return RL_ERR_BAD_SHAPE;
  p.status = reinterpret_cast<int*>(ws);
  p.counters = reinterpret_cast<int*>(ws + wl.counters_off);
  p.ssq_partials = reinterpret_cast<float*>(ws + wl.ssq_off);
  p.partials = reinterpret_cast<float*>(ws + wl.partials_off);
  int grid = sms < RL_MAX_CTAS ? sms : RL_MAX_CTAS;
  if (units < grid) grid = (int)units;
  // every CTA owns floor(tiles / grid) tiles whole; the k-loops of the other tiles are shared out evenly.
  // Only in the 16-token configuration: measured, it gains 0.6 % there and costs 6 % at 64 tokens, where the
  // plain contiguous split (every tile's k-loop shared) is kept.
  p.whole_per_cta = (Cfg::MPAD <= 16) ? p.n_tiles / grid : 0;
  p.sk_tiles = p.n_tiles - p.whole_per_cta * grid;
  p.units_total = p.sk_tiles * p.KB;
  cudaError_t e = set_smem_once(decode_kernel<Cfg>, Cfg::SMEM_BYTES, Cfg::MINB > 1);
  if (e != cudaSuccess) return cuda_err(e);
  // Programmatic stream serialisation: this grid's prologue (barrier setup, tensor-memory allocation,
  // descriptor fetch) may overlap the tail of the previous kernel in the stream.  The kernel touches no
  // global memory before griddepcontrol.wait, so nothing else changes for the caller.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(Cfg::THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_kernel<Cfg>, tw, tx, p);
  return e == cudaSuccess ? RL_OK : cuda_err(e);
}

struct Fp8WsLayout {
  size_t row_scale_off, xq_off, tail_off, min_total, total;
};
Fp8WsLayout fp8_ws_layout(int M, int K) {
  Fp8WsLayout w{};
  w.row_scale_off = STATUS_BYTES + COUNTER_BYTES;  // behind the tile-counter region, which must stay zero
  w.xq_off = align_up(w.row_scale_off + (size_t)M * 4, 1024);
  w.tail_off = align_up(w.xq_off + (size_t)M * (size_t)K, 1024);
  w.min_total = w.tail_off;            // enough to run; the tail tiles are then computed whole
  w.total = w.tail_off + TAIL_BYTES;   // with room for the partial blocks of k-split tail tiles
  return w;
}

int launch_rowquant(const void* x, const void* gamma, void* q, float* row_scale, int M, int K, int64_t ldx,
                    int64_t ldq, float eps, cudaStream_t st) {
  RowQuantParams p{};
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  p.q = reinterpret_cast<uint8_t*>(q);
  p.row_scale = row_scale;
  p.M = M; p.K = K; p.ldx = ldx; p.ldq = ldq; p.eps = eps;
  // a programmatic dependent of whatever runs in front of it (the kernel waits for that to complete before it
  // reads anything): 16x28672x4096 with e4m3 weights, steps back to back, 26.8 -> 25.3 us
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3((unsigned)M);
  lc.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  cudaError_t e;
  if (K <= 4096) { lc.blockDim = dim3(128); e = cudaLaunchKernelEx(&lc, rowquant_kernel<128>, p); }
  else if (K <= 8192) { lc.blockDim = dim3(256); e = cudaLaunchKernelEx(&lc, rowquant_kernel<256>, p); }
  else { lc.blockDim = dim3(512); e = cudaLaunchKernelEx(&lc, rowquant_kernel<512>, p); }
  return e == cudaSuccess ? RL_OK : cuda_err(e);
}

// ---- self-test of the bounded waits: one CTA waits on an mbarrier that nothing ever arrives on, with a
// short limit, and must come back with an error record instead of hanging.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ CtaCtl ctl;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    ctl.abort = 0;
    ctl.status = status;
    ctl.limit_ns = limit_ns;
    fence_mbar_init();
  }
  __syncthreads();
  // every thread waits for phase 0, which never completes; the first to run out of time aborts the CTA
  const bool ok = mbar_wait(smem_u32(&bar), 0, &ctl, /*role=*/9, /*bar_id=*/0, /*idx=*/(int)threadIdx.x);
  __syncthreads();
  if (threadIdx.x == 0 && status != nullptr) status[6] = ok ? 1 : 2;  // 2: the wait gave up, as it should
}

// ---- scratch for the allocation-free entry point: lives in the library's device image, one copy per
// GPU that loads the library, held until the process exits.  In host code this name is only a handle
// for cudaGetSymbolAddress, never a device address to pass to a kernel.
constexpr size_t RL_STATIC_SCRATCH_BYTES = 3u << 20;  // 3 MiB: enough for M <= 16 tokens, any N the decode kernel takes
static __device__ __align__(256) unsigned char g_static_scratch[RL_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.
int static_scratch_address(uint8_t** out) {
  static std::mutex mu;
  static void* cache[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_err(e);
  if (dev < 0 || dev >= 64) return RL_ERR_UNSUPPORTED_ARCH;
  std::lock_guard<std::mutex> lk(mu);
  if (cache[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return cuda_err(e);
    if (ptr == nullptr) return RL_ERR_WORKSPACE;
    cache[dev] = ptr;
  }
  *out = reinterpret_cast<uint8_t*>(cache[dev]);
  return RL_OK;
}

// What RL_VARIANT_AUTO runs for a bf16 call.
int select_variant(int M, int N, bool has_gamma, bool has_workspace, int sms, bool ws_holds_copy = false) {
  if (M <= 64) return RL_VARIANT_DECODE;
  // 64 < M <= 128 runs on the CTA-pair kernel as well (half of each 256-row tile is padding, but the tiles can be
  // cut along K over all pairs: measured 20-30 % faster than one CTA per 128 x 192 tile, which leaves SMs idle)
  // Without gamma (the reference operator) x needs no fold: the MMA reads it straight from shared memory,
  // which frees tensor memory for a second accumulator.
  // Row statistics: from the overlapped pre-pass when there is a workspace and more than one round of tiles
  // (or few enough tiles that their k-loops get split): every column tile would otherwise recompute the same
  // sums on warps that share schedulers with the MMA warp.  With one round, not split, the pre-pass only adds
  // a second read of x and a launch in front of an epilogue that has to wait for it (12-15 % at K >= 4096):
  // there the transform warps accumulate the sums themselves.
  int pairs = sms / 2;
  (void)max_cta_pairs<PairFold>(sms, &pairs);
  const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
  const bool one_round = tiles <= pairs && 2 * tiles > pairs;
  if (!has_workspace || one_round) return has_gamma ? RL_VARIANT_PREFILL_PAIR_N256 : RL_VARIANT_PREFILL_PAIR_DIRECT;
  // wide layers: gamma folded once per activation by the pre-pass instead of once per column tile in the main loop
  if (has_gamma && ws_holds_copy) return RL_VARIANT_PREFILL_PAIR_PRESCALED;
  return has_gamma ? RL_VARIANT_PREFILL_PAIR_PRESTATS : RL_VARIANT_PREFILL_PAIR_DIRECT_PRESTATS;
}

// select_variant, then 256 x 512 tiles in place of the transform-free 256 x 256 kernels where those pay.
int auto_variant(int M, int N, int K, bool has_gamma, bool has_workspace, bool ws_holds_copy, int sms) {
  const int v = select_variant(M, N, has_gamma, has_workspace, sms, ws_holds_copy);
  if (v != RL_VARIANT_PREFILL_PAIR_DIRECT_PRESTATS && v != RL_VARIANT_PREFILL_PAIR_PRESCALED) return v;
  int pairs = 0;
  if (max_cta_pairs<PairWide>(sms, &pairs) != RL_OK || !wide_tiles_pay(M, N, K, pairs)) return v;
  return RL_VARIANT_PREFILL_PAIR_WIDE;
}

}  // namespace

extern "C" {

int rl_version(void) { return 1000; }

const char* rl_error_string(int code) {
  switch (code) {
    case RL_OK: return "ok";
    case RL_ERR_NULL_POINTER: return "a required pointer is NULL";
    case RL_ERR_BAD_SHAPE: return "M, N and K must be positive and leading dimensions must cover a row";
    case RL_ERR_ALIGNMENT:
      return "K and the leading dimensions must be multiples of 8 elements (16 for e4m3) and pointers 16-byte aligned";
    case RL_ERR_BAD_DTYPE: return "unknown weight dtype";
    case RL_ERR_WORKSPACE: return "workspace missing or smaller than rl_workspace_bytes()";
    case RL_ERR_UNSUPPORTED_ARCH: return "the current device is not an sm_100 (B200) GPU";
    case RL_ERR_BAD_VARIANT: return "unknown kernel variant, or one that cannot run this shape";
    case RL_ERR_TENSOR_MAP: return "the driver rejected a TMA descriptor";
    case RL_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out of time";
    case RL_ERR_STATIC_SCRATCH:
      return "shape exceeds the built-in scratch of the allocation-free entry point (M <= 16 tokens)";
    default: break;
  }
  if (code <= RL_ERR_CUDA) return cudaGetErrorString((cudaError_t)(RL_ERR_CUDA - code));
  return "unknown error code";
}

size_t rl_workspace_bytes(int M, int N, int K, int w_dtype) {
  if (M <= 0 || N <= 0 || K <= 0) return STATUS_BYTES;
  if (w_dtype == RL_W_E4M3) return fp8_ws_layout(M, K).total;
  return ws_layout(M, N, K).total;
}

int rl_plan_tail_split(int M, int N, int K, int pairs, int* tail_tiles, int* split) {
  if (M <= 0 || N <= 0 || K <= 0 || pairs <= 0) return RL_ERR_BAD_SHAPE;
  const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
  const TailPlan tp = plan_tail(tiles, pairs, (K + 63) / 64);
  if (tail_tiles) *tail_tiles = tp.tiles;
  if (split) *split = tp.split;
  return RL_OK;
}

int rl_select_variant(int M, int N, int K, int has_gamma, int has_workspace) {
  if (M <= 0 || N <= 0 || K <= 0) return RL_ERR_BAD_SHAPE;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (di.cc_major != 10) return RL_ERR_UNSUPPORTED_ARCH;
  return auto_variant(M, N, K, has_gamma != 0, has_workspace != 0, has_workspace != 0 && prescale_pays(M, N, K), di.sms);
}

int rl_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return RL_ERR_NULL_POINTER;
  if (workspace_bytes < STATUS_BYTES) return RL_ERR_WORKSPACE;
  cudaError_t e = cudaMemsetAsync(workspace, 0, workspace_bytes, (cudaStream_t)stream);
  return e == cudaSuccess ? RL_OK : cuda_err(e);
}

int rl_rmsnorm_linear_bf16(const void* x, const void* gamma, const void* W, void* y, int M, int N, int K,
                           int64_t ldx, int64_t ldw, int64_t ldy, float eps, void* workspace,
                           size_t workspace_bytes, int variant, void* stream) {
  if (!x || !W || !y) return RL_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || ldy < N) return RL_ERR_BAD_SHAPE;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || !aligned16(x) || !aligned16(W) || (gamma && !aligned16(gamma)))
    return RL_ERR_ALIGNMENT;
  const bool auto_whole = (variant == RL_VARIANT_AUTO_WHOLE);  // AUTO, but no kernel whose CTAs wait for each other
  if (auto_whole) variant = RL_VARIANT_AUTO;
  const bool decode = (variant == RL_VARIANT_DECODE) || (variant == RL_VARIANT_AUTO && M <= 64);
  if (decode && M > 64) return RL_ERR_BAD_VARIANT;
  if (!decode && ((ldy & 7) || !aligned16(y))) return RL_ERR_ALIGNMENT;
  const WsLayout wl = ws_layout(decode || M > 65 ? M : 65, N, K);
  if (decode && !workspace) return RL_ERR_WORKSPACE;
  if (workspace && workspace_bytes < (decode ? wl.total : wl.min_total)) return RL_ERR_WORKSPACE;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (di.cc_major != 10) return RL_ERR_UNSUPPORTED_ARCH;
  cudaStream_t st = (cudaStream_t)stream;
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(gamma);
  int* status = reinterpret_cast<int*>(workspace);

  if (decode) {
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    if (M <= 16) return launch_decode<DecodeCfg16>(x, g, W, y, M, N, K, ldx, ldw, ldy, eps, ws, wl, di.sms, st);
    if (M <= 32) return launch_decode<DecodeCfg<32, 8>>(x, g, W, y, M, N, K, ldx, ldw, ldy, eps, ws, wl, di.sms, st);
    return launch_decode<DecodeCfg<64, 8>>(x, g, W, y, M, N, K, ldx, ldw, ldy, eps, ws, wl, di.sms, st);
  }

  // M > 128: CTA pairs on 256 x 256 tiles; a single row-tile of tokens runs on the one-CTA kernel
  const bool ws_holds_copy = workspace != nullptr && wl.xs_bytes > 0 && workspace_bytes >= wl.total;
  if (variant == RL_VARIANT_AUTO) variant = auto_variant(M, N, K, g != nullptr, workspace != nullptr, ws_holds_copy, di.sms);
  const bool split_tail = !auto_whole && (variant != RL_VARIANT_PREFILL_PAIR_PRESTATS_WHOLE);
  PairArgs pa;
  pa.x = x; pa.gamma = g; pa.W = W; pa.y = y;
  pa.M = M; pa.N = N; pa.K = K; pa.ldx = ldx; pa.ldw = ldw; pa.ldy = ldy; pa.eps = eps;
  pa.status = status; pa.ws_bytes = workspace_bytes; pa.tail_off = wl.tail_off; pa.ws_total = wl.tail_total; pa.sync_off = wl.sync_off;
  pa.sms = di.sms; pa.st = st; pa.split_tail = split_tail;
#define RL_PREFILL(BN, ST, AM, TG) \
  launch_prefill<PrefillCfg<BN, ST, AM, TG>>(x, g, W, y, M, N, K, ldx, ldw, ldy, eps, status, di.sms, st)
  switch (variant) {
    case RL_VARIANT_PREFILL_TS_N192: return RL_PREFILL(192, 4, A_TS_FOLD, 2);
    case RL_VARIANT_PREFILL_SS_N192: return g ? RL_PREFILL(192, 4, A_SS_FOLD, 2) : RL_PREFILL(192, 4, A_SS_DIRECT, 2);
    case RL_VARIANT_PREFILL_SS_N256: return g ? RL_PREFILL(256, 4, A_SS_FOLD, 1) : RL_PREFILL(256, 4, A_SS_DIRECT, 1);
    case RL_VARIANT_PREFILL_TS_N128: return RL_PREFILL(128, 4, A_TS_FOLD, 2);
    case RL_VARIANT_PREFILL_SS_N128: return g ? RL_PREFILL(128, 4, A_SS_FOLD, 2) : RL_PREFILL(128, 4, A_SS_DIRECT, 2);
    case RL_VARIANT_PREFILL_PAIR_N256: return launch_prefill_pair<PairFoldFused>(pa);
    case RL_VARIANT_PREFILL_PAIR_N192: return launch_prefill_pair<PairFoldN192>(pa);
    case RL_VARIANT_PREFILL_PAIR_DIRECT: return launch_prefill_pair<PairDirectFused>(pa);
    case RL_VARIANT_PREFILL_PAIR_PRESTATS:
    case RL_VARIANT_PREFILL_PAIR_PRESTATS_WHOLE: return launch_prefill_pair<PairFold>(pa);
    case RL_VARIANT_PREFILL_PAIR_DIRECT_PRESTATS: return launch_prefill_pair<PairDirect>(pa);
    case RL_VARIANT_PREFILL_PAIR_WIDE:
    case RL_VARIANT_PREFILL_PAIR_PRESCALED: {
      // any width when asked for by name; the workspace must hold the copy (rl_workspace_bytes sizes it for wide layers only)
      const bool by_name_wide = (variant == RL_VARIANT_PREFILL_PAIR_WIDE);
      if (workspace == nullptr || (g == nullptr && !by_name_wide)) return RL_ERR_BAD_VARIANT;
      if (g != nullptr) {
        const size_t copy_bytes = align_up((size_t)M * (size_t)K * 2, 256);
        if (workspace_bytes < wl.xs_off + copy_bytes) return RL_ERR_WORKSPACE;
        pa.xs = reinterpret_cast<uint8_t*>(workspace) + wl.xs_off;
      }
      return by_name_wide ? launch_prefill_pair<PairWide>(pa) : launch_prefill_pair<PairDirect>(pa);
    }
    default: return RL_ERR_BAD_VARIANT;
  }
#undef RL_PREFILL
}

int rl_quantize_rows_e4m3(const void* x, const void* gamma, void* q, float* row_scale, int M, int K, int64_t ldx,
                          int64_t ldq, float eps, void* stream) {
  if (!x || !q || !row_scale) return RL_ERR_NULL_POINTER;
  if (M <= 0 || K <= 0 || ldx < K || ldq < K) return RL_ERR_BAD_SHAPE;
  if ((K & 7) || (ldx & 7) || (ldq & 7) || !aligned16(x) || !aligned16(q) || (gamma && !aligned16(gamma)))
    return RL_ERR_ALIGNMENT;
  return launch_rowquant(x, gamma, q, row_scale, M, K, ldx, ldq, eps, (cudaStream_t)stream);
}

int rl_row_stats(const void* x, const void* gamma, float* inv_rms, float* amax, int M, int K, int64_t ldx, float eps,
                 void* stream) {
  if (!x || !inv_rms) return RL_ERR_NULL_POINTER;
  if (M <= 0 || K <= 0 || ldx < K) return RL_ERR_BAD_SHAPE;
  if ((K & 7) || (ldx & 7) || !aligned16(x) || (gamma && !aligned16(gamma))) return RL_ERR_ALIGNMENT;
  rowstats_amax_kernel<<<M, 128, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                            reinterpret_cast<const __nv_bfloat16*>(gamma), inv_rms, amax, M,
                                                            K, ldx, eps);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? RL_OK : cuda_err(e);
}

int rl_rmsnorm_linear_fp8w(const void* x, const void* gamma, const void* Wq, const float* w_scale, void* y, int M, int N,
                           int K, int64_t ldx, int64_t ldw, int64_t ldy, float eps, void* workspace,
                           size_t workspace_bytes, int variant, void* stream) {
  if (!x || !Wq || !w_scale || !y) return RL_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || ldy < N) return RL_ERR_BAD_SHAPE;
  if ((K & 15) || (ldx & 7) || (ldw & 15) || (ldy & 7) || !aligned16(x) || !aligned16(Wq) || !aligned16(y) ||
      (gamma && !aligned16(gamma)))
    return RL_ERR_ALIGNMENT;
  if (variant != RL_VARIANT_AUTO && variant != RL_VARIANT_AUTO_WHOLE) return RL_ERR_BAD_VARIANT;
  const Fp8WsLayout wl = fp8_ws_layout(M, K);
  // M <= 64 runs the stream-K kernel, whose partial tiles live where the large-M kernel keeps its k-split blocks
  if (!workspace || workspace_bytes < (M <= 64 ? wl.total : wl.min_total)) return RL_ERR_WORKSPACE;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (di.cc_major != 10) return RL_ERR_UNSUPPORTED_ARCH;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  float* row_scale = reinterpret_cast<float*>(ws + wl.row_scale_off);
  uint8_t* xq = ws + wl.xq_off;
  if ((rc = launch_rowquant(x, gamma, xq, row_scale, M, K, ldx, K, eps, st))) return rc;
  if (M <= 64) {
    // small M: memory bound on the weights, which e4m3 halves.  The operand-swapped stream-K kernel on the
    // quantised activations; its counters sit in the region every layout keeps at the same place.
    WsLayout dl{};
    dl.counters_off = STATUS_BYTES;
    dl.ssq_off = wl.row_scale_off;      // not used by the FP8 configuration
    dl.partials_off = wl.tail_off;
    static_assert(TAIL_BYTES >= (size_t)RL_MAX_CTAS * 2 * 64 * 128 * 4, "the k-split region holds the stream-K partial tiles");
    if (M <= 16)
      return launch_decode<DecodeCfg<16, RL_DEC16_STAGES, RL_DEC16_TW, RL_DEC16_MINB, true>>(
          xq, nullptr, Wq, y, M, N, K, K, ldw, ldy, eps, ws, dl, di.sms, st, row_scale, w_scale);
    if (M <= 32)
      return launch_decode<DecodeCfg<32, 8, 4, 1, true>>(xq, nullptr, Wq, y, M, N, K, K, ldw, ldy, eps, ws, dl, di.sms, st,
                                                         row_scale, w_scale);
    return launch_decode<DecodeCfg<64, 8, 4, 1, true>>(xq, nullptr, Wq, y, M, N, K, K, ldw, ldy, eps, ws, dl, di.sms, st,
                                                       row_scale, w_scale);
  }
  PairArgs pa;
  pa.x = xq; pa.W = Wq; pa.y = y;
  pa.M = M; pa.N = N; pa.K = K; pa.ldx = K; pa.ldw = ldw; pa.ldy = ldy; pa.eps = eps;
  pa.status = reinterpret_cast<int*>(ws); pa.ws_bytes = workspace_bytes; pa.tail_off = wl.tail_off; pa.ws_total = wl.total;
  pa.sms = di.sms; pa.st = st;
  pa.split_tail = (variant != RL_VARIANT_AUTO_WHOLE);
  pa.row_scale = row_scale; pa.w_scale = w_scale;
  return launch_prefill_pair<PairFp8>(pa);
}

int rl_rmsnorm_linear_bf16_noalloc(const void* x, const void* gamma, const void* W, void* y, int M, int N, int K,
                                   int64_t ldx, int64_t ldw, int64_t ldy, float eps, void* stream) {
  if (!x || !W || !y) return RL_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || ldy < N) return RL_ERR_BAD_SHAPE;
  if ((K & 7) || (ldx & 7) || (ldw & 7) || !aligned16(x) || !aligned16(W) || (gamma && !aligned16(gamma)))
    return RL_ERR_ALIGNMENT;
  // the built-in scratch is sized for the 16-token configuration of the small-M kernel
  if (M > 16) return RL_ERR_STATIC_SCRATCH;
  const WsLayout wl = ws_layout(M, N);
  if (wl.total > RL_STATIC_SCRATCH_BYTES) return RL_ERR_STATIC_SCRATCH;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (di.cc_major != 10) return RL_ERR_UNSUPPORTED_ARCH;
  uint8_t* scratch = nullptr;
  if ((rc = static_scratch_address(&scratch))) return rc;  // first call on a device resolves the symbol
  cudaStream_t st = (cudaStream_t)stream;
  // The array keeps whatever the previous call left.  The status block and the tile counters must start
  // at zero; partial tiles are always written before they are read and need no clearing.
  cudaError_t e = cudaMemsetAsync(scratch, 0, wl.ssq_off, st);
  if (e != cudaSuccess) return cuda_err(e);
  return launch_decode<DecodeCfg16>(x, reinterpret_cast<const __nv_bfloat16*>(gamma), W, y, M, N, K, ldx, ldw,
                                          ldy, eps, scratch, wl, di.sms, st);
}

int rl_rmsnorm_swiglu_bf16(const void* x, const void* gamma, const void* W, void* y, int M, int N, int K, int64_t ldx,
                           int64_t ldw, int64_t ldy, float eps, void* workspace, size_t workspace_bytes,
                           void* stream) {
  if (!x || !W || !y) return RL_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || ldy < N) return RL_ERR_BAD_SHAPE;
  // a tile pairs 128 gate rows with 128 up rows: N a multiple of 128 keeps a tile from straddling the two halves
  if ((K & 7) || (ldx & 7) || (ldw & 7) || (ldy & 7) || (N & 127) || !aligned16(x) || !aligned16(W) || !aligned16(y) ||
      (gamma && !aligned16(gamma)))
    return RL_ERR_ALIGNMENT;
  // the layout of a linear layer with the same 2N weight rows: wide layers get room for the gamma-folded copy of x
  const WsLayout wl = ws_layout(65 > M ? 65 : M, 2 * N, K);
  if (!workspace || workspace_bytes < wl.min_total) return RL_ERR_WORKSPACE;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (di.cc_major != 10) return RL_ERR_UNSUPPORTED_ARCH;
  PairArgs pa;
  pa.x = x; pa.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma); pa.W = W; pa.y = y;
  pa.M = M; pa.N = N; pa.K = K; pa.ldx = ldx; pa.ldw = ldw; pa.ldy = ldy; pa.eps = eps;
  pa.status = reinterpret_cast<int*>(workspace); pa.ws_bytes = workspace_bytes; pa.sync_off = wl.sync_off;
  pa.sms = di.sms; pa.st = (cudaStream_t)stream;
  // without gamma there is nothing to fold: x straight from shared memory.  With gamma the same kernel runs on the
  // copy the pre-pass folds it into, where the layer is wide enough to pay for the copy and the workspace holds it.
  const bool folded_copy = gamma != nullptr && wl.xs_bytes > 0 && workspace_bytes >= wl.total;
  if (gamma != nullptr && !folded_copy) return launch_prefill_pair<PairSwiglu>(pa);
  if (folded_copy) pa.xs = reinterpret_cast<uint8_t*>(workspace) + wl.xs_off;
  // 256 x 512 tiles where their whole rounds (neither width cuts its last round here) cost clearly less
  int pairs = 0;
  if (K >= 4096 && max_cta_pairs<PairSwigluWide>(di.sms, &pairs) == RL_OK && pairs > 0) {
    const long long m_tiles = (M + 255) / 256;
    const long long t_wide = m_tiles * ((N + 255) / 256), t_narrow = m_tiles * ((N + 127) / 128);
    const long long r_wide = (t_wide + pairs - 1) / pairs, r_narrow = (t_narrow + pairs - 1) / pairs;
    if (t_wide >= 3LL * pairs && 2.0 * 0.93 * (double)r_wide < 0.98 * (double)r_narrow)
      return launch_prefill_pair<PairSwigluWide>(pa);
  }
  return launch_prefill_pair<PairSwigluDirect>(pa);
}

int rl_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                 void* workspace, size_t workspace_bytes, void* stream) {
  if (!A || !B || !C) return RL_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < K || ldc < N) return RL_ERR_BAD_SHAPE;
  if ((K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7) || !aligned16(A) || !aligned16(B) || !aligned16(C))
    return RL_ERR_ALIGNMENT;
  if (workspace && workspace_bytes < STATUS_BYTES) return RL_ERR_WORKSPACE;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (di.cc_major != 10) return RL_ERR_UNSUPPORTED_ARCH;
  const WsLayout wl = ws_layout(M > 65 ? M : 65, N);
  PairArgs pa;
  pa.x = A; pa.W = B; pa.y = C;
  pa.M = M; pa.N = N; pa.K = K; pa.ldx = lda; pa.ldw = ldb; pa.ldy = ldc;
  pa.status = reinterpret_cast<int*>(workspace); pa.ws_bytes = workspace_bytes; pa.tail_off = wl.tail_off; pa.ws_total = wl.total; pa.sync_off = wl.sync_off;
  pa.sms = di.sms; pa.st = (cudaStream_t)stream;
  pa.no_norm = true;
  int wide_pairs = 0;
  if (max_cta_pairs<PairWide>(di.sms, &wide_pairs) == RL_OK && wide_tiles_pay(M, N, K, wide_pairs))
    return launch_prefill_pair<PairWide>(pa);
  return launch_prefill_pair<PairDirect>(pa);
}

int rl_lora_linear_bf16(const void* a, const void* b, const void* xa, const void* lb, void* y, int M, int N, int K, int L,
                        int64_t lda, int64_t ldb, int64_t ldxa, int64_t ldlb, int64_t ldy, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (!a || !b || !xa || !lb || !y) return RL_ERR_NULL_POINTER;
  if (M <= 0 || N <= 0 || K <= 0 || L <= 0 || L > 64 || lda < K || ldb < K || ldxa < L || ldlb < L || ldy < N)
    return RL_ERR_BAD_SHAPE;
  if ((K & 7) || (L & 7) || (lda & 7) || (ldb & 7) || (ldxa & 7) || (ldlb & 7) || (ldy & 7) || !aligned16(a) ||
      !aligned16(b) || !aligned16(xa) || !aligned16(lb) || !aligned16(y))
    return RL_ERR_ALIGNMENT;
  if (workspace && workspace_bytes < STATUS_BYTES) return RL_ERR_WORKSPACE;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc) return rc;
  if (di.cc_major != 10) return RL_ERR_UNSUPPORTED_ARCH;
  const WsLayout wl = ws_layout(M > 65 ? M : 65, N);
  PairArgs pa;
  pa.x = a; pa.W = b; pa.y = y;
  pa.M = M; pa.N = N; pa.K = K; pa.ldx = lda; pa.ldw = ldb; pa.ldy = ldy;
  pa.status = reinterpret_cast<int*>(workspace); pa.ws_bytes = workspace_bytes; pa.tail_off = wl.tail_off; pa.ws_total = wl.total; pa.sync_off = wl.sync_off;
  pa.sms = di.sms; pa.st = (cudaStream_t)stream;
  pa.no_norm = true;
  pa.x2 = xa; pa.w2 = lb; pa.L = L; pa.ldx2 = ldxa; pa.ldw2 = ldlb;
  return launch_prefill_pair<PairDirect>(pa);
}

int rl_selftest_wait_timeout(void* workspace, size_t workspace_bytes, unsigned long long limit_ns, void* stream) {
  if (!workspace) return RL_ERR_NULL_POINTER;
  if (workspace_bytes < STATUS_BYTES) return RL_ERR_WORKSPACE;
  if (limit_ns == 0 || limit_ns > 1000000000ull) return RL_ERR_BAD_SHAPE;  // keep the self-test short
  wait_timeout_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(reinterpret_cast<int*>(workspace), limit_ns);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? RL_OK : cuda_err(e);
}

int rl_read_status(const void* workspace, int* detail) {
  if (!workspace) return RL_ERR_NULL_POINTER;
  int h[8] = {0};
  cudaError_t e = cudaMemcpy(h, workspace, sizeof(h), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_err(e);
  if (detail)
    for (int i = 0; i < 8; ++i) detail[i] = h[i];
  return h[0] == 0 ? RL_OK : RL_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
