/* C ABI of librmsnorm_linear: fused RMSNorm -> Linear on NVIDIA B200 (sm_100a).
 *
 *     y[m, n] = rsqrt(mean_k x[m,k]^2 + eps) * sum_k x[m,k] * gamma[k] * W[n,k]
 *
 * Every entry point takes plain pointers and sizes; device pointers belong to
 * the caller, and every launch is asynchronous on the stream that is passed in.
 * The library never calls an allocator and keeps no pointer of the caller's; the
 * one piece of device memory it owns is the fixed 3 MiB scratch array of
 * rl_rmsnorm_linear_bf16_noalloc, which is part of the library's device image
 * (see that function).  All functions return 0 on success or a negative RL_ERR_*
 * code; nothing throws.
 *
 * Concurrency.  Calls on one stream may follow each other freely.  The large-M
 * kernels that cut the tiles of a partly filled last round along K
 * (rl_plan_tail_split) make CTA pairs of one launch wait for each other through
 * the workspace, which relies on the whole grid being resident: keep at most
 * one such launch in flight per device, or pass RL_VARIANT_AUTO_WHOLE on the
 * streams that run concurrently - the same choice of kernels with every tile
 * computed whole and no CTA waiting for another.  Two such launches sharing
 * the SMs can starve each other; each then gives up after its wait limit (2 s)
 * with RL_ERR_DEVICE_TIMEOUT in the status block, its output is wrong, and the
 * workspace must be cleared with rl_workspace_init before it is used again.
 *
 * Each function names the interface of the reference project
 * (dungwoong/kernel-benchmarking) that it stands in for.
 */
#ifndef RMSNORM_LINEAR_H_
#define RMSNORM_LINEAR_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  RL_OK = 0,
  RL_ERR_NULL_POINTER = -1,     /* a required pointer is NULL */
  RL_ERR_BAD_SHAPE = -2,        /* M, N or K <= 0, or a leading dimension smaller than the row */
  RL_ERR_ALIGNMENT = -3,        /* K or a leading dimension not a multiple of 8 (16 for e4m3) elements, or a pointer not 16-byte aligned */
  RL_ERR_BAD_DTYPE = -4,        /* unknown weight dtype code */
  RL_ERR_WORKSPACE = -5,        /* workspace missing or smaller than rl_workspace_bytes() */
  RL_ERR_UNSUPPORTED_ARCH = -6, /* current device is not compute capability 10.x */
  RL_ERR_BAD_VARIANT = -7,      /* unknown kernel variant, or one that cannot run this shape */
  RL_ERR_TENSOR_MAP = -8,       /* the driver rejected a TMA descriptor */
  RL_ERR_DEVICE_TIMEOUT = -9,   /* a bounded wait inside a kernel ran out (reported by rl_read_status) */
  RL_ERR_STATIC_SCRATCH = -10,  /* rl_rmsnorm_linear_bf16_noalloc: the shape needs more scratch than the built-in buffer */
  RL_ERR_CUDA = -1000           /* RL_ERR_CUDA - cudaError_t of the failing runtime call */
};

/* weight dtype codes */
enum { RL_W_BF16 = 0, RL_W_E4M3 = 1 };

/* kernel variants (0 picks by shape) */
enum {
  RL_VARIANT_AUTO = 0,
  RL_VARIANT_PREFILL_TS_N192 = 1,  /* gamma-folded activations handed to the MMA through tensor memory */
  RL_VARIANT_PREFILL_SS_N192 = 2,  /* gamma folded in place in shared memory */
  RL_VARIANT_PREFILL_SS_N256 = 3,
  RL_VARIANT_PREFILL_TS_N128 = 4,
  RL_VARIANT_PREFILL_SS_N128 = 5,
  RL_VARIANT_PREFILL_PAIR_N256 = 9,   /* CTA pairs (cta_group::2): 256 x 256 tiles, A operand through tensor memory */
  RL_VARIANT_PREFILL_PAIR_N192 = 10,  /* CTA pairs: 256 x 192 tiles, two accumulators (epilogue overlaps the next tile) */
  RL_VARIANT_PREFILL_PAIR_PRESTATS = 14, /* CTA pairs, 256 x 256: 1/rms per token from a row-statistics pre-pass (needs a workspace);
                                            the tiles of a partly filled last round are split along K across the idle pairs */
  RL_VARIANT_PREFILL_PAIR_PRESTATS_WHOLE = 15, /* as 14, every tile computed whole by one pair */
  RL_VARIANT_PREFILL_PAIR_DIRECT_PRESTATS = 16, /* gamma == NULL only: 1/rms from the pre-pass, x straight from shared memory, two accumulators */
  RL_VARIANT_PREFILL_PAIR_PRESCALED = 17, /* gamma != NULL: the pre-pass also writes bf16(x * gamma) into the workspace and the GEMM runs as 16
                                           on that copy; what AUTO runs for N >= 6144 and M * N * K >= 3e10 when the workspace holds the copy
                                           (rl_workspace_bytes counts it for such shapes); by name for any shape, with M * K * 2 + 256
                                           bytes added to rl_workspace_bytes */
  RL_VARIANT_PREFILL_PAIR_WIDE = 18,     /* as 16 (gamma == NULL) or 17 (gamma != NULL) on 256 x 512 tiles: every pair reads half the
                                           activation bytes per FLOP; last round cut along K like 14's.  What AUTO runs in place of 16 / 17
                                           for K >= 4096 when the 512-column tiles' rounds cost less than the 256-column tiles' */
  RL_VARIANT_PREFILL_PAIR_DIRECT = 11, /* CTA pairs, gamma == NULL only: x straight from shared memory, 256 x 256, two accumulators */
  RL_VARIANT_DECODE = 20,          /* M <= 64: operand-swapped, stream-K over (channel tile, k block) units */
  RL_VARIANT_AUTO_WHOLE = 30       /* as AUTO, but never a kernel whose CTAs wait for one another (no k-split last round, no
                                      alignment of the CTA pairs at tile boundaries): for callers that keep several launches
                                      in flight on one device */
};

/* Library version (major * 1000 + minor).  No reference counterpart. */
int rl_version(void);

/* Text for an RL_ERR_* code.  Stands in for the exception text of the
 * reference's native extension (third_party/cublas_gemm/python/ext_kernel.cu:10-22). */
const char* rl_error_string(int code);

/* Bytes of caller-provided workspace a call with this shape needs (status
 * block; for M <= 64 the split-K partial tiles and tile counters; for M > 64
 * 1/rms per token, the partial blocks of k-split tiles and, with bf16 weights
 * N >= 6144 and M * N * K >= 3e10, M * K * 2 bytes for the gamma-folded copy of x - a call
 * given less than that still runs, folding gamma in the main loop).  Pure
 * arithmetic, needs no GPU.  No reference counterpart (the reference's kernels
 * allocate through their DSL runtimes). */
size_t rl_workspace_bytes(int M, int N, int K, int w_dtype);

/* How the M > 128 pre-pass kernels treat the last, partly filled round of 256 x 256 tiles on `pairs` CTA pairs
 * (74 on a B200): *tail_tiles tiles are each cut along K into *split (2, 3 or 4) slices computed by different pairs
 * and summed in slice order; 0 / 0 = every tile computed whole.  Pure arithmetic, needs no GPU.  No reference
 * counterpart (its kernels leave scheduling to their DSL compilers). */
int rl_plan_tail_split(int M, int N, int K, int pairs, int* tail_tiles, int* split);

/* The variant RL_VARIANT_AUTO runs for a bf16 call of this shape on the current device (it asks the device for its
 * SM count and CTA-pair occupancy, so it needs a GPU); a negative RL_ERR_* code on failure.  Lets a benchmark label
 * its numbers with the kernel that ran.  No reference counterpart (the reference's kernels are picked by name in
 * its `kernels` dict, demo/new_profiling/rmsnorm_linear_new.py:97-103). */
int rl_select_variant(int M, int N, int K, int has_gamma, int has_workspace);

/* Zero the workspace (status block and tile counters) on `stream`.  Must run
 * once before the first use of a workspace; kernels leave it clean afterwards. */
int rl_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* bf16 fused RMSNorm -> Linear.
 *   x [M, K] bf16 row-major (leading dimension ldx elements), gamma [K] bf16 or
 *   NULL (= ones, the reference's semantics), W [N, K] bf16 row-major (ldw),
 *   y [M, N] bf16 row-major (ldy), fp32 accumulation.
 * Replaces, for this path, the reference's kernel callables
 *   torch_kernel(a, b, eps)                      demo/rmsnorm_linear.py:36-38
 *   baselines.rmsnorm_linear(a, b, eps)          python/baselines/rmsnorm_swiglu.py:28-34
 *   rmsnorm_lin_kernel(x, y, eps)                python/bench_kernels/helion/rmsnorm_linear.py:5-35
 *   rmsnorm_matmul_persistent(X, W, eps, ...)    python/bench_kernels/tilelang/tilelang_rmsnorm_linear.py:7-87
 *   compiled_gemm(a, b, o, eps)                  demo/rmsnorm_linear.py:65-68
 * `workspace` may be NULL for M > 64 (then device-side timeouts go unreported). */
int rl_rmsnorm_linear_bf16(const void* x, const void* gamma, const void* W, void* y,
                           int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy,
                           float eps, void* workspace, size_t workspace_bytes,
                           int variant, void* stream);

/* FP8-weight fused RMSNorm -> Linear (quantised-inference path).
 *   x [M, K] bf16, gamma [K] bf16 or NULL, Wq [N, K] e4m3 codes row-major (ldw bytes = elements),
 *   w_scale [N] fp32 per-output-channel scales (W = Wq * w_scale[n]), y [M, N] bf16.
 *   The normalised activations are quantised to e4m3 per token on the device:
 *   q = e4m3(x * gamma * 448 / amax_m); y = (q @ Wq^T) * rsqrt(mean x^2 + eps) * amax_m / 448 * w_scale[n].
 *   K and ldw must be multiples of 16.  The workspace (rl_workspace_bytes with RL_W_E4M3) holds
 *   the quantised activations, the per-token scales and the partial blocks of a k-split last round.
 *   M <= 64 (memory bound on the weights, which e4m3 halves) runs the operand-swapped stream-K kernel on the
 *   quantised activations; larger M the CTA-pair kernel.
 *   `variant`: RL_VARIANT_AUTO or RL_VARIANT_AUTO_WHOLE.
 * No reference counterpart: the reference project has no quantised path; the operator semantics
 * are those of rl_rmsnorm_linear_bf16 applied to the dequantised weights. */
int rl_rmsnorm_linear_fp8w(const void* x, const void* gamma, const void* Wq, const float* w_scale, void* y,
                           int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy,
                           float eps, void* workspace, size_t workspace_bytes,
                           int variant, void* stream);

/* Per-token statistics on their own: inv_rms[m] = rsqrt(mean_k x[m,k]^2 + eps) and, unless amax is NULL,
 * amax[m] = max_k |x[m,k] * gamma[k]| (gamma NULL = ones).  These are what the fused kernels derive their
 * epilogue scale (bf16 path) and their per-token quantisation step (FP8 path) from; the reference computes the
 * first inside `F.rms_norm` (python/baselines/rmsnorm_swiglu.py:26) and has no counterpart for the second. */
int rl_row_stats(const void* x, const void* gamma, float* inv_rms, float* amax,
                 int M, int K, int64_t ldx, float eps, void* stream);

/* The first kernel of the FP8 path on its own: per row, q = e4m3(x * gamma * 448 / amax) into
 * q [M, ldq] and row_scale[m] = rsqrt(mean x^2 + eps) * amax / 448.  No reference counterpart. */
int rl_quantize_rows_e4m3(const void* x, const void* gamma, void* q, float* row_scale,
                          int M, int K, int64_t ldx, int64_t ldq, float eps, void* stream);

/* The small-M kernel for callers that cannot allocate.
 *
 * rl_rmsnorm_linear_bf16 needs a caller-provided workspace for M <= 64, which means the caller
 * must be able to obtain device memory.  Some callers cannot: a plug-in that is handed raw input and
 * output pointers by a host engine which has already claimed all device memory for its own arena; a
 * component that is forbidden to touch the CUDA allocator because cudaMalloc / cudaFree synchronise
 * the whole device and would stall the engine's other streams; a bare C caller with no allocator at
 * hand.  For them this entry point takes only inputs and outputs and keeps its scratch (status block,
 * tile counters, split-K partial tiles) in a 3 MiB array that is part of the library's device image.
 * It calls no cudaMalloc, cudaFree or allocating library routine.
 *
 *   - Limit: M <= 16 tokens (any N and K the small-M kernel accepts); larger M returns
 *     RL_ERR_STATIC_SCRATCH.  The 3 MiB stay resident on every GPU that loads the library until exit.
 *     They are claimed when the CUDA runtime loads the library's device image on that GPU, which with
 *     lazy loading can be inside the first call: on a device with no memory left that call returns
 *     RL_ERR_CUDA - cudaErrorMemoryAllocation.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
 *     should therefore be made, once per device, before any stream capture begins.
 *   - All calls on a device share the one array: two calls whose kernels overlap on the GPU (different
 *     streams, or different host threads on different streams) race on it.  Serialise them on one
 *     stream.  The part that must start from zero is cleared on `stream` before every launch.
 *   - Arguments and results are those of rl_rmsnorm_linear_bf16; device-side timeouts are recorded in
 *     the internal array and are not retrievable through rl_read_status.
 * This function has no counterpart in the reference project. */
int rl_rmsnorm_linear_bf16_noalloc(const void* x, const void* gamma, const void* W, void* y,
                                   int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy,
                                   float eps, void* stream);

/* Fused RMSNorm -> SwiGLU: y[M, N] = silu(h[:, :N]) * h[:, N:] with h = rmsnorm(x) * gamma @ W^T, W [2N, K] =
 * gate rows followed by up rows.  Replaces `rmsnorm_swiglu(a, bb1, eps)`
 * (python/baselines/rmsnorm_swiglu.py:36-42, profiled by demo/new_profiling/swiglu_new.py).  N must be a
 * multiple of 128; needs a workspace of rl_workspace_bytes(max(M, 65), 2 * N, K, RL_W_BF16) bytes (the size for a
 * linear layer with the same 2N weight rows; with no more than rl_workspace_bytes(max(M, 65), N, K, RL_W_BF16)
 * the call still runs, folding gamma in the main loop). */
int rl_rmsnorm_swiglu_bf16(const void* x, const void* gamma, const void* W, void* y, int M, int N, int K,
                           int64_t ldx, int64_t ldw, int64_t ldy, float eps,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Plain bf16 GEMM C[M, N] = A[M, K] . B[N, K]^T (fp32 accumulation) on the same CTA-pair machinery with
 * the norm switched off: the "max" line the reference times beside every fused kernel
 * (`torch_gemm`, demo/new_profiling/rmsnorm_linear_new.py:29-31; native form
 * third_party/cublas_gemm/python/ext_kernel.cu:30-53).  `workspace` (>= 256 bytes) may be NULL. */
int rl_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                 int64_t lda, int64_t ldb, int64_t ldc, void* workspace, size_t workspace_bytes, void* stream);

/* LoRA-fused linear: y[M, N] = a[M, K] . b[N, K]^T + xa[M, L] . lb[N, L]^T in one pass (fp32 accumulation, one
 * bf16 rounding), with xa = a . lA^T computed beforehand (rl_gemm_bf16 does) as the reference's fused kernels
 * take it (`compiled_gemm(a_, b_, lxa, lB_, o)`, demo/new_profiling/lora_new.py:46-50; semantics `torch_lora`,
 * python/baselines/lora.py:4-13).  The low-rank term rides as one more k-block of the main loop.
 * L <= 64 and a multiple of 8; all leading dimensions multiples of 8. */
int rl_lora_linear_bf16(const void* a, const void* b, const void* xa, const void* lb, void* y,
                        int M, int N, int K, int L,
                        int64_t lda, int64_t ldb, int64_t ldxa, int64_t ldlb, int64_t ldy,
                        void* workspace, size_t workspace_bytes, void* stream);

/* Self-test of the kernels' failure detection.  Launches one small CTA that waits on a barrier nothing
 * ever arrives on, with the given limit (<= 1 s); the wait must give up, record RL_ERR_DEVICE_TIMEOUT
 * in the workspace's status block (role 9) and return, leaving the context usable.  Afterwards
 * rl_read_status reports the timeout; rl_workspace_init clears it.  No reference counterpart (the
 * reference has no failure handling; its native code exits on a CUDA error,
 * third_party/cublas_gemm/cublas_gemm.cu:17-29). */
int rl_selftest_wait_timeout(void* workspace, size_t workspace_bytes, unsigned long long limit_ns, void* stream);

/* Read the status block of a workspace (synchronises the stream's device: use
 * outside the hot loop).  Returns RL_OK or RL_ERR_DEVICE_TIMEOUT; when `detail`
 * is not NULL it receives 8 ints: code, role, barrier, block, index, parity, 0, 0.
 * Stands in for the reference's CUDA_CHECK after a launch
 * (third_party/cublas_gemm/cublas_gemm.cu:17-29). */
int rl_read_status(const void* workspace, int* detail);

#ifdef __cplusplus
}
#endif
#endif /* RMSNORM_LINEAR_H_ */
