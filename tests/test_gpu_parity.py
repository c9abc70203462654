"""Parity of the CUDA kernels (called through the C ABI) with the CPU oracle and the golden vectors.

Tolerances (max|y - y_ref| / max|y_ref|, y_ref = the reference's torch path on the widened inputs):
bf16 path <= 1e-2.  Everything here needs a B200 and the compiled library.
"""
import os

import numpy as np
import pytest
import torch

import kernel_benchmarking_b200 as kb
from kernel_benchmarking_b200 import _lib
from oracle import rmsnorm_linear_oracle as orc

pytestmark = pytest.mark.gpu
BF16_TOL = 1e-2
ONE_ULP = 2.0 ** -7   # largest step between neighbouring bf16 values, relative to the value
DEV = "cuda:0"


def bf16(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def run(x, g, W, eps, **kw):
    y = kb.rmsnorm_linear(x.to(DEV), None if g is None else g.to(DEV), W.to(DEV), eps, **kw)
    torch.cuda.synchronize()
    kb.check_status()
    return y.cpu()


def test_library_is_loaded_native():
    lib = _lib.load()
    assert lib.rl_version() >= 1000
    assert os.path.exists(os.path.join(os.path.dirname(kb.__file__), "librmsnorm_linear.so"))


@pytest.mark.parametrize("name,has_gamma", [("bf16_outliers_128x256x128.npz", False), ("bf16_gamma_67x136x192.npz", True)])
def test_golden_vectors(golden_dir, name, has_gamma):
    g = np.load(os.path.join(golden_dir, name))
    x, W, eps = bf16(g["x_bits"]), bf16(g["W_bits"]), float(g["eps"])
    gm = bf16(g["gamma_bits"]) if has_gamma else None
    ref = torch.from_numpy(g["y_ref_fp64"])
    assert orc.rel_max_err(run(x, gm, W, eps), ref) <= BF16_TOL
    # the same vectors through the small-M kernel: first 16 / 64 rows
    for m in (1, 16, 64):
        assert orc.rel_max_err(run(x[:m].contiguous(), gm, W, eps), ref[:m]) <= BF16_TOL


SHAPES = [(M, N, K) for M in (1, 3, 16, 17, 64, 65, 127, 128, 129, 256)
          for (N, K) in ((8, 64), (128, 128), (136, 64), (256, 320), (520, 128), (1000, 4096))]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("has_gamma", [False, True])
def test_small_and_ragged_shapes(M, N, K, has_gamma):
    x, gm, W = orc.make_inputs(M, N, K, seed=M * 1000 + N + K, gamma=has_gamma)
    eps = 1e-6 if has_gamma else 1e-5
    ref = orc.reference_fp32(x, gm, W, eps)
    y = run(x, gm, W, eps)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert orc.rel_max_err(y, ref) <= BF16_TOL


@pytest.mark.parametrize("variant", ["prefill_ts_n192", "prefill_ss_n192", "prefill_ss_n256", "prefill_ts_n128",
                                     "prefill_ss_n128", "prefill_pair_n256", "prefill_pair_n192",
                                     "prefill_pair_direct", "prefill_pair_prestats", "prefill_pair_direct_prestats",
                                     "prefill_pair_prestats_whole", "prefill_pair_prescaled", "prefill_pair_wide"])
@pytest.mark.parametrize("has_gamma", [False, True])
@pytest.mark.parametrize("M,N,K", [(384, 776, 448), (1100, 2048, 1024)])
def test_every_prefill_variant(variant, has_gamma, M, N, K):
    if variant in ("prefill_pair_direct", "prefill_pair_direct_prestats") and has_gamma:
        with pytest.raises(ValueError):   # those variants read x straight from shared memory: no gamma fold
            x, gm, W = orc.make_inputs(256, 256, 64, gamma=True)
            kb.rmsnorm_linear(x.to(DEV), gm.to(DEV), W.to(DEV), 1e-6, variant=variant)
        return
    if variant == "prefill_pair_prescaled" and not has_gamma:
        with pytest.raises(ValueError):   # the pre-pass folds gamma into a copy of x: nothing to do without one
            x, _, W = orc.make_inputs(256, 256, 64, gamma=False)
            kb.rmsnorm_linear(x.to(DEV), None, W.to(DEV), 1e-6, variant=variant)
        return
    x, gm, W = orc.make_inputs(M, N, K, seed=11, gamma=has_gamma)
    ref = orc.reference_fp32(x, gm, W, 1e-6)
    assert orc.rel_max_err(run(x, gm, W, 1e-6, variant=variant), ref) <= BF16_TOL


def test_reference_outlier_distribution():
    x, _, W = orc.make_inputs_outliers(512, 1024, 2048, seed=18)
    ref = orc.reference_fp32(x, None, W, 1e-5, dtype=torch.float64)
    y = run(x, None, W, 1e-5)
    assert orc.rel_max_err(y, ref) <= BF16_TOL
    rmse, max_abs, max_rel = orc.ref_metrics(ref.float(), y.float())
    # torch's own bf16 path (the reference's "torch" line) has the same order of error
    y_t = orc.torch_rmsnorm_linear(x, None, W, 1e-5)
    rmse_t, _, _ = orc.ref_metrics(ref.float(), y_t.float())
    assert rmse <= 2.0 * rmse_t + 1e-6


def test_output_buffer_is_not_overrun():
    """y is carved out of a larger buffer filled with a sentinel; nothing outside y may change."""
    for (M, N, K) in [(130, 200, 128), (5, 200, 128), (64, 136, 192)]:
        x, gm, W = orc.make_inputs(M, N, K, seed=2)
        big = torch.full((M + 16, N + 56), 7.0, dtype=torch.bfloat16, device=DEV)
        out = big[8:8 + M, 24:24 + N]
        kb.rmsnorm_linear(x.to(DEV), gm.to(DEV), W.to(DEV), 1e-6, out=out)
        torch.cuda.synchronize()
        ref = orc.reference_fp32(x, gm, W, 1e-6)
        assert orc.rel_max_err(out.cpu(), ref) <= BF16_TOL
        mask = torch.ones_like(big, dtype=torch.bool)
        mask[8:8 + M, 24:24 + N] = False
        assert bool((big[mask] == 7.0).all())


def test_non_multiple_of_8_columns():
    x, gm, W = orc.make_inputs(200, 77, 128, seed=4)
    y = run(x, gm, W, 1e-6)
    assert y.shape == (200, 77)
    assert orc.rel_max_err(y, orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL


def test_bad_arguments_raise():
    x, gm, W = orc.make_inputs(16, 64, 64)
    x, gm, W = x.to(DEV), gm.to(DEV), W.to(DEV)
    with pytest.raises(ValueError):
        kb.rmsnorm_linear(x.float(), gm, W)
    with pytest.raises(ValueError):
        kb.rmsnorm_linear(x, gm, W[:, :60].contiguous())
    with pytest.raises(ValueError):
        kb.rmsnorm_linear(x.t().contiguous().t(), gm, W)            # not row-major
    with pytest.raises(ValueError):
        kb.rmsnorm_linear(x[:, :60].contiguous(), gm[:60].contiguous(), W[:, :60].contiguous())  # K % 8 != 0
    assert kb.rmsnorm_linear(x[:0], gm, W).shape == (0, 64)


def _tail_plan(M, N, K, pairs=74):
    import ctypes
    a, b = ctypes.c_int(), ctypes.c_int()
    _lib.check(_lib.load().rl_plan_tail_split(M, N, K, pairs, ctypes.byref(a), ctypes.byref(b)), "rl_plan_tail_split")
    return a.value, b.value


@pytest.mark.parametrize("M,N,K,has_gamma", [
    (512, 1024, 4096, True),     # fewer tiles than CTA pairs: every tile is split in 4
    (300, 520, 2048, False),     # ragged rows and columns, no gamma (the shared-memory operand kernel)
    (2560, 4096, 2056, True),    # two full rounds, then 12 tiles split in 4; the last k-block is partial
    (4096, 4096, 4096, True),    # 3.46 rounds: 34 tail tiles split in 2
    (4096, 1536, 7168, True),    # 1.3 rounds: 22 tail tiles split in 3 (column chunks dealt 1, 1, 2)
    (1024, 2304, 8192, True),    # long K
    (4096, 6144, 4096, False),   # the prefill benchmark shape without gamma
])
def test_tail_tiles_split_along_k(M, N, K, has_gamma):
    """The last, partly filled round of tiles is cut along K across CTA pairs and the partial sums are exchanged
    through the workspace.  Same results as whole tiles to one bf16 ulp, within tolerance of the reference, and
    identical from run to run whichever pair finishes first."""
    tail, split = _tail_plan(M, N, K)
    assert tail > 0 and split in (2, 3, 4)   # on a B200 (74 pairs) these shapes do take the split path
    x, gm, W = orc.make_inputs(M, N, K, seed=M + N + K, gamma=has_gamma)
    ref = orc.reference_fp32(x, gm, W, 1e-6)
    y_split = run(x, gm, W, 1e-6)            # the default path
    y_whole = run(x, gm, W, 1e-6, variant="prefill_pair_prestats_whole")
    assert orc.rel_max_err(y_split, ref) <= BF16_TOL
    assert orc.rel_max_err(y_whole, ref) <= BF16_TOL
    assert orc.rel_max_err(y_split, y_whole.float()) <= ONE_ULP
    for _ in range(3):
        assert torch.equal(run(x, gm, W, 1e-6), y_split)
    # the shared counters are back at zero: a small-M call on the same workspace is undisturbed
    xs, gs, Ws = orc.make_inputs(8, 1024, 512, seed=3)
    assert orc.rel_max_err(run(xs, gs, Ws, 1e-6), orc.reference_fp32(xs, gs, Ws, 1e-6)) <= BF16_TOL


def test_k_split_calls_on_two_streams_at_once():
    """The contributors of a k-split tile wait for each other inside the kernel.  Two streams launching such
    kernels at the same time (each with its own workspace) share the SMs; every call must still complete, with the
    same bits and a clean status."""
    for (M, N, K) in [(4096, 6144, 4096), (512, 1024, 4096)]:
        assert _tail_plan(M, N, K)[1] >= 2
        x, gm, W = orc.make_inputs(M, N, K, seed=21)
        xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
        ref = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
        torch.cuda.synchronize()
        streams = [torch.cuda.Stream(device=DEV), torch.cuda.Stream(device=DEV)]
        for s in streams:
            s.wait_stream(torch.cuda.current_stream())
        outs = []
        for _ in range(6):
            for s in streams:
                with torch.cuda.stream(s):
                    outs.append(kb.rmsnorm_linear(xd, gd, Wd, 1e-6))
        torch.cuda.synchronize()
        kb.check_status()
        assert all(torch.equal(o, ref) for o in outs)


def test_tail_split_in_the_plain_gemm():
    M, N, K = 768, 1280, 4096
    assert _tail_plan(M, N, K)[1] >= 2
    g = torch.Generator().manual_seed(5)
    A = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    B = (torch.randn(N, K, generator=g) * K ** -0.5).bfloat16().to(DEV)
    C = kb.gemm_nt(A, B)
    torch.cuda.synchronize()
    kb.check_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = A.float() @ B.float().t()
    assert orc.rel_max_err(C, ref) <= BF16_TOL
    assert torch.equal(kb.gemm_nt(A, B), C)


def test_deterministic_and_workspace_reuse_across_shapes():
    """Back-to-back launches of different shapes share one workspace; results repeat bit for bit."""
    outs = {}
    for rep in range(2):
        for (M, N, K) in [(4, 28672, 512), (64, 1000, 4096), (16, 384, 256), (300, 520, 320), (1, 28672, 512)]:
            x, gm, W = orc.make_inputs(M, N, K, seed=9)
            y = run(x, gm, W, 1e-6)
            if rep == 0:
                outs[(M, N, K)] = y
                assert orc.rel_max_err(y, orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL
            else:
                assert torch.equal(y, outs[(M, N, K)])


# ---------------------------------------------------------------- benchmark configurations
def _sample_check(x, gm, W, y, eps, rows, tol=BF16_TOL):
    ref = orc.reference_fp32(x[rows], gm, W, eps)
    return orc.rel_max_err(y[rows], ref)


def test_config2_prefill_qkv():
    M, N, K = 4096, 6144, 4096
    x, gm, W = orc.make_inputs(M, N, K, seed=18)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
    torch.cuda.synchronize()
    kb.check_status()
    # full tensor against torch fp32 on the GPU (TF32 off), a row sample against the CPU oracle
    torch.backends.cuda.matmul.allow_tf32 = False
    ref_gpu = orc.reference_fp32(xd, gd, Wd, 1e-6)
    assert orc.rel_max_err(y, ref_gpu) <= BF16_TOL
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(0))[:48]
    assert _sample_check(x, gm, W, y.cpu(), 1e-6, rows) <= BF16_TOL
    # size-independent properties
    y2 = kb.rmsnorm_linear(xd * 4, gd, Wd, 1e-6)                      # rms_norm is scale-invariant (eps aside)
    assert orc.rel_max_err(y2, y.float()) <= 5e-3                     # one bf16 ulp at max|y| is 3.9e-3
    # a column shard reproduces its columns: bit for bit when every tile is computed whole, to one bf16 ulp when
    # the tiles of the last round are summed in k-slices (which tiles those are depends on the shard's tile count)
    n0, n1 = 1536, 3072
    yw = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_prestats_whole")
    assert torch.equal(kb.rmsnorm_linear(xd, gd, Wd[n0:n1], 1e-6, variant="prefill_pair_prestats_whole"), yw[:, n0:n1])
    assert orc.rel_max_err(kb.rmsnorm_linear(xd, gd, Wd[n0:n1], 1e-6), y[:, n0:n1].float()) <= ONE_ULP
    assert orc.rel_max_err(yw, y.float()) <= ONE_ULP
    assert torch.equal(kb.rmsnorm_linear(xd, gd, Wd, 1e-6), y)        # run-to-run identical


@pytest.mark.parametrize("M", [1, 4, 16, 64])
def test_config3_decode(M):
    N, K = 28672, 4096
    x, gm, W = orc.make_inputs(M, N, K, seed=18 + M)
    y = run(x, gm, W, 1e-6)
    ref = orc.reference_fp32(x, gm, W, 1e-6)
    assert orc.rel_max_err(y, ref) <= BF16_TOL
    assert torch.equal(run(x, gm, W, 1e-6), y)
    # the same rows through the large-M kernel agree to bf16 rounding
    xp = torch.zeros(128, K, dtype=torch.bfloat16)
    xp[:M] = x
    yp = run(xp, gm, W, 1e-6, variant="prefill_ts_n192")[:M]
    assert orc.rel_max_err(yp, y.float()) <= 1e-2
    xp2 = torch.zeros(256, K, dtype=torch.bfloat16)
    xp2[:M] = x
    yp = run(xp2, gm, W, 1e-6, variant="prefill_pair_n256")[:M]
    assert orc.rel_max_err(yp, y.float()) <= 1e-2


def test_config4_one_of_eight_shards():
    """16384 x 57344 x 8192 split over 8 ranks: rank 3's shard (7168 channels) at full M and K."""
    M, N, K, G, r = 16384, 57344, 8192, 8, 3
    g = torch.Generator().manual_seed(18)
    x = torch.randn(M, K, generator=g).bfloat16()
    gm = (1 + 0.1 * torch.randn(K, generator=g)).bfloat16()
    Wl = (torch.randn(N // G, K, generator=g) * K ** -0.5).bfloat16()
    xd, gd, Wd = x.to(DEV), gm.to(DEV), Wl.to(DEV)
    y = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
    torch.cuda.synchronize()
    kb.check_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    worst = 0.0
    for m0 in range(0, M, 4096):
        ref = orc.reference_fp32(xd[m0:m0 + 4096], gd, Wd, 1e-6)
        worst = max(worst, orc.rel_max_err(y[m0:m0 + 4096], ref))
    assert worst <= BF16_TOL
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(r))[:16]
    assert _sample_check(x, gm, Wl, y.cpu(), 1e-6, rows) <= BF16_TOL


# ---------------------------------------------------------------- FP8-weight path
FP8_TOL = 3e-2        # at the benchmark's K = 4096
FP8_TOL_SMALL_K = 5e-2  # fewer terms per output average less of the e4m3 rounding noise


def run_fp8(x, g, Wq, w_scale, eps):
    y = kb.rmsnorm_linear(x.to(DEV), None if g is None else g.to(DEV), Wq.to(DEV), eps, w_scale=w_scale.to(DEV))
    torch.cuda.synchronize()
    kb.check_status()
    return y.cpu()


def test_fp8_golden_vector(golden_dir):
    g = np.load(os.path.join(golden_dir, "fp8w_32x64x256.npz"))
    x, gm = bf16(g["x_bits"]), bf16(g["gamma_bits"])
    Wq = torch.from_numpy(g["Wq_codes"]).view(torch.float8_e4m3fn)
    w_scale = torch.from_numpy(g["w_scale"])
    y = run_fp8(x, gm, Wq, w_scale, float(g["eps"]))
    assert orc.rel_max_err(y, torch.from_numpy(g["y_ref_fp64"])) <= FP8_TOL_SMALL_K


@pytest.mark.parametrize("M,K,has_gamma", [(1, 64, True), (37, 256, True), (300, 4096, True), (64, 1024, False)])
def test_row_quantisation_is_bit_exact(M, K, has_gamma):
    """The pre-pass against the oracle's arithmetic: same e4m3 codes, same per-token scale."""
    x, gm, _ = orc.make_inputs(M, 8, K, seed=K + M, gamma=has_gamma)
    q, rs = kb.quantize_rows_e4m3(x.to(DEV), None if gm is None else gm.to(DEV), 1e-6)
    x32 = x.float()
    xg = x32 if gm is None else x32 * gm.float()
    amax = xg.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    qs = torch.full_like(amax, 448.0) / amax          # IEEE division, as on the device
    q_ref = (xg * qs).clamp(-448, 448).to(torch.float8_e4m3fn)
    rs_ref = torch.rsqrt(x32.pow(2).mean(dim=1) + 1e-6) * amax[:, 0] / 448.0
    codes, codes_ref = q.cpu().view(torch.uint8), q_ref.view(torch.uint8)
    same = (codes == codes_ref) | ((codes & 0x7F) == 0) & ((codes_ref & 0x7F) == 0)   # +0 / -0
    # The device's cvt.rn.satfinite and torch's CPU cast may pick different neighbours for a value that
    # sits (to fp32 precision) on a rounding boundary: such codes must be adjacent and very rare.
    if not bool(same.all()):
        d = (codes.int() - codes_ref.int()).abs()[~same]
        assert int(d.max()) <= 1, "a quantised activation is off by more than one e4m3 step"
        assert float((~same).float().mean()) <= 1e-4, f"{int((~same).sum())} of {same.numel()} codes differ"
    torch.testing.assert_close(rs.cpu(), rs_ref, rtol=2e-6, atol=0)


@pytest.mark.parametrize("M,K,has_gamma", [(1, 64, True), (37, 256, False), (300, 4096, True), (4096, 8192, True)])
def test_row_statistics(M, K, has_gamma):
    """inv_rms to fp32 summation order, amax exactly (a product of two bf16 values is exact in fp32)."""
    x, gm, _ = orc.make_inputs(M, 8, K, seed=K + M, gamma=has_gamma)
    inv_rms, amax = kb.row_stats(x.to(DEV), None if gm is None else gm.to(DEV), 1e-6)
    torch.cuda.synchronize()
    x32 = x.float()
    ref_rms = torch.rsqrt(x32.double().pow(2).mean(dim=1) + 1e-6).float()
    ref_amax = (x32 * (gm.float() if gm is not None else 1.0)).abs().amax(dim=1)
    assert torch.allclose(inv_rms.cpu(), ref_rms, rtol=2e-6, atol=0)
    assert torch.equal(amax.cpu(), ref_amax)
    only_rms, none = kb.row_stats(x.to(DEV), None if gm is None else gm.to(DEV), 1e-6, want_amax=False)
    assert none is None and torch.equal(only_rms, inv_rms)


@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (300, 520, 2048), (1000, 1032, 4096), (5, 264, 1024),
                                   (300, 520, 272), (512, 264, 1040), (64, 136, 16)])   # K not a multiple of 128
def test_fp8_shapes(M, N, K):
    x, gm, W = orc.make_inputs(M, N, K, seed=M + N)
    Wq, w_scale = orc.quantize_weight_e4m3(W)
    y = run_fp8(x, gm, Wq, w_scale, 1e-6)
    ref = orc.reference_fp32(x, gm, Wq, 1e-6, w_scale=w_scale)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert orc.rel_max_err(y, ref) <= (FP8_TOL if K >= 4096 else FP8_TOL_SMALL_K)
    # the kernels follow the oracle's arithmetic model to bf16 rounding
    assert orc.rel_max_err(y, orc.fp8_kernel_model(x, gm, Wq, w_scale, 1e-6).float()) <= 1e-2


def test_fp8_strided_operands():
    """x and Wq as column slices of wider buffers (ldx > K, ldw > K), K not a multiple of the 128-element k-block."""
    for (M, N, K) in [(300, 520, 1040), (200, 264, 2048)]:
        x, gm, W = orc.make_inputs(M, N, K, seed=M + K)
        Wq, w_scale = orc.quantize_weight_e4m3(W)
        xb = torch.full((M, K + 64), 3.0, dtype=torch.bfloat16, device=DEV)
        Wb = torch.full((N, K + 128), 1.0, dtype=torch.bfloat16, device=DEV).to(torch.float8_e4m3fn)
        xb[:, :K] = x.to(DEV)
        Wb.view(torch.uint8)[:, :K] = Wq.view(torch.uint8).to(DEV)
        y = kb.rmsnorm_linear(xb[:, :K], gm.to(DEV), Wb[:, :K], 1e-6, w_scale=w_scale.to(DEV))
        torch.cuda.synchronize()
        kb.check_status()
        ref = orc.reference_fp32(x, gm, Wq, 1e-6, w_scale=w_scale)
        assert orc.rel_max_err(y.cpu(), ref) <= (FP8_TOL if K >= 4096 else FP8_TOL_SMALL_K)
        assert orc.rel_max_err(y.cpu(), orc.fp8_kernel_model(x, gm, Wq, w_scale, 1e-6).float()) <= 1e-2


@pytest.mark.parametrize("M,N,K", [(512, 1024, 4096), (2560, 4096, 4096), (8192, 1792, 4096)])
def test_fp8_tail_tiles_split_along_k(M, N, K):
    """The FP8 kernel cuts the tiles of a partly filled last round along K like the bf16 kernel does: same results
    as whole tiles to one bf16 ulp, identical from run to run.  The last shape is one of eight column shards of
    the FP8 benchmark configuration (224 tiles on 74 pairs: two tiles left for a fourth round)."""
    import ctypes
    a, b = ctypes.c_int(), ctypes.c_int()
    _lib.check(_lib.load().rl_plan_tail_split(M, N, K // 2, 74, ctypes.byref(a), ctypes.byref(b)), "plan")  # K/128 k-blocks
    assert a.value > 0 and b.value >= 2
    x, gm, W = orc.make_inputs(M, N, K, seed=M + N)
    Wq, w_scale = orc.quantize_weight_e4m3(W)
    xd, gd, Wqd, wsd = x.to(DEV), gm.to(DEV), Wq.to(DEV), w_scale.to(DEV)
    y = kb.rmsnorm_linear(xd, gd, Wqd, 1e-6, w_scale=wsd)
    yw = kb.rmsnorm_linear(xd, gd, Wqd, 1e-6, w_scale=wsd, variant="auto_whole")
    torch.cuda.synchronize()
    kb.check_status()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:32]
    ref = orc.reference_fp32(x[rows], gm, Wq, 1e-6, w_scale=w_scale)
    assert orc.rel_max_err(y.cpu()[rows], ref) <= FP8_TOL_SMALL_K      # a row sample's own maximum is a noisy denominator
    assert orc.rel_max_err(y.cpu()[rows], orc.fp8_kernel_model(x[rows], gm, Wq, w_scale, 1e-6).float()) <= 1e-2
    assert orc.rel_max_err(y, yw.float()) <= ONE_ULP
    for _ in range(3):
        assert torch.equal(kb.rmsnorm_linear(xd, gd, Wqd, 1e-6, w_scale=wsd), y)


@pytest.mark.parametrize("M", [1, 16, 33, 64])
def test_fp8_small_m_runs_the_stream_k_kernel(M):
    """e4m3 weights with M <= 64 (the memory-bound case, where e4m3 halves the bytes): the operand-swapped stream-K
    kernel on per-token quantised activations, at the decode benchmark's width."""
    N, K = 28672, 4096
    x, gm, W = orc.make_inputs(M, N, K, seed=40 + M)
    Wq, w_scale = orc.quantize_weight_e4m3(W)
    y = run_fp8(x, gm, Wq, w_scale, 1e-6)
    assert y.shape == (M, N)
    assert orc.rel_max_err(y, orc.reference_fp32(x, gm, Wq, 1e-6, w_scale=w_scale)) <= FP8_TOL_SMALL_K
    assert orc.rel_max_err(y, orc.fp8_kernel_model(x, gm, Wq, w_scale, 1e-6).float()) <= 1e-2
    assert torch.equal(run_fp8(x, gm, Wq, w_scale, 1e-6), y)
    # the same rows through the large-M kernel (padded to 128 tokens) agree to bf16 rounding
    xp = torch.zeros(128, K, dtype=torch.bfloat16)
    xp[:M] = x
    yp = run_fp8(xp, gm, Wq, w_scale, 1e-6)[:M]
    assert orc.rel_max_err(yp, y.float()) <= 1e-2


def test_config5_fp8_weights():
    M, N, K = 8192, 14336, 4096
    g = torch.Generator().manual_seed(18)
    x = torch.randn(M, K, generator=g).bfloat16()
    gm = (1 + 0.1 * torch.randn(K, generator=g)).bfloat16()
    W = (torch.randn(N, K, generator=g) * K ** -0.5).bfloat16()
    Wq, w_scale = orc.quantize_weight_e4m3(W)
    xd, gd, Wqd, wsd = x.to(DEV), gm.to(DEV), Wq.to(DEV), w_scale.to(DEV)
    y = kb.rmsnorm_linear(xd, gd, Wqd, 1e-6, w_scale=wsd)
    torch.cuda.synchronize()
    kb.check_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    Wdq = Wqd.float() * wsd[:, None]
    # the metric over the whole tensor: max |y - y_ref| / max |y_ref|, y_ref by torch fp32 on the GPU in slabs
    max_err, max_ref = 0.0, 0.0
    for m0 in range(0, M, 1024):
        ref = orc.torch_rmsnorm_linear(xd[m0:m0 + 1024].float(), gd.float(), Wdq, 1e-6)
        max_err = max(max_err, float((y[m0:m0 + 1024].float() - ref).abs().max()))
        max_ref = max(max_ref, float(ref.abs().max()))
    assert max_err / max_ref <= FP8_TOL
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(5))[:16]
    # the CPU oracle on a row sample, against the same denominator (a 16-row sample's own max is much noisier)
    ref = orc.reference_fp32(x[rows], gm, Wq, 1e-6, w_scale=w_scale)
    assert float((y.cpu()[rows].float() - ref).abs().max()) / max_ref <= FP8_TOL
    assert torch.equal(kb.rmsnorm_linear(xd, gd, Wqd, 1e-6, w_scale=wsd), y)


def test_fp8_bad_arguments():
    x, gm, W = orc.make_inputs(16, 64, 64)
    Wq, w_scale = orc.quantize_weight_e4m3(W)
    with pytest.raises(ValueError):
        kb.rmsnorm_linear(x.to(DEV), gm.to(DEV), Wq.to(DEV), 1e-6)                 # scales missing
    with pytest.raises(ValueError):
        kb.rmsnorm_linear(x.to(DEV), gm.to(DEV), W.to(DEV), 1e-6, w_scale=w_scale.to(DEV))  # scales with bf16 W


def test_host_buffer_front_end():
    """Pinned host in, pinned host out, several steps in flight; results equal the direct call."""
    M, N, K = 300, 520, 320
    x, gm, W = orc.make_inputs(M, N, K, seed=21)
    op = kb.HostRMSNormLinear(gm.to(DEV), W.to(DEV), 1e-6, max_tokens=M, depth=2)
    xs = [(x * (i + 1)).pin_memory() for i in range(5)]
    ys = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in range(5)]
    for xh, yh in zip(xs, ys):
        op.submit(xh, yh)
    op.wait()
    kb.check_status()
    for xh, yh in zip(xs, ys):
        assert orc.rel_max_err(yh, orc.reference_fp32(xh, gm, W, 1e-6)) <= BF16_TOL
    with pytest.raises(ValueError):
        op.submit(x, ys[0])          # not pinned


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 520, 320), (2048, 2048, 2048), (4096, 1024, 4096)])
def test_plain_gemm_max_line(M, N, K):
    """The norm-free GEMM (the reference's "max" line) against fp32 matmul."""
    x, _, W = orc.make_inputs(M, N, K, seed=M + K)
    y = kb.gemm_nt(x.to(DEV), W.to(DEV))
    torch.cuda.synchronize()
    kb.check_status()
    ref = x.float() @ W.float().t()
    assert orc.rel_max_err(y.cpu(), ref) <= BF16_TOL


def test_plain_gemm_on_wide_tiles():
    """A shape whose 256 x 512 tiles fill their rounds (8 x 37 tiles = 4 rounds of 74 pairs): the norm-free GEMM
    takes them too; full tensor against fp32 matmul on the GPU."""
    M, N, K = 2048, 18944, 4096
    x, _, W = orc.make_inputs(M, N, K, seed=41)
    xd, Wd = x.to(DEV), W.to(DEV)
    y = kb.gemm_nt(xd, Wd)
    torch.cuda.synchronize()
    kb.check_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    assert orc.rel_max_err(y, xd.float() @ Wd.float().t()) <= BF16_TOL


def test_harness_job_runs_and_reports(tmp_path):
    """The reference-style job on its smallest shape: rows for b200 / torch / max, accuracy columns filled."""
    from kernel_benchmarking_b200 import harness
    job = harness.rmsnorm_linear_job(0)
    rows = job.run(pause_s=0.0)
    by = {r.label.split(":")[-1]: r for r in rows}
    assert set(by) == {"b200", "torch", "max", "max_b200"}
    assert by["b200"].rmse is not None and by["b200"].rmse <= 2.0 * by["torch"].rmse + 1e-3
    assert by["b200"].ms_median > 0 and by["b200"].baseline_speedup > 0
    harness.write_rows(rows, str(tmp_path / "r.csv"))
    assert (tmp_path / "r.csv").read_text().startswith("rmsnorm_linear:0:b200,2048,2048,2048,")


def test_swiglu_golden_and_shapes(golden_dir):
    """Fused RMSNorm -> SwiGLU: the reference's golden vector, then larger shapes with gamma."""
    g = np.load(os.path.join(golden_dir, "swiglu_bf16_48x128x192.npz"))
    x, W = bf16(g["x_bits"]), bf16(g["W_bits"])
    y = kb.rmsnorm_swiglu(x.to(DEV), None, W.to(DEV), float(g["eps"]))
    torch.cuda.synchronize()
    kb.check_status()
    assert orc.rel_max_err(y.cpu(), torch.from_numpy(g["y_ref_fp64"])) <= BF16_TOL
    for (M, n, K) in [(300, 256, 320), (1024, 1792, 1024), (4096, 2048, 4096)]:
        x, gm, W = orc.make_inputs(M, 2 * n, K, seed=n)
        y = kb.rmsnorm_swiglu(x.to(DEV), gm.to(DEV), W.to(DEV), 1e-6)
        torch.cuda.synchronize()
        kb.check_status()
        ref = orc.torch_rmsnorm_swiglu(x.float(), gm.float(), W.float(), 1e-6)
        assert y.shape == (M, n)
        assert orc.rel_max_err(y.cpu(), ref) <= BF16_TOL
    with pytest.raises(ValueError):
        kb.rmsnorm_swiglu(x.to(DEV), gm.to(DEV), W[:200].contiguous().to(DEV), 1e-6)   # n not a multiple of 128


def test_swiglu_wide_layers_fold_gamma_in_the_pre_pass():
    """2n >= 6144 weight rows (and a GEMM large enough): gamma is folded into a copy of x by the pre-pass and the GEMM reads x straight from
    shared memory (as it always does without gamma); with a workspace too small for the copy the fold happens in
    the main loop.  Same bits either way."""
    import ctypes
    lib = _lib.load()
    M, n, K = 2048, 3072, 2560
    x, gm, W = orc.make_inputs(M, 2 * n, K, seed=31)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y = kb.rmsnorm_swiglu(xd, gd, Wd, 1e-6)
    y_nogamma = kb.rmsnorm_swiglu(xd, None, Wd, 1e-6)
    torch.cuda.synchronize()
    kb.check_status()
    assert orc.rel_max_err(y.cpu(), orc.torch_rmsnorm_swiglu(x.float(), gm.float(), W.float(), 1e-6)) <= BF16_TOL
    assert orc.rel_max_err(y_nogamma.cpu(), orc.torch_rmsnorm_swiglu(x.float(), torch.ones(K), W.float(), 1e-6)) <= BF16_TOL
    small = lib.rl_workspace_bytes(M, n, K, _lib.RL_W_BF16)
    assert small + M * K * 2 <= lib.rl_workspace_bytes(M, 2 * n, K, _lib.RL_W_BF16)
    ws = torch.zeros(small, dtype=torch.uint8, device=DEV)
    y2 = torch.empty(M, n, dtype=torch.bfloat16, device=DEV)
    rc = lib.rl_rmsnorm_swiglu_bf16(xd.data_ptr(), gd.data_ptr(), Wd.data_ptr(), y2.data_ptr(), M, n, K, K, K, n,
                                    ctypes.c_float(1e-6), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(y2, y)


def test_swiglu_on_wide_tiles():
    """A SwiGLU layer whose 256 x 512 tiles (256 gate + 256 up columns of the same 256 output channels) fill four
    rounds: same bits as the 256-column tiles (reached here through a workspace without room for the folded copy,
    which folds gamma in the main loop), and the whole tensor against fp32 torch on the GPU."""
    import ctypes
    lib = _lib.load()
    M, n, K = 2048, 9472, 4096
    x, gm, W = orc.make_inputs(M, 2 * n, K, seed=33)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y = kb.rmsnorm_swiglu(xd, gd, Wd, 1e-6)
    y_nogamma = kb.rmsnorm_swiglu(xd, None, Wd, 1e-6)
    torch.cuda.synchronize()
    kb.check_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    assert orc.rel_max_err(y, orc.torch_rmsnorm_swiglu(xd.float(), gd.float(), Wd.float(), 1e-6)) <= BF16_TOL
    assert orc.rel_max_err(y_nogamma, orc.torch_rmsnorm_swiglu(xd.float(), None, Wd.float(), 1e-6)) <= BF16_TOL
    ws = torch.zeros(lib.rl_workspace_bytes(M, n, K, _lib.RL_W_BF16) - M * K * 2, dtype=torch.uint8, device=DEV)
    y2 = torch.empty(M, n, dtype=torch.bfloat16, device=DEV)
    rc = lib.rl_rmsnorm_swiglu_bf16(xd.data_ptr(), gd.data_ptr(), Wd.data_ptr(), y2.data_ptr(), M, n, K, K, K, n,
                                    ctypes.c_float(1e-6), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(y2, y)


def test_lora_golden_and_shapes(golden_dir):
    """LoRA-fused linear (the low-rank term as one more k-block of the main loop) against the reference's
    `torch_lora` output and, on larger shapes, against the restatement in fp32 on the GPU."""
    g = np.load(os.path.join(golden_dir, "lora_bf16_64x136x192_l16.npz"))
    a, b, lA, lB = (bf16(g[k]).to(DEV) for k in ("a_bits", "b_bits", "lA_bits", "lB_bits"))
    y = kb.lora_linear(a, b, lA, lB)
    torch.cuda.synchronize()
    kb.check_status()
    assert orc.rel_max_err(y.cpu(), torch.from_numpy(g["y_ref_fp64"])) <= BF16_TOL
    torch.backends.cuda.matmul.allow_tf32 = False
    for (M, N, K, L) in [(300, 520, 320, 16), (2048, 2048, 2048, 16), (4096, 1024, 4096, 16), (512, 1024, 4096, 64),
                         (1024, 768, 1000, 8)]:
        gen = torch.Generator().manual_seed(M + N + K + L)
        a = torch.randn(M, K, generator=gen).bfloat16().to(DEV)
        b = (torch.randn(N, K, generator=gen) * K ** -0.5).bfloat16().to(DEV)
        lA = (torch.randn(L, K, generator=gen) * K ** -0.5).bfloat16().to(DEV)
        lB = torch.randn(N, L, generator=gen).bfloat16().to(DEV)      # a low-rank term as large as the main one
        y = kb.lora_linear(a, b, lA, lB)
        torch.cuda.synchronize()
        kb.check_status()
        ref = orc.torch_lora(a.float(), b.float(), lA.float(), lB.float())
        assert orc.rel_max_err(y, ref) <= BF16_TOL, (M, N, K, L)
        # the low-rank term really is in there
        assert orc.rel_max_err(kb.gemm_nt(a, b), ref) > 5 * BF16_TOL
        assert torch.equal(kb.lora_linear(a, b, lA, lB), y)
    with pytest.raises(ValueError):
        kb.lora_linear(a, b, lA[:4], lB[:, :4].contiguous())         # lora_dim 4: not a multiple of 8


def test_bounded_wait_reports_instead_of_hanging():
    """Failure detection: a wait that can never be satisfied runs out after its limit, leaves an error record
    in the status block and the context stays usable (no trap, no hang)."""
    import ctypes
    lib = _lib.load()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(4096, dtype=torch.uint8, device=DEV)
    assert lib.rl_workspace_init(ws.data_ptr(), ws.numel(), stream) == _lib.RL_OK
    assert lib.rl_selftest_wait_timeout(ws.data_ptr(), ws.numel(), 2_000_000, stream) == _lib.RL_OK   # 2 ms
    detail = (ctypes.c_int * 8)()
    assert lib.rl_read_status(ws.data_ptr(), detail) == _lib.RL_ERR_DEVICE_TIMEOUT
    assert detail[0] == 1 and detail[1] == 9 and detail[6] == 2      # timeout, role 9, the waiters gave up
    # the context is alive: clear the record and run the operator
    assert lib.rl_workspace_init(ws.data_ptr(), ws.numel(), stream) == _lib.RL_OK
    assert lib.rl_read_status(ws.data_ptr(), detail) == _lib.RL_OK
    x, gm, W = orc.make_inputs(16, 256, 128, seed=3)
    assert orc.rel_max_err(run(x, gm, W, 1e-6), orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL


def test_chained_calls_need_no_synchronise_between_them():
    """A small-M call (whose kernel lets its successor start early) feeding the plain GEMM and the LoRA linear,
    back to back on one stream: the consumers must see the finished y, as if a synchronise stood between."""
    M, N, K, N2 = 16, 1024, 512, 768
    x, gm, W = orc.make_inputs(M, N, K, seed=7)
    g = torch.Generator().manual_seed(8)
    W2 = (torch.randn(N2, N, generator=g) * N ** -0.5).bfloat16().to(DEV)
    lA = (torch.randn(16, N, generator=g) * N ** -0.5).bfloat16().to(DEV)
    lB = torch.randn(N2, 16, generator=g).bfloat16().to(DEV)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    xpad = torch.zeros(256, K, dtype=torch.bfloat16, device=DEV)
    xpad[:M] = xd
    # reference chain with a synchronise after every call
    y1 = kb.rmsnorm_linear(xpad, gd, Wd, 1e-6)
    torch.cuda.synchronize()
    z_ref = kb.gemm_nt(y1, W2)
    torch.cuda.synchronize()
    l_ref = kb.lora_linear(y1, W2, lA, lB)
    torch.cuda.synchronize()
    ysm = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
    torch.cuda.synchronize()
    zs_ref = kb.gemm_nt(ysm, W2)
    torch.cuda.synchronize()
    y_buf, ysm_buf = torch.empty_like(y1), torch.empty_like(ysm)
    for _ in range(50):
        y_buf.zero_()
        ysm_buf.zero_()
        kb.rmsnorm_linear(xpad, gd, Wd, 1e-6, out=y_buf)
        z = kb.gemm_nt(y_buf, W2)
        lo = kb.lora_linear(y_buf, W2, lA, lB)
        kb.rmsnorm_linear(xd, gd, Wd, 1e-6, out=ysm_buf)      # small-M kernel: triggers its dependents early
        zs = kb.gemm_nt(ysm_buf, W2)
        assert torch.equal(z, z_ref) and torch.equal(lo, l_ref) and torch.equal(zs, zs_ref)
    kb.check_status()


def test_bad_output_buffers_raise():
    """A caller-supplied `out` of the wrong shape or on the wrong device must be refused on the host: the kernel's
    store is laid out from M and N and would write past a smaller buffer."""
    x, gm, W = orc.make_inputs(256, 256, 64, seed=1)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    small = torch.empty(128, 256, dtype=torch.bfloat16, device=DEV)
    for call in (lambda: kb.rmsnorm_linear(xd, gd, Wd, 1e-6, out=small),
                 lambda: kb.gemm_nt(xd, Wd, out=small),
                 lambda: kb.rmsnorm_swiglu(xd, gd, Wd, 1e-6, out=small),
                 lambda: kb.rmsnorm_swiglu(xd, gd, Wd, 1e-6, out=torch.empty(256, 256, dtype=torch.bfloat16, device=DEV)),
                 lambda: kb.rmsnorm_swiglu(xd, gd[:32], Wd, 1e-6),
                 lambda: kb.rmsnorm_swiglu(xd, gd.float(), Wd, 1e-6),
                 lambda: kb.gemm_nt(xd, Wd, out=torch.empty(256, 256, dtype=torch.bfloat16))):
        with pytest.raises(ValueError):
            call()


def test_status_check_clears_the_workspace_after_a_timeout():
    """check_status() raises on a recorded device-side timeout and leaves the workspace clean, so the next call
    on the same stream works and reports nothing."""
    from kernel_benchmarking_b200 import ops
    x, gm, W = orc.make_inputs(16, 256, 128, seed=3)
    ref = orc.reference_fp32(x, gm, W, 1e-6)
    assert orc.rel_max_err(run(x, gm, W, 1e-6), ref) <= BF16_TOL         # makes sure this stream has a workspace
    stream = ops._stream_ptr(torch.device(DEV))
    ws = ops._workspaces[(0, stream)]
    lib = _lib.load()
    ws[256:256 + 64].fill_(1)                                             # a counter left non-zero, as after a timeout
    assert lib.rl_selftest_wait_timeout(ws.data_ptr(), ws.numel(), 2_000_000, stream) == _lib.RL_OK
    with pytest.raises(RuntimeError):
        kb.check_status()
    kb.check_status()                                                     # clean again
    assert int(ws[:4096].to(torch.int32).sum()) == 0
    assert orc.rel_max_err(run(x, gm, W, 1e-6), ref) <= BF16_TOL


@pytest.mark.parametrize("M,N,K", [(300, 520, 328), (1100, 2048, 1024), (512, 6144, 256), (2048, 8192, 512)])
def test_gamma_folded_by_the_pre_pass_gives_the_bits_of_the_main_loop_fold(M, N, K):
    """Wide layers fold gamma once per activation in the row-statistics pre-pass (a copy of x in the workspace)
    instead of once per column tile in the GEMM's main loop: the product is rounded to bf16 the same way and the
    MMAs add in the same order, so the two give the same bits."""
    x, gm, W = orc.make_inputs(M, N, K, seed=21)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y_pre = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_prescaled")
    y_loop = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_prestats")
    torch.cuda.synchronize()
    kb.check_status()
    assert torch.equal(y_pre, y_loop)
    assert orc.rel_max_err(y_pre.cpu(), orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL
    # x as a column slice of a wider buffer: the copy is dense whatever the caller's leading dimension
    xb = torch.zeros(M, K + 72, dtype=torch.bfloat16, device=DEV)
    xb[:, :K] = xd
    assert torch.equal(kb.rmsnorm_linear(xb[:, :K], gd, Wd, 1e-6, variant="prefill_pair_prescaled"), y_pre)
    kb.check_status()


@pytest.mark.parametrize("M,N,K", [(300, 520, 328), (257, 700, 64), (512, 1032, 256), (1000, 8, 128), (2048, 7168, 1024)])
@pytest.mark.parametrize("has_gamma", [False, True])
def test_wide_tiles_give_the_bits_of_whole_narrow_tiles(M, N, K, has_gamma):
    """256 x 512 tiles (two MMA-wide column halves sharing one activation tile) against 256 x 256 tiles computed
    whole: the same k order per output element, so the same bits - including tiles whose second half, or whose
    second half's tail, lies beyond N."""
    x, gm, W = orc.make_inputs(M, N, K, seed=23, gamma=has_gamma)
    xd, Wd = x.to(DEV), W.to(DEV)
    gd = gm.to(DEV) if has_gamma else None
    y_wide = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_wide")
    narrow = "prefill_pair_prestats_whole" if has_gamma else "prefill_pair_direct_prestats"
    y_narrow = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant=narrow)
    torch.cuda.synchronize()
    kb.check_status()
    assert orc.rel_max_err(y_wide.cpu(), orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL
    # (without gamma the narrow kernel may cut its last round along K: one bf16 ulp there)
    if has_gamma:
        assert torch.equal(y_wide, y_narrow)
    else:
        assert orc.rel_max_err(y_wide, y_narrow.float()) <= ONE_ULP


@pytest.mark.parametrize("M,N,K,has_gamma", [(2048, 5120, 2048, True),      # 80 wide tiles = 74 + 6: the 6 cut in 4
                                             (2304, 8192, 2560, False),     # 144 = 74 + 70: nothing to cut
                                             (4608, 4608, 2048, True),      # 162 = 2 x 74 + 14: cut in 4
                                             (2560, 6144, 3072, True)])     # 120 = 74 + 46: too many to cut
def test_wide_tiles_split_their_last_round_along_k(M, N, K, has_gamma):
    """The tiles of a partly filled last round of 256 x 512 tiles are cut along K like those of 256 x 256 tiles
    (partial blocks of 128 x 512 per CTA): one bf16 ulp from tiles computed whole, same bits run to run."""
    x, gm, W = orc.make_inputs(M, N, K, seed=27, gamma=has_gamma)
    xd, Wd = x.to(DEV), W.to(DEV)
    gd = gm.to(DEV) if has_gamma else None
    y = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_wide")
    y_again = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_wide")
    narrow = "prefill_pair_prestats_whole" if has_gamma else "prefill_pair_direct_prestats"
    y_narrow = kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant=narrow)
    torch.cuda.synchronize()
    kb.check_status()
    assert torch.equal(y, y_again)
    assert orc.rel_max_err(y, y_narrow.float()) <= ONE_ULP
    torch.backends.cuda.matmul.allow_tf32 = False
    assert orc.rel_max_err(y, orc.reference_fp32(xd, gd, Wd, 1e-6)) <= BF16_TOL


def test_auto_picks_wide_tiles_for_long_k_loops_that_fill_their_rounds():
    lib = _lib.load()
    name = lambda *a: _lib.VARIANT_NAMES[lib.rl_select_variant(*a)]
    assert name(16384, 57344, 8192, 1, 1) == "prefill_pair_wide"      # the whole MLP layer: 97 rounds of wide tiles
    assert name(16384, 7168, 8192, 1, 1) == "prefill_pair_wide"       # one of eight shards: 13 rounds beat 24.2 narrow ones
    assert name(8192, 8192, 8192, 0, 1) == "prefill_pair_wide"        # without gamma as well
    assert name(4096, 6144, 4096, 1, 1) == "prefill_pair_prescaled"   # 2.6 rounds of wide tiles would run as 3
    assert name(4096, 28672, 2048, 1, 1) == "prefill_pair_prescaled"  # short k-loop: the drain of a wide tile shows
    M, N, K = 2048, 18944, 4096                                       # 8 x 37 wide tiles = 4 rounds of 74 pairs
    assert name(M, N, K, 1, 1) == "prefill_pair_wide"
    assert name(M, N, K, 0, 1) == "prefill_pair_wide"
    x, gm, W = orc.make_inputs(M, N, K, seed=24)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
    assert torch.equal(y, kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_wide"))
    assert torch.equal(y, kb.rmsnorm_linear(xd, gd, Wd, 1e-6, variant="prefill_pair_prestats_whole"))
    torch.cuda.synchronize()
    kb.check_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    assert orc.rel_max_err(y, orc.reference_fp32(xd, gd, Wd, 1e-6)) <= BF16_TOL


def test_auto_folds_gamma_in_the_pre_pass_only_when_the_workspace_holds_the_copy():
    import ctypes
    lib = _lib.load()
    M, N, K = 2048, 6144, 2560                   # wide enough (N >= 6144) and large enough (M N K >= 3e10) for the copy to pay
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(M, N, K, 1, 1)] == "prefill_pair_prescaled"
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(M, N - 256, K, 1, 1)] == "prefill_pair_prestats"
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(M, N, K, 0, 1)] == "prefill_pair_direct_prestats"
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(256, 8192, 4096, 1, 1)] == "prefill_pair_prestats"   # a 30 us GEMM: no copy
    full = lib.rl_workspace_bytes(M, N, K, _lib.RL_W_BF16)
    narrow = lib.rl_workspace_bytes(M, N - 256, K, _lib.RL_W_BF16)
    assert full >= narrow + M * K * 2            # the copy is counted for wide layers only
    x, gm, W = orc.make_inputs(M, N, K, seed=22)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y_auto = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
    # the same call through the C ABI with a workspace that ends before the copy: still runs (gamma folded in the
    # main loop) and, the two forms being bit-identical, gives the same result
    ws = torch.zeros(narrow, dtype=torch.uint8, device=DEV)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.rl_rmsnorm_linear_bf16(xd.data_ptr(), gd.data_ptr(), Wd.data_ptr(), y.data_ptr(), M, N, K, K, K, N,
                                    ctypes.c_float(1e-6), ws.data_ptr(), ws.numel(), 0, st)
    assert rc == 0
    # asked for by name with that workspace: refused, nothing launched
    rc = lib.rl_rmsnorm_linear_bf16(xd.data_ptr(), gd.data_ptr(), Wd.data_ptr(), y.data_ptr(), M, N, K, K, K, N,
                                    ctypes.c_float(1e-6), ws.data_ptr(), ws.numel(),
                                    _lib.VARIANTS["prefill_pair_prescaled"], st)
    assert rc == _lib.RL_ERR_WORKSPACE
    torch.cuda.synchronize()
    assert torch.equal(y, y_auto)
    assert orc.rel_max_err(y.cpu(), orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL


def test_auto_whole_never_splits_and_matches():
    """`variant="auto_whole"`: the kernels AUTO picks, every tile computed whole (no CTA waits for another)."""
    for (M, N, K, has_gamma) in [(4096, 1536, 7168, True), (512, 1024, 4096, False), (8, 1024, 512, True)]:
        x, gm, W = orc.make_inputs(M, N, K, seed=5, gamma=has_gamma)
        ya = run(x, gm, W, 1e-6)
        yw = run(x, gm, W, 1e-6, variant="auto_whole")
        assert orc.rel_max_err(yw, orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL
        assert orc.rel_max_err(yw, ya.float()) <= ONE_ULP
    lib = _lib.load()
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(4096, 6144, 4096, 1, 1)] == "prefill_pair_prescaled"
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(4096, 4096, 4096, 1, 1)] == "prefill_pair_prestats"
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(4096, 6144, 4096, 0, 1)] == "prefill_pair_direct_prestats"
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(16, 28672, 4096, 1, 1)] == "decode"
    assert _lib.VARIANT_NAMES[lib.rl_select_variant(100, 512, 512, 1, 1)] == "prefill_pair_prestats"


@pytest.mark.skipif(torch.cuda.is_available() and torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_parallel_two_gpus_nccl():
    """W split over two GPUs, x replicated, y assembled with one NCCL all-gather: equals the oracle."""
    import subprocess
    import sys as _sys
    import socket
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_column_parallel_worker.py")
    with socket.socket() as sock:          # a port nobody holds right now: two suites on one box do not collide
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    r = subprocess.run([_sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), worker],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_decode_call_in_a_cuda_graph():
    """The small-M call captured in a CUDA graph and replayed: same bits as the eager call."""
    M, N, K = 8, 2048, 1024
    x, gm, W = orc.make_inputs(M, N, K, seed=31)
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y_eager = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    y_graph = torch.zeros_like(y_eager)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        kb.rmsnorm_linear(xd, gd, Wd, 1e-6, out=y_graph)      # creates this stream's workspace before capture
        side.synchronize()
        with torch.cuda.graph(g, stream=side):
            kb.rmsnorm_linear(xd, gd, Wd, 1e-6, out=y_graph)
    torch.cuda.current_stream().wait_stream(side)
    y_graph.zero_()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    kb.check_status()
    assert torch.equal(y_graph, y_eager)
    assert orc.rel_max_err(y_graph.cpu(), orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL


def test_strided_operands():
    """x, W and y as column slices of wider buffers (leading dimensions larger than the rows)."""
    for (M, N, K) in [(200, 264, 192), (9, 264, 192)]:
        x, gm, W = orc.make_inputs(M, N, K, seed=12)
        xb = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
        Wb = torch.zeros(N, K + 128, dtype=torch.bfloat16, device=DEV)
        xb[:, :K] = x.to(DEV)
        Wb[:, :K] = W.to(DEV)
        y = kb.rmsnorm_linear(xb[:, :K], gm.to(DEV), Wb[:, :K], 1e-6)
        torch.cuda.synchronize()
        kb.check_status()
        assert orc.rel_max_err(y.cpu(), orc.reference_fp32(x, gm, W, 1e-6)) <= BF16_TOL


def test_config4_whole_layer_on_one_gpu():
    """16384 x 57344 x 8192 unsharded (x 268 MB, W 940 MB, y 1.88 GB): row sample against the CPU oracle,
    column blocks against torch fp32 on the GPU."""
    M, N, K = 16384, 57344, 8192
    g = torch.Generator().manual_seed(18)
    x = torch.randn(M, K, generator=g).bfloat16()
    gm = (1 + 0.1 * torch.randn(K, generator=g)).bfloat16()
    W = torch.empty(N, K, dtype=torch.bfloat16)
    for n0 in range(0, N, 8192):
        W[n0:n0 + 8192] = (torch.randn(8192, K, generator=g) * K ** -0.5).bfloat16()
    xd, gd, Wd = x.to(DEV), gm.to(DEV), W.to(DEV)
    y = kb.rmsnorm_linear(xd, gd, Wd, 1e-6)
    torch.cuda.synchronize()
    kb.check_status()
    rows = torch.tensor([0, 1, 255, 256, 4097, 9999, 16000, 16383])
    assert orc.rel_max_err(y[rows.to(DEV)].cpu(), orc.reference_fp32(x[rows], gm, W, 1e-6)) <= BF16_TOL
    torch.backends.cuda.matmul.allow_tf32 = False
    for n0 in (0, 28672 - 128, 57344 - 256):
        ref = orc.torch_rmsnorm_linear(xd.float(), gd.float(), Wd[n0:n0 + 256].float(), 1e-6)
        assert orc.rel_max_err(y[:, n0:n0 + 256], ref) <= BF16_TOL
    del y, xd, Wd
    torch.cuda.empty_cache()
