"""The oracle against the golden vectors produced by the reference's own functions
(tests/golden/make_golden.py), and its two restatements against each other."""
import os

import numpy as np
import pytest
import torch

from oracle import rmsnorm_linear_oracle as orc


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def bf16(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def test_tiny_fp32_no_gamma(golden_dir):
    g = load(golden_dir, "tiny_fp32_nogamma.npz")
    x, W, eps = torch.from_numpy(g["x"]), torch.from_numpy(g["W"]), float(g["eps"])
    y = orc.torch_rmsnorm_linear(x, None, W, eps)
    np.testing.assert_allclose(y.numpy(), g["y_ref_fp32"], rtol=1e-5, atol=1e-6)
    y64 = orc.np_rmsnorm_linear(g["x"], None, g["W"], eps)
    np.testing.assert_allclose(y64, g["y_ref_fp64"], rtol=1e-12, atol=1e-13)
    yd = orc.torch_rmsnorm_linear_decomposed(x, None, W, eps)
    np.testing.assert_allclose(yd.numpy(), g["y_trt_module"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(orc.np_fused_form(g["x"], None, g["W"], eps), g["y_ref_fp64"], rtol=1e-12, atol=1e-13)


def test_small_fp32_gamma(golden_dir):
    g = load(golden_dir, "small_fp32_gamma.npz")
    eps = float(g["eps"])
    y_np = orc.np_rmsnorm_linear(g["x"], g["gamma"], g["W"], eps)
    np.testing.assert_allclose(y_np, g["y_ref_fp64"], rtol=1e-11, atol=1e-12)
    y_t = orc.torch_rmsnorm_linear(torch.from_numpy(g["x"]).double(), torch.from_numpy(g["gamma"]).double(),
                                   torch.from_numpy(g["W"]).double(), eps)
    np.testing.assert_allclose(y_t.numpy(), g["y_ref_fp64"], rtol=1e-11, atol=1e-12)
    y_f = orc.np_fused_form(g["x"], g["gamma"], g["W"], eps)
    np.testing.assert_allclose(y_f, g["y_ref_fp64"], rtol=1e-11, atol=1e-12)
    y32 = orc.reference_fp32(torch.from_numpy(g["x"]), torch.from_numpy(g["gamma"]), torch.from_numpy(g["W"]), eps)
    assert orc.rel_max_err(y32, torch.from_numpy(g["y_ref_fp64"])) < 1e-5


def test_bf16_outliers(golden_dir):
    g = load(golden_dir, "bf16_outliers_128x256x128.npz")
    x, W, eps = bf16(g["x_bits"]), bf16(g["W_bits"]), float(g["eps"])
    y64 = orc.reference_fp32(x, None, W, eps, dtype=torch.float64)
    np.testing.assert_allclose(y64.float().numpy(), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
    y_np = orc.np_rmsnorm_linear(orc.bf16_bits_to_f32(g["x_bits"]), None, orc.bf16_bits_to_f32(g["W_bits"]), eps)
    np.testing.assert_allclose(y_np.astype(np.float32), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
    # the reference's own bf16 run stays within the bf16 tolerance of its fp64 run
    y_bf = bf16(g["y_ref_bf16_bits"])
    assert orc.rel_max_err(y_bf, torch.from_numpy(g["y_ref_fp64"])) < 1e-2
    assert orc.rel_max_err(orc.torch_rmsnorm_linear(x, None, W, eps), torch.from_numpy(g["y_ref_fp64"])) < 1e-2


def test_bf16_gamma_ragged(golden_dir):
    g = load(golden_dir, "bf16_gamma_67x136x192.npz")
    x, gm, W, eps = bf16(g["x_bits"]), bf16(g["gamma_bits"]), bf16(g["W_bits"]), float(g["eps"])
    y64 = orc.reference_fp32(x, gm, W, eps, dtype=torch.float64)
    np.testing.assert_allclose(y64.float().numpy(), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
    y32 = orc.reference_fp32(x, gm, W, eps)
    assert orc.rel_max_err(y32, torch.from_numpy(g["y_ref_fp64"])) < 1e-5


def test_fp8_weights(golden_dir):
    g = load(golden_dir, "fp8w_32x64x256.npz")
    x, gm, Wb, eps = bf16(g["x_bits"]), bf16(g["gamma_bits"]), bf16(g["W_bf16_bits"]), float(g["eps"])
    Wq, w_scale = orc.quantize_weight_e4m3(Wb)
    np.testing.assert_array_equal(Wq.view(torch.uint8).numpy(), g["Wq_codes"])
    np.testing.assert_allclose(w_scale.numpy(), g["w_scale"], rtol=1e-7)
    y64 = orc.reference_fp32(x, gm, Wq, eps, w_scale=w_scale, dtype=torch.float64)
    np.testing.assert_allclose(y64.float().numpy(), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
    # numpy path through the bit-level decode table
    Wdq = orc.e4m3_decode_table()[g["Wq_codes"]].astype(np.float64) * g["w_scale"].astype(np.float64)[:, None]
    y_np = orc.np_rmsnorm_linear(orc.bf16_bits_to_f32(g["x_bits"]), orc.bf16_bits_to_f32(g["gamma_bits"]), Wdq, eps)
    np.testing.assert_allclose(y_np.astype(np.float32), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
    # arithmetic model of the FP8 kernel (per-token e4m3 activations).  With only K=256 terms per
    # output the quantisation noise averages less than at the benchmark's K=4096 (where the
    # tolerance is 3e-2), so this small case is held to 5e-2.
    y_model = orc.fp8_kernel_model(x, gm, Wq, w_scale, eps)
    assert orc.rel_max_err(y_model, torch.from_numpy(g["y_ref_fp64"])) < 5e-2


def test_e4m3_tables_match_torch():
    codes = torch.arange(256, dtype=torch.uint8)
    t = codes.view(torch.float8_e4m3fn).float().numpy()
    tab = orc.e4m3_decode_table()
    finite = ~np.isnan(tab)
    np.testing.assert_array_equal(tab[finite], t[finite])
    assert np.isnan(t[~finite]).all()
    rng = np.random.default_rng(0)
    v = np.concatenate([rng.normal(size=4096) * 100, rng.normal(size=4096), rng.normal(size=4096) * 1e-2,
                        np.array([0.0, -0.0, 448.0, -448.0, 1000.0, -1e9, 2 ** -9, 2 ** -10, 3 * 2 ** -10])]).astype(np.float32)
    mine = orc.f32_to_e4m3_bits(v)
    ref = torch.from_numpy(v).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.testing.assert_array_equal(mine & 0x7F, ref & 0x7F)
    nz = (mine & 0x7F) != 0
    np.testing.assert_array_equal(mine[nz], ref[nz])


def test_bf16_bit_helpers():
    v = torch.randn(1000)
    bits = orc.f32_to_bf16_bits(v.numpy())
    np.testing.assert_array_equal(bits, v.bfloat16().view(torch.int16).numpy().view(np.uint16))
    np.testing.assert_array_equal(orc.bf16_bits_to_f32(bits), v.bfloat16().float().numpy())


@pytest.mark.parametrize("M,N,K", [(1, 8, 64), (5, 24, 128), (33, 40, 320)])
def test_fused_form_equals_unfused(M, N, K):
    x, gm, W = orc.make_inputs(M, N, K, seed=3, dtype=torch.float32)
    a = orc.np_rmsnorm_linear(x.numpy(), gm.numpy(), W.numpy(), 1e-6)
    b = orc.np_fused_form(x.numpy(), gm.numpy(), W.numpy(), 1e-6)
    np.testing.assert_allclose(a, b, rtol=1e-11, atol=1e-12)
    c = orc.torch_rmsnorm_linear(x.double(), gm.double(), W.double(), 1e-6).numpy()
    np.testing.assert_allclose(a, c, rtol=1e-11, atol=1e-12)


def test_config1_cpu_plumbing():
    """fp32, x [128, 4096], W [4096, 4096], gamma = 1 + 0.1 N(0,1), eps 1e-6: the reference torch path on CPU."""
    x, gm, W = orc.make_inputs(128, 4096, 4096, seed=18, dtype=torch.float32)
    y = orc.torch_rmsnorm_linear(x, gm, W, 1e-6)
    y64 = orc.torch_rmsnorm_linear(x.double(), gm.double(), W.double(), 1e-6)
    assert y.shape == (128, 4096)
    assert orc.rel_max_err(y, y64) < 1e-5
    rmse, max_abs, max_rel = orc.ref_metrics(y64.float(), y)
    assert rmse < 1e-5 and max_abs < 1e-4 and max_rel < 1e-4


def test_swiglu_golden(golden_dir):
    """The RMSNorm -> SwiGLU restatement against the reference's own `rmsnorm_swiglu` output."""
    g = load(golden_dir, "swiglu_bf16_48x128x192.npz")
    x, W, eps = bf16(g["x_bits"]), bf16(g["W_bits"]), float(g["eps"])
    y = orc.torch_rmsnorm_swiglu(x.double(), None, W.double(), eps)
    np.testing.assert_allclose(y.float().numpy(), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
    # numpy restatement: h = rmsnorm(x) @ W^T, silu(gate) * up
    h = orc.np_rmsnorm_linear(orc.bf16_bits_to_f32(g["x_bits"]), None, orc.bf16_bits_to_f32(g["W_bits"]), eps)
    n = h.shape[1] // 2
    y_np = h[:, :n] / (1.0 + np.exp(-h[:, :n])) * h[:, n:]
    np.testing.assert_allclose(y_np.astype(np.float32), g["y_ref_fp64"], rtol=1e-5, atol=1e-6)


def test_lora_golden(golden_dir):
    """The LoRA restatement against the reference's own `torch_lora` output (fp64 run and its bf16 run)."""
    g = load(golden_dir, "lora_bf16_64x136x192_l16.npz")
    a, b, lA, lB = (bf16(g[k]) for k in ("a_bits", "b_bits", "lA_bits", "lB_bits"))
    y = orc.torch_lora(a.double(), b.double(), lA.double(), lB.double())
    np.testing.assert_allclose(y.float().numpy(), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
    assert torch.equal(orc.torch_lora(a, b, lA, lB), bf16(g["y_ref_bf16_bits"]))
    # numpy restatement in fp64
    f = orc.bf16_bits_to_f32
    a64, b64, lA64, lB64 = (f(g[k]).astype(np.float64) for k in ("a_bits", "b_bits", "lA_bits", "lB_bits"))
    y_np = a64 @ b64.T + (a64 @ lA64.T) @ lB64.T
    np.testing.assert_allclose(y_np.astype(np.float32), g["y_ref_fp64"], rtol=1e-6, atol=1e-6)
