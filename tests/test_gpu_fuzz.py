"""Seeded random shapes through every operator of the library, against the oracle's torch path evaluated in fp32
on the GPU.  The fixed grids of test_gpu_parity.py probe the edges that are known; this sweep looks for the ones
that are not (ragged M, N and K in every size class, with and without gamma, every weight format)."""
import random

import pytest
import torch

import kernel_benchmarking_b200 as kb
from oracle import rmsnorm_linear_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_TOL = 1e-2


def _shape(rng):
    M = rng.choice([rng.randint(1, 64), rng.randint(65, 300), rng.randint(300, 3000), rng.choice([128, 256, 512, 1024])])
    # (the last class is wide enough for gamma to be folded by the pre-pass instead of in the main loop)
    N = rng.choice([rng.randint(1, 40) * 8, rng.randint(1, 500) * 8, rng.choice([256, 1024, 4096]),
                    rng.randint(768, 1100) * 8])
    K = rng.choice([rng.randint(1, 40) * 16, rng.randint(1, 260) * 16, rng.choice([64, 128, 4096])])
    return M, N, K


def _inputs(M, N, K, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(M, K, generator=gen, device=DEV).bfloat16()
    g = (1 + 0.1 * torch.randn(K, generator=gen, device=DEV)).bfloat16()
    W = (torch.randn(N, K, generator=gen, device=DEV) * K ** -0.5).bfloat16()
    return x, g, W, gen


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes_every_operator(seed):
    rng = random.Random(1000 + seed)
    torch.backends.cuda.matmul.allow_tf32 = False
    for case in range(20):
        kind = rng.choice(["bf16", "bf16", "no_gamma", "fp8", "gemm", "swiglu", "lora"])
        M, N, K = _shape(rng)
        if kind == "swiglu":
            N = max(128, N // 128 * 128)
        x, g, W, gen = _inputs(M, (2 * N) if kind == "swiglu" else N, K, seed * 100 + case)
        tol = BF16_TOL
        if kind in ("bf16", "no_gamma"):
            gg = g if kind == "bf16" else None
            # (256 x 512 tiles by name as well: AUTO only picks them for sweeps larger than this test draws)
            variants = ["auto", "auto_whole"] + (["prefill_pair_wide"] if M > 64 else [])
            y = kb.rmsnorm_linear(x, gg, W, 1e-6, variant=rng.choice(variants))
            ref = orc.reference_fp32(x, gg, W, 1e-6)
        elif kind == "fp8":
            Wq, w_scale = orc.quantize_weight_e4m3(W)
            y = kb.rmsnorm_linear(x, g, Wq, 1e-6, w_scale=w_scale)
            ref = orc.reference_fp32(x, g, Wq, 1e-6, w_scale=w_scale)
            tol = 8e-2 if K < 1024 else 5e-2      # few terms average little of the e4m3 rounding noise
        elif kind == "gemm":
            y = kb.gemm_nt(x, W)
            ref = x.float() @ W.float().t()
        elif kind == "swiglu":
            y = kb.rmsnorm_swiglu(x, g, W, 1e-6)
            ref = orc.torch_rmsnorm_swiglu(x.float(), g.float(), W.float(), 1e-6)
        else:
            L = rng.choice([8, 16, 64])
            lA = (torch.randn(L, K, generator=gen, device=DEV) * K ** -0.5).bfloat16()
            lB = torch.randn(N, L, generator=gen, device=DEV).bfloat16()
            y = kb.lora_linear(x, W, lA, lB)
            ref = x.float() @ W.float().t() + (x.float() @ lA.float().t()).bfloat16().float() @ lB.float().t()
        torch.cuda.synchronize()
        kb.check_status()
        assert tuple(y.shape) == tuple(ref.shape), (kind, M, N, K)
        assert bool(torch.isfinite(y.float()).all()), (kind, M, N, K)
        assert orc.rel_max_err(y, ref) <= tol, (kind, M, N, K)
