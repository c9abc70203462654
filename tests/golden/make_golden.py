"""Generate the golden vectors under tests/golden/ from the REFERENCE's own code.

Run on a machine that has the reference checkout (pure torch on CPU):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `baselines.rmsnorm_swiglu` (python/baselines/
rmsnorm_swiglu.py:25-34), `RMSNormLinearModule` (python/baselines/
rmsnorm_swiglu_trt.py:7-21) and `baselines.lora.torch_lora` (python/baselines/
lora.py:4-13), feeds them seeded inputs and stores inputs and
outputs in one compressed .npz per case.  bf16 tensors are stored as uint16 bit
patterns, e4m3 as uint8 codes.  The reference operator has no gamma; cases with
gamma call the reference on (x, W * gamma[None, :]) in fp64, which is the same
contraction.  The test-suite only reads the .npz files.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "python"))
    from baselines.rmsnorm_swiglu import rmsnorm_linear as ref_rmsnorm_linear  # noqa: E402
    from baselines.rmsnorm_swiglu import rmsnorm_swiglu as ref_rmsnorm_swiglu  # noqa: E402
    from baselines.rmsnorm_swiglu_trt import RMSNormLinearModule  # noqa: E402

    torch.manual_seed(18)  # the reference's seed, demo/rmsnorm_linear.py:20

    # ---- case 1: tiny fp32, no gamma (exact reference semantics, eps 1e-5) ----
    x = torch.randn(4, 64, dtype=torch.float32)
    W = torch.randn(8, 64, dtype=torch.float32) / 8.0
    np.savez_compressed(
        os.path.join(HERE, "tiny_fp32_nogamma.npz"),
        x=x.numpy(), W=W.numpy(), eps=np.float64(1e-5),
        y_ref_fp32=ref_rmsnorm_linear(x, W, 1e-5).numpy(),
        y_ref_fp64=ref_rmsnorm_linear(x.double(), W.double(), 1e-5).numpy(),
        y_trt_module=RMSNormLinearModule(eps=1e-5)(x, W).numpy(),
    )

    # ---- case 2: fp32 with gamma, reduced "CPU plumbing" shape, eps 1e-6 ----
    M, N, K = 16, 32, 256
    x = torch.randn(M, K, dtype=torch.float32)
    gamma = 1.0 + 0.1 * torch.randn(K, dtype=torch.float32)
    W = torch.randn(N, K, dtype=torch.float32) * K ** -0.5
    y64 = ref_rmsnorm_linear(x.double(), W.double() * gamma.double()[None, :], 1e-6)
    np.savez_compressed(
        os.path.join(HERE, "small_fp32_gamma.npz"),
        x=x.numpy(), gamma=gamma.numpy(), W=W.numpy(), eps=np.float64(1e-6),
        y_ref_fp64=y64.numpy(),
    )

    # ---- case 3: bf16 inputs, the reference's outlier distribution, no gamma ----
    M, N, K = 128, 256, 128

    def normal_bernoulli(shape, p=0.001):
        # python/profile_utils.py:255-262
        base = torch.randn(shape, dtype=torch.float64)
        large = torch.randn(shape, dtype=torch.float64) * 10
        mask = torch.bernoulli(torch.full(shape, p, dtype=torch.float64))
        return base + large * mask

    a = normal_bernoulli((M, K)).to(torch.bfloat16)
    b = normal_bernoulli((N, K)).to(torch.bfloat16)
    np.savez_compressed(
        os.path.join(HERE, "bf16_outliers_128x256x128.npz"),
        x_bits=bf16_bits(a), W_bits=bf16_bits(b), eps=np.float64(1e-5),
        y_ref_fp64=ref_rmsnorm_linear(a.double(), b.double(), 1e-5).float().numpy(),
        y_ref_bf16_bits=bf16_bits(ref_rmsnorm_linear(a, b, 1e-5)),
    )

    # ---- case 4: bf16 inputs with gamma, ragged shape, BASELINE distributions ----
    M, N, K = 67, 136, 192
    x = torch.randn(M, K).to(torch.bfloat16)
    gamma = (1.0 + 0.1 * torch.randn(K)).to(torch.bfloat16)
    W = (torch.randn(N, K) * K ** -0.5).to(torch.bfloat16)
    y64 = ref_rmsnorm_linear(x.double(), W.double() * gamma.double()[None, :], 1e-6)
    np.savez_compressed(
        os.path.join(HERE, "bf16_gamma_67x136x192.npz"),
        x_bits=bf16_bits(x), gamma_bits=bf16_bits(gamma), W_bits=bf16_bits(W), eps=np.float64(1e-6),
        y_ref_fp64=y64.float().numpy(),
    )

    # ---- case 5: e4m3 weights with per-channel scales ----
    M, N, K = 32, 64, 256
    x = torch.randn(M, K).to(torch.bfloat16)
    gamma = (1.0 + 0.1 * torch.randn(K)).to(torch.bfloat16)
    W = (torch.randn(N, K) * K ** -0.5).to(torch.bfloat16)
    w_scale = (W.float().abs().amax(dim=1) / 448.0)
    Wq = (W.float() / w_scale[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    Wdq = Wq.double() * w_scale.double()[:, None]
    y64 = ref_rmsnorm_linear(x.double(), Wdq * gamma.double()[None, :], 1e-6)
    np.savez_compressed(
        os.path.join(HERE, "fp8w_32x64x256.npz"),
        x_bits=bf16_bits(x), gamma_bits=bf16_bits(gamma), W_bf16_bits=bf16_bits(W),
        Wq_codes=Wq.view(torch.uint8).numpy(), w_scale=w_scale.numpy(), eps=np.float64(1e-6),
        y_ref_fp64=y64.float().numpy(),
    )
    # ---- case 6: fused RMSNorm -> SwiGLU (gate rows then up rows), bf16 inputs, no gamma ----
    M, n, K = 48, 128, 192
    x = torch.randn(M, K).to(torch.bfloat16)
    bb1 = (torch.randn(2 * n, K) * K ** -0.5).to(torch.bfloat16)
    np.savez_compressed(
        os.path.join(HERE, "swiglu_bf16_48x128x192.npz"),
        x_bits=bf16_bits(x), W_bits=bf16_bits(bb1), eps=np.float64(1e-5),
        y_ref_fp64=ref_rmsnorm_swiglu(x.double(), bb1.double(), 1e-5).float().numpy(),
    )
    # ---- case 7: LoRA-fused linear, lora_dim 16 (its own seed: independent of the cases above) ----
    from baselines.lora import torch_lora as ref_lora  # noqa: E402
    torch.manual_seed(1818)
    M, N, K, L = 64, 136, 192, 16
    a = torch.randn(M, K).to(torch.bfloat16)
    b = (torch.randn(N, K) * K ** -0.5).to(torch.bfloat16)
    lA = (torch.randn(L, K) * K ** -0.5).to(torch.bfloat16)
    lB = (torch.randn(N, L) * L ** -0.5).to(torch.bfloat16)
    np.savez_compressed(
        os.path.join(HERE, "lora_bf16_64x136x192_l16.npz"),
        a_bits=bf16_bits(a), b_bits=bf16_bits(b), lA_bits=bf16_bits(lA), lB_bits=bf16_bits(lB),
        y_ref_fp64=ref_lora(a.double(), b.double(), lA.double(), lB.double()).float().numpy(),
        y_ref_bf16_bits=bf16_bits(ref_lora(a, b, lA, lB)),
    )
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    main(sys.argv[1])
