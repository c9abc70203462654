"""CPU oracle for the fused RMSNorm -> Linear operator.

TEST INFRASTRUCTURE ONLY: the product path never imports this module and has
no CPU fallback.  Only the tests, the smoke check and the benchmark's CPU
baseline leg use it.

Parity status: the reference project ships no golden vectors, known-answer
tests or fixtures for this path (its scripts compute a torch fp64 result live
and only print error figures, python/profile_utils.py:52-56,415).  The oracle
is therefore pinned against outputs of the reference's own functions
(python/baselines/rmsnorm_swiglu.py:25-34) imported on the build machine; the
committed vectors and the script that made them live in tests/golden/.

Two independent restatements are kept so that one checks the other:

* ``torch_*``  - the same torch calls the reference makes, extended with
  ``weight=gamma`` (the reference has no gamma; gamma=None reproduces it).
* ``np_*``     - plain numpy arithmetic, no torch ops in the math.
"""
from __future__ import annotations

import numpy as np
import torch

E4M3_MAX = 448.0


# --------------------------------------------------------------------------
# torch restatement (same calls as the reference)
# --------------------------------------------------------------------------
def torch_rmsnorm(a: torch.Tensor, gamma: torch.Tensor | None = None, eps: float = 1e-5) -> torch.Tensor:
    """python/baselines/rmsnorm_swiglu.py:25-26 (`rmsnorm`), plus optional weight."""
    return torch.nn.functional.rms_norm(a, normalized_shape=(a.shape[-1],), weight=gamma, eps=eps)


def torch_rmsnorm_linear(a: torch.Tensor, gamma: torch.Tensor | None, b: torch.Tensor,
                         eps: float = 1e-5) -> torch.Tensor:
    """python/baselines/rmsnorm_swiglu.py:28-34 (`rmsnorm_linear`) and the
    identical `torch_kernel` at demo/rmsnorm_linear.py:36-38:
    ``rms_norm(a) @ b.t()`` with a [M,K], b [N,K]."""
    return torch_rmsnorm(a, gamma, eps) @ b.t()


def torch_rmsnorm_linear_decomposed(a: torch.Tensor, gamma: torch.Tensor | None, b: torch.Tensor,
                                    eps: float = 1e-5) -> torch.Tensor:
    """python/baselines/rmsnorm_swiglu_trt.py:14-21 (`RMSNormLinearModule.forward`):
    explicit fp32 decomposition, cast back to the input dtype, then matmul."""
    a32 = a.float()
    n = a32 * torch.rsqrt(a32.pow(2).mean(dim=-1, keepdim=True) + eps)
    if gamma is not None:
        n = n * gamma.float()
    return n.to(a.dtype) @ b.t()


def torch_rmsnorm_swiglu(a: torch.Tensor, gamma: torch.Tensor | None, bb1: torch.Tensor,
                         eps: float = 1e-5) -> torch.Tensor:
    """python/baselines/rmsnorm_swiglu.py:36-42 (`rmsnorm_swiglu`) with `swiglu_concat` (:3-10): bb1 is [2n, k];
    o = rms_norm(a) @ bb1.t(); silu(o[:, :n]) * o[:, n:]."""
    o = torch_rmsnorm(a, gamma, eps) @ bb1.t()
    o1, o2 = o.chunk(2, dim=1)
    return torch.nn.functional.silu(o1) * o2


def torch_lora(a: torch.Tensor, b: torch.Tensor, lA: torch.Tensor, lB: torch.Tensor) -> torch.Tensor:
    """python/baselines/lora.py:4-13 (`torch_lora`): a [m, k], b [n, k], lA [l, k], lB [n, l], everything k-major;
    (a @ b.t()) + ((a @ lA.t()) @ lB.t())."""
    return (a @ b.t()) + ((a @ lA.t()) @ lB.t())


def reference_fp32(x: torch.Tensor, gamma: torch.Tensor | None, W: torch.Tensor, eps: float,
                   w_scale: torch.Tensor | None = None, dtype=torch.float32) -> torch.Tensor:
    """The parity target for the GPU kernels: inputs (bf16 / e4m3 bit patterns as
    given) widened to fp32 (or fp64), then the reference's torch path.  For e4m3
    weights the given (Wq, w_scale) pair is the input: W = Wq * w_scale[:, None]."""
    x_ = x.to(dtype)
    g_ = None if gamma is None else gamma.to(dtype)
    W_ = W.to(dtype)
    if w_scale is not None:
        W_ = W_ * w_scale.to(dtype)[:, None]
    return torch_rmsnorm_linear(x_, g_, W_, eps)


# --------------------------------------------------------------------------
# numpy restatement
# --------------------------------------------------------------------------
def np_rmsnorm_linear(x: np.ndarray, gamma: np.ndarray | None, W: np.ndarray, eps: float,
                      dtype=np.float64) -> np.ndarray:
    """y[m,n] = sum_k x[m,k] * rsqrt(mean_k x[m,k]^2 + eps) * gamma[k] * W[n,k]."""
    x = np.asarray(x, dtype=dtype)
    W = np.asarray(W, dtype=dtype)
    ms = np.mean(x * x, axis=-1, keepdims=True)
    xn = x / np.sqrt(ms + dtype(eps))
    if gamma is not None:
        xn = xn * np.asarray(gamma, dtype=dtype)[None, :]
    return xn @ W.T


def np_fused_form(x: np.ndarray, gamma: np.ndarray | None, W: np.ndarray, eps: float,
                  dtype=np.float64) -> np.ndarray:
    """The epilogue-scaled form every fused kernel of the reference uses
    (python/bench_kernels/helion/rmsnorm_linear.py:20-34): accumulate
    x@W^T and sum(x^2) together, multiply by rsqrt(sum/K + eps) at the end."""
    x = np.asarray(x, dtype=dtype)
    W = np.asarray(W, dtype=dtype)
    xg = x if gamma is None else x * np.asarray(gamma, dtype=dtype)[None, :]
    acc = xg @ W.T
    ss = np.sum(x * x, axis=-1, keepdims=True)
    return acc / np.sqrt(ss / x.shape[-1] + dtype(eps))


# --------------------------------------------------------------------------
# bf16 / e4m3 helpers (bit-level, numpy)
# --------------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(v: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (finite inputs)."""
    u = np.asarray(v, dtype=np.float32).view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))
    return (r >> 16).astype(np.uint16)


def e4m3_decode_table() -> np.ndarray:
    """All 256 e4m3fn codes as fp32 (bias 7, no infinities, 0x7f/0xff = NaN)."""
    t = np.zeros(256, dtype=np.float32)
    for c in range(256):
        s = -1.0 if c & 0x80 else 1.0
        e = (c >> 3) & 0xF
        m = c & 7
        if e == 0xF and m == 7:
            t[c] = np.nan
        elif e == 0:
            t[c] = s * (m / 8.0) * 2.0 ** (-6)
        else:
            t[c] = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return t


def f32_to_e4m3_bits(v: np.ndarray) -> np.ndarray:
    """Saturating round-to-nearest-even fp32 -> e4m3fn code (what
    cvt.rn.satfinite.e4m3x2.f32 does on the device)."""
    tab = e4m3_decode_table()
    pos = tab[:127].astype(np.float64)           # codes 0..126 are the finite non-negative values, ascending
    a = np.minimum(np.abs(np.asarray(v, dtype=np.float64)), E4M3_MAX)
    hi = np.clip(np.searchsorted(pos, a, side="left"), 0, 126)
    lo = np.clip(hi - 1, 0, 126)
    dlo = a - pos[lo]
    dhi = pos[hi] - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    code = np.where(a == pos[hi], hi, code).astype(np.uint8)
    sign = (np.signbit(np.asarray(v, dtype=np.float32))).astype(np.uint8) << 7
    return (code | sign).astype(np.uint8)


def quantize_weight_e4m3(W: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel weight quantiser used to build the FP8 inputs:
    w_scale[n] = absmax_k |W[n,k]| / 448, Wq = clamp(W / w_scale, +-448) -> e4m3fn.
    (torch's CPU cast does not saturate, hence the clamp.)"""
    W32 = W.float()
    w_scale = (W32.abs().amax(dim=1) / E4M3_MAX).clamp_min(1e-30)
    Wq = (W32 / w_scale[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return Wq, w_scale.float()


def fp8_kernel_model(x: torch.Tensor, gamma: torch.Tensor | None, Wq: torch.Tensor,
                     w_scale: torch.Tensor, eps: float) -> torch.Tensor:
    """Bit-level model of the FP8 kernel's arithmetic, for error budgeting:
    q = e4m3(x*gamma*448/amax_m) with amax_m = max_k |x*gamma|; fp32 accumulate;
    y = acc * rsqrt(mean(x^2)+eps) * amax_m/448 * w_scale[n]; bf16 output."""
    x32 = x.float()
    xg = x32 if gamma is None else x32 * gamma.float()
    amax = xg.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    # tensor / tensor is an IEEE division; `scalar / tensor` in torch is reciprocal-then-multiply (two roundings)
    qs = torch.full_like(amax, E4M3_MAX) / amax
    q = (xg * qs).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()
    acc = q @ Wq.float().t()
    r = torch.rsqrt(x32.pow(2).mean(dim=1, keepdim=True) + eps)
    y = acc * (r * amax / E4M3_MAX) * w_scale.float()[None, :]
    return y.to(torch.bfloat16)


# --------------------------------------------------------------------------
# error metrics
# --------------------------------------------------------------------------
def rel_max_err(y: torch.Tensor, y_ref: torch.Tensor) -> float:
    """max|y - y_ref| / max|y_ref| : the tolerance metric (bf16 <= 1e-2, fp8 <= 3e-2)."""
    y = y.double()
    y_ref = y_ref.double()
    return float((y - y_ref).abs().max() / y_ref.abs().max().clamp_min(1e-30))


def ref_metrics(ref: torch.Tensor, o: torch.Tensor) -> tuple[float, float, float]:
    """(rmse, max_abs, max_rel) as python/profile_utils.py:204-217 defines them
    (max_rel divides by |ref| clamped to >= 1)."""
    ref = ref.float()
    o = o.float()
    diff = (o - ref).abs()
    rmse = float(torch.nn.functional.mse_loss(o.flatten(), ref.flatten()).sqrt())
    return rmse, float(diff.max()), float((diff / ref.abs().clamp(min=1.0)).max())


# --------------------------------------------------------------------------
# seeded synthetic inputs
# --------------------------------------------------------------------------
def make_inputs(M: int, N: int, K: int, seed: int = 18, dtype=torch.bfloat16, gamma: bool = True):
    """x ~ N(0,1), gamma = 1 + 0.1 N(0,1), W ~ N(0, 1/K); generated in fp32 on the
    CPU with a seeded generator, then cast (seed 18 is the reference's,
    demo/rmsnorm_linear.py:20)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32).to(dtype)
    gm = (1.0 + 0.1 * torch.randn(K, generator=g, dtype=torch.float32)).to(dtype) if gamma else None
    W = (torch.randn(N, K, generator=g, dtype=torch.float32) * (K ** -0.5)).to(dtype)
    return x, gm, W


def make_inputs_outliers(M: int, N: int, K: int, seed: int = 18, p: float = 0.001, dtype=torch.bfloat16):
    """The reference's stress distribution for x and W both: N(0,1) + 10 N(0,1) Bernoulli(p)
    (python/profile_utils.py:255-262, `get_normal_bernoulli`)."""
    g = torch.Generator().manual_seed(seed)

    def one(shape):
        base = torch.randn(shape, generator=g, dtype=torch.float32)
        large = torch.randn(shape, generator=g, dtype=torch.float32) * 10
        mask = torch.bernoulli(torch.full(shape, p), generator=g)
        return (base + large * mask).to(dtype)

    return one((M, K)), None, one((N, K))
