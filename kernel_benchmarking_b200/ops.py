"""`rmsnorm_linear(x, gamma, W, eps) -> y` on torch tensors: the reference's kernel call surface.

The reference registers a kernel as any callable `fn(a, b, eps) -> out[M, N]`
on bf16 CUDA tensors a [M, K], b [N, K] (demo/new_profiling/rmsnorm_linear_new.py:97-103,
python/baselines/rmsnorm_swiglu.py:28-34).  This module provides that callable on
top of the C ABI; PyTorch only supplies device memory and the current stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib

_workspaces: dict = {}


def _stream_ptr(device: Optional[torch.device] = None) -> int:
    """Raw handle of torch's current stream on `device` (the fast C accessor when torch has it)."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    return raw(idx) if raw is not None else torch.cuda.current_stream(idx).cuda_stream


class _on_device:
    """`with torch.cuda.device(d)` only when d is not already current: the context manager costs several
    microseconds, which is a tenth of a decode-size kernel."""

    def __init__(self, device: torch.device):
        self.ctx = None if device.index == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None:
            self.ctx.__exit__(*a)


def _workspace(device: torch.device, nbytes: int, stream: int) -> torch.Tensor:
    """Per (device, stream) scratch for the status block and split-K partials; grown on demand,
    zeroed once by the library when created."""
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 12), dtype=torch.uint8, device=device)
        _lib.check(_lib.load().rl_workspace_init(ws.data_ptr(), ws.numel(), stream), "rl_workspace_init")
        _workspaces[key] = ws
    return ws


def _check_matrix(name: str, t: torch.Tensor, dtype: torch.dtype) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this operator has no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
    if t.stride(1) != 1:
        raise ValueError(f"{name} must be row-major with unit stride along its last dimension")


def _check_gamma(gamma: Optional[torch.Tensor], x: torch.Tensor, K: int) -> None:
    if gamma is None:
        return
    if not isinstance(gamma, torch.Tensor) or not gamma.is_cuda or gamma.device != x.device or gamma.dtype != torch.bfloat16:
        raise ValueError("gamma must be a bf16 CUDA tensor on x's device")
    if gamma.dim() != 1 or gamma.shape[0] != K or gamma.stride(0) != 1:
        raise ValueError(f"gamma must be a contiguous vector of length K={K}")


def _check_out(out: torch.Tensor, M: int, N: int, like: torch.Tensor) -> None:
    """A caller-supplied output: the kernel's TMA store is laid out from M and N, not from the buffer, so a
    smaller buffer or one on another device would be written out of bounds."""
    _check_matrix("out", out, torch.bfloat16)
    if tuple(out.shape) != (M, N) or out.device != like.device:
        raise ValueError(f"out must be [{M}, {N}] on the inputs' device, got {tuple(out.shape)} on {out.device}")


def rmsnorm_linear(x: torch.Tensor, gamma: Optional[torch.Tensor], W: torch.Tensor, eps: float = 1e-6, *,
                   w_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                   variant: str | int = "auto") -> torch.Tensor:
    """y = rms_norm(x, weight=gamma, eps) @ W.t() in one fused sm_100a kernel.

    x [M, K] bf16, gamma [K] bf16 or None (None = ones, which is the reference operator:
    `F.rms_norm(a, (K,), eps=eps) @ b.t()`, demo/rmsnorm_linear.py:36-38), W [N, K] bf16.
    Returns y [M, N] bf16 (fp32 accumulation).  Runs on the current CUDA stream, asynchronously.

    Quantised-inference path: W of dtype float8_e4m3fn with `w_scale` [N] fp32 per-output-channel
    scales (W_real = W * w_scale[:, None]); the normalised activations are quantised to e4m3 per
    token on the device.
    """
    _check_matrix("x", x, torch.bfloat16)
    fp8 = isinstance(W, torch.Tensor) and W.dtype == torch.float8_e4m3fn
    _check_matrix("W", W, torch.float8_e4m3fn if fp8 else torch.bfloat16)
    if fp8:
        if w_scale is None:
            raise ValueError("e4m3 weights need w_scale (fp32, one scale per output channel)")
        if (not w_scale.is_cuda or w_scale.device != x.device or w_scale.dtype != torch.float32
                or w_scale.dim() != 1 or w_scale.shape[0] != W.shape[0] or w_scale.stride(0) != 1):
            raise ValueError("w_scale must be a contiguous fp32 CUDA vector of length N on x's device")
    elif w_scale is not None:
        raise ValueError("w_scale is only meaningful with float8_e4m3fn weights")
    M, K = x.shape
    N, K2 = W.shape
    if K2 != K:
        raise ValueError(f"x is [M, {K}] but W is [N, {K2}]: inner dimensions differ")
    if W.device != x.device:
        raise ValueError("x and W must be on the same device")
    _check_gamma(gamma, x, K)
    if M == 0 or N == 0:
        return torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if out is None:
        ldy = (N + 7) // 8 * 8  # rows of y start on 16-byte boundaries for the TMA store
        buf = torch.empty((M, ldy), dtype=torch.bfloat16, device=x.device)
        out = buf if ldy == N else buf[:, :N]
    else:
        _check_out(out, M, N, x)
    v = _lib.VARIANTS[variant] if isinstance(variant, str) else int(variant)
    lib = _lib.load()
    stream = _stream_ptr(x.device)
    if fp8:
        with _on_device(x.device):
            ws = _workspace(x.device, lib.rl_workspace_bytes(M, N, K, _lib.RL_W_E4M3), stream)
            rc = lib.rl_rmsnorm_linear_fp8w(
                x.data_ptr(), None if gamma is None else gamma.data_ptr(), W.data_ptr(), w_scale.data_ptr(),
                out.data_ptr(), M, N, K, x.stride(0), W.stride(0), out.stride(0), ctypes.c_float(eps),
                ws.data_ptr(), ws.numel(), v, stream)
        _lib.check(rc, "rl_rmsnorm_linear_fp8w")
        return out
    with _on_device(x.device):
        nbytes = lib.rl_workspace_bytes(M, N, K, _lib.RL_W_BF16)
        if v in (_lib.VARIANTS["prefill_pair_prescaled"], _lib.VARIANTS["prefill_pair_wide"]):
            nbytes += M * K * 2 + 256  # room for the gamma-folded copy of x at widths where AUTO would not make one
        ws = _workspace(x.device, nbytes, stream)
        rc = lib.rl_rmsnorm_linear_bf16(
            x.data_ptr(), None if gamma is None else gamma.data_ptr(), W.data_ptr(), out.data_ptr(),
            M, N, K, x.stride(0), W.stride(0), out.stride(0), ctypes.c_float(eps),
            ws.data_ptr(), ws.numel(), v, stream)
    _lib.check(rc, "rl_rmsnorm_linear_bf16")
    return out


def rmsnorm_swiglu(x: torch.Tensor, gamma: Optional[torch.Tensor], W: torch.Tensor, eps: float = 1e-6, *,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(h[:, :n]) * h[:, n:] with h = rms_norm(x, weight=gamma) @ W.t(), W [2n, K] (gate rows, then up rows):
    the reference's `rmsnorm_swiglu(a, bb1, eps)` (python/baselines/rmsnorm_swiglu.py:36-42) in one kernel."""
    _check_matrix("x", x, torch.bfloat16)
    _check_matrix("W", W, torch.bfloat16)
    M, K = x.shape
    N2, K2 = W.shape
    if K2 != K or W.device != x.device or N2 % 2:
        raise ValueError("W must be [2n, K] on x's device")
    N = N2 // 2
    _check_gamma(gamma, x, K)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    else:
        _check_out(out, M, N, x)
    if M == 0:
        return out
    lib = _lib.load()
    stream = _stream_ptr(x.device)
    with _on_device(x.device):
        ws = _workspace(x.device, lib.rl_workspace_bytes(max(M, 65), 2 * N, K, _lib.RL_W_BF16), stream)
        rc = lib.rl_rmsnorm_swiglu_bf16(x.data_ptr(), None if gamma is None else gamma.data_ptr(), W.data_ptr(),
                                        out.data_ptr(), M, N, K, x.stride(0), W.stride(0), out.stride(0),
                                        ctypes.c_float(eps), ws.data_ptr(), ws.numel(), stream)
    _lib.check(rc, "rl_rmsnorm_swiglu_bf16")
    return out


def gemm_nt(a: torch.Tensor, b: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] @ b [N, K].t() in bf16 with fp32 accumulation, no norm: the reference's "max" line
    (`torch_gemm`, demo/new_profiling/rmsnorm_linear_new.py:29-31) on this library's CTA-pair kernel."""
    _check_matrix("a", a, torch.bfloat16)
    _check_matrix("b", b, torch.bfloat16)
    M, K = a.shape
    N, K2 = b.shape
    if K2 != K or b.device != a.device:
        raise ValueError("a [M, K] and b [N, K] must share K and the device")
    if out is None:
        ldc = (N + 7) // 8 * 8
        buf = torch.empty((M, ldc), dtype=torch.bfloat16, device=a.device)
        out = buf if ldc == N else buf[:, :N]
    else:
        _check_out(out, M, N, a)
    if M == 0 or N == 0:
        return out
    stream = _stream_ptr(a.device)
    with _on_device(a.device):
        # sized like the fused operator's: with room for the partial blocks of a k-split last round of tiles
        ws = _workspace(a.device, _lib.load().rl_workspace_bytes(max(M, 65), N, K, _lib.RL_W_BF16), stream)
        rc = _lib.load().rl_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                      out.stride(0), ws.data_ptr(), ws.numel(), stream)
    _lib.check(rc, "rl_gemm_bf16")
    return out


def lora_linear(a: torch.Tensor, b: torch.Tensor, lA: torch.Tensor, lB: torch.Tensor, *,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] @ b [N, K].t() + (a @ lA [L, K].t()) @ lB [N, L].t(): the reference's `torch_lora`
    (python/baselines/lora.py:4-13).  As in its fused kernels (demo/new_profiling/lora_new.py:44-50) the narrow
    product a @ lA.t() is computed first (here by this library's own GEMM) and rounded to bf16; the second kernel
    adds the low-rank term inside the main GEMM's accumulator.  L <= 64, a multiple of 8."""
    for name, t in (("a", a), ("b", b), ("lA", lA), ("lB", lB)):
        _check_matrix(name, t, torch.bfloat16)
    M, K = a.shape
    N, L = lB.shape
    if b.shape != (N, K) or lA.shape != (L, K) or any(t.device != a.device for t in (b, lA, lB)):
        raise ValueError("expected a [M, K], b [N, K], lA [L, K], lB [N, L] on one device")
    if L > 64 or L % 8:
        raise ValueError(f"lora_dim must be a multiple of 8 and at most 64, got {L}")
    if out is None:
        ldy = (N + 7) // 8 * 8
        buf = torch.empty((M, ldy), dtype=torch.bfloat16, device=a.device)
        out = buf if ldy == N else buf[:, :N]
    else:
        _check_out(out, M, N, a)
    if M == 0 or N == 0:
        return out
    xa = gemm_nt(a, lA)
    lib = _lib.load()
    stream = _stream_ptr(a.device)
    with _on_device(a.device):
        ws = _workspace(a.device, lib.rl_workspace_bytes(max(M, 65), N, K, _lib.RL_W_BF16), stream)
        rc = lib.rl_lora_linear_bf16(a.data_ptr(), b.data_ptr(), xa.data_ptr(), lB.data_ptr(), out.data_ptr(), M, N, K, L,
                                     a.stride(0), b.stride(0), xa.stride(0), lB.stride(0), out.stride(0),
                                     ws.data_ptr(), ws.numel(), stream)
    _lib.check(rc, "rl_lora_linear_bf16")
    return out


def quantize_rows_e4m3(x: torch.Tensor, gamma: Optional[torch.Tensor], eps: float = 1e-6):
    """First kernel of the FP8 path on its own: returns (q [M, K] float8_e4m3fn, row_scale [M] fp32) with
    q = e4m3(x * gamma * 448 / amax_row) and row_scale = rsqrt(mean x^2 + eps) * amax_row / 448."""
    _check_matrix("x", x, torch.bfloat16)
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    rs = torch.empty((M,), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        rc = _lib.load().rl_quantize_rows_e4m3(x.data_ptr(), None if gamma is None else gamma.data_ptr(), q.data_ptr(),
                                               rs.data_ptr(), M, K, x.stride(0), K, ctypes.c_float(eps),
                                               _stream_ptr(x.device))
    _lib.check(rc, "rl_quantize_rows_e4m3")
    return q.view(torch.float8_e4m3fn), rs


def row_stats(x: torch.Tensor, gamma: Optional[torch.Tensor], eps: float = 1e-6, *, want_amax: bool = True):
    """Per-token statistics: (inv_rms [M] fp32 = rsqrt(mean x^2 + eps), amax [M] fp32 = max |x * gamma| or None)."""
    _check_matrix("x", x, torch.bfloat16)
    M, K = x.shape
    if gamma is not None and (gamma.dtype != torch.bfloat16 or gamma.device != x.device or gamma.shape != (K,)
                              or gamma.stride(0) != 1):
        raise ValueError(f"gamma must be a contiguous bf16 vector of length K={K} on x's device")
    inv_rms = torch.empty((M,), dtype=torch.float32, device=x.device)
    amax = torch.empty((M,), dtype=torch.float32, device=x.device) if want_amax else None
    if M == 0:
        return inv_rms, amax
    with _on_device(x.device):
        rc = _lib.load().rl_row_stats(x.data_ptr(), None if gamma is None else gamma.data_ptr(), inv_rms.data_ptr(),
                                      None if amax is None else amax.data_ptr(), M, K, x.stride(0), ctypes.c_float(eps),
                                      _stream_ptr(x.device))
    _lib.check(rc, "rl_row_stats")
    return inv_rms, amax


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel launched through this module recorded a device-side
    timeout.  Kept out of `rmsnorm_linear` so the hot call never synchronises.

    A kernel that gave up a wait may leave tile counters of its workspace non-zero, and every later call on
    that workspace would then be wrong: the workspace is cleared again before the error is raised, so the
    caller can go on after handling it."""
    lib = _lib.load()
    first_error = None
    for (dev, stream), ws in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, dev):
            continue
        detail = (ctypes.c_int * 8)()
        with torch.cuda.device(dev):
            torch.cuda.synchronize()
            rc = lib.rl_read_status(ws.data_ptr(), detail)
            if rc != _lib.RL_OK:
                _lib.check(lib.rl_workspace_init(ws.data_ptr(), ws.numel(), stream), "rl_workspace_init")
                torch.cuda.synchronize()
                if first_error is None:
                    first_error = f"rmsnorm_linear: {_lib.error_string(rc)}; detail={list(detail)}"
    if first_error is not None:
        raise RuntimeError(first_error)
