"""The allocation-free entry point against the regular one (collected last on purpose).

rl_rmsnorm_linear_bf16_noalloc serves callers that have no way to obtain device memory - a plug-in
inside an engine that owns the whole GPU arena, or code that must not touch the CUDA allocator because
cudaMalloc / cudaFree stall every stream of the device.  It runs the same small-M kernel as
rl_rmsnorm_linear_bf16 but keeps its scratch in an array built into the library.  Both are called here
straight through the C ABI on the same inputs, twice in a row: the second call finds the array as the
first one left it.
"""
import ctypes

import pytest
import torch

from kernel_benchmarking_b200 import _lib
from oracle import rmsnorm_linear_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_TOL = 1e-2   # the tolerance of the bf16 parity tests


def _call_regular(lib, x, g, W, y, ws, stream):
    M, K = x.shape
    N = W.shape[0]
    return lib.rl_rmsnorm_linear_bf16(x.data_ptr(), None if g is None else g.data_ptr(), W.data_ptr(), y.data_ptr(), M, N, K, x.stride(0),
                                      W.stride(0), y.stride(0), ctypes.c_float(1e-6), ws.data_ptr(), ws.numel(),
                                      _lib.VARIANTS["decode"], stream)


def _call_noalloc(lib, x, g, W, y, stream):
    M, K = x.shape
    N = W.shape[0]
    return lib.rl_rmsnorm_linear_bf16_noalloc(x.data_ptr(), None if g is None else g.data_ptr(), W.data_ptr(), y.data_ptr(), M, N, K,
                                              x.stride(0), W.stride(0), y.stride(0), ctypes.c_float(1e-6), stream)


@pytest.mark.parametrize("M,N,K", [(1, 28672, 4096), (16, 28672, 4096), (5, 1000, 320)])
def test_noalloc_matches_regular_entry_point_twice(M, N, K):
    lib = _lib.load()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(lib.rl_workspace_bytes(M, N, K, _lib.RL_W_BF16), dtype=torch.uint8, device=DEV)
    assert lib.rl_workspace_init(ws.data_ptr(), ws.numel(), stream) == _lib.RL_OK
    for call in range(2):
        x, g, W = orc.make_inputs(M, N, K, seed=100 + call)
        x, g, W = x.to(DEV), g.to(DEV), W.to(DEV)
        y_ref = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        y_new = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        assert _call_regular(lib, x, g, W, y_ref, ws, stream) == _lib.RL_OK
        assert _call_noalloc(lib, x, g, W, y_new, stream) == _lib.RL_OK
        torch.cuda.synchronize()
        assert orc.rel_max_err(y_new, y_ref.float()) <= BF16_TOL
        assert orc.rel_max_err(y_new.cpu(), orc.reference_fp32(x.cpu(), g.cpu(), W.cpu(), 1e-6)) <= BF16_TOL


def test_noalloc_without_gamma_and_across_shapes():
    """gamma == NULL (the reference operator), and calls of different widths one after the other: each finds in the
    shared array the partial tiles a differently shaped call left there."""
    lib = _lib.load()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    for (M, N, K) in [(4, 1024, 512), (16, 28672, 512), (4, 1024, 512), (7, 520, 4096)]:
        x, _, W = orc.make_inputs(M, N, K, seed=M + N, gamma=False)
        x, W = x.to(DEV), W.to(DEV)
        ws = torch.empty(lib.rl_workspace_bytes(M, N, K, _lib.RL_W_BF16), dtype=torch.uint8, device=DEV)
        assert lib.rl_workspace_init(ws.data_ptr(), ws.numel(), stream) == _lib.RL_OK
        y_ref = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        y_new = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        assert _call_regular(lib, x, None, W, y_ref, ws, stream) == _lib.RL_OK
        assert _call_noalloc(lib, x, None, W, y_new, stream) == _lib.RL_OK
        torch.cuda.synchronize()
        assert torch.equal(y_new, y_ref)        # the same kernel on the same inputs: the same bits
        assert orc.rel_max_err(y_new.cpu(), orc.reference_fp32(x.cpu(), None, W.cpu(), 1e-6)) <= BF16_TOL


def test_noalloc_rejects_what_its_scratch_cannot_hold():
    lib = _lib.load()
    x, g, W = orc.make_inputs(17, 256, 64)
    x, g, W = x.to(DEV), g.to(DEV), W.to(DEV)
    y = torch.empty(17, 256, dtype=torch.bfloat16, device=DEV)
    rc = _call_noalloc(lib, x, g, W, y, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.RL_ERR_STATIC_SCRATCH
    assert "allocation-free" in _lib.error_string(rc)
