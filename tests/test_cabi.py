"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

from kernel_benchmarking_b200 import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return _lib.load()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "rmsnorm_linear.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rl_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol(lib):
    names = header_symbols()
    assert "rl_rmsnorm_linear_bf16" in names and "rl_workspace_bytes" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/rmsnorm_linear.h but not exported"
    assert sorted(s[0] for s in _lib.SYMBOLS) == names


def test_version_and_error_strings(lib):
    assert lib.rl_version() >= 1000
    assert _lib.error_string(0) == "ok"
    for code in (-1, -2, -3, -4, -5, -6, -7, -8, -9):
        s = _lib.error_string(code)
        assert s and s != "unknown error code"
    assert _lib.error_string(-12345)


def test_workspace_bytes_is_pure_arithmetic(lib):
    small = lib.rl_workspace_bytes(4096, 4096, 4096, 0)
    # status block + counter region + one 1/rms per token + one 128 x 512 fp32 partial block per CTA of the
    # largest grid (160) for the k-split tiles of a partly filled last round (256-column tiles use half of each)
    # (+ 1 KB of progress words, one per CTA pair, for the alignment of the pairs at tile boundaries)
    assert small == 256 + 65536 + 4096 * 4 + 1024 + 160 * 128 * 512 * 4
    # layers of 6144 channels and more: room for the gamma-folded copy of x [M, K] as well
    assert lib.rl_workspace_bytes(4096, 6144, 4096, 0) == small + 4096 * 4096 * 2
    assert lib.rl_workspace_bytes(4096, 6144 - 8, 4096, 0) == small
    # ... and only where the GEMM is long enough for the copy to pay (M N K >= 3e10)
    assert lib.rl_workspace_bytes(256, 8192, 4096, 0) == small - (4096 - 256) * 4
    w16 = lib.rl_workspace_bytes(16, 28672, 4096, 0)
    w1 = lib.rl_workspace_bytes(1, 28672, 4096, 0)
    w64 = lib.rl_workspace_bytes(64, 28672, 4096, 0)
    assert w1 == w16 < w64
    # the counter region does not move with N: a workspace stays valid across shapes
    assert lib.rl_workspace_bytes(16, 128, 64, 0) == w16
    assert w64 < 64 << 20


def _plan(lib, M, N, K, pairs=74):
    a, b = ctypes.c_int(-1), ctypes.c_int(-1)
    assert lib.rl_plan_tail_split(M, N, K, pairs, ctypes.byref(a), ctypes.byref(b)) == 0
    return a.value, b.value


def test_tail_split_plan(lib):
    """Which tiles of the M > 128 kernels are cut along K: those of a last round that fills at most half the CTA
    pairs, in as many slices (4, 3 or 2) as there are idle pairs for, and only when K is long enough to pay for
    the exchange of partial sums."""
    assert _plan(lib, 16384, 28672, 8192) == (0, 0)        # 7168 tiles = 96.9 rounds: last round nearly full
    assert _plan(lib, 256 * 74, 256, 4096) == (0, 0)       # exactly one round
    assert _plan(lib, 512, 512, 1024) == (0, 0)            # K too short
    assert _plan(lib, 4096, 6144, 4096) == (14, 4)         # the prefill benchmark shape: 384 tiles = 5 rounds + 14
    assert _plan(lib, 4096, 4096, 4096) == (34, 2)         # 256 tiles = 3 rounds + 34
    assert _plan(lib, 4096, 1536, 7168) == (22, 3)         # 96 tiles = 1 round + 22
    assert _plan(lib, 16384, 7168, 8192) == (16, 4)        # one of eight shards of the MLP layer: 1792 = 24 x 74 + 16
    assert _plan(lib, 512, 1024, 4096) == (8, 4)           # fewer tiles than pairs
    assert _plan(lib, 8192, 8192, 8192) == (0, 0)          # 1024 = 13 x 74 + 62: more than half a round
    assert _plan(lib, 1024, 16384, 2048) == (0, 0)         # 34 tail tiles could only be halved, and K is short
    assert _plan(lib, 1024, 16384, 4096) == (34, 2)
    for pairs in (1, 7, 60, 64, 74, 80):
        for (M, N) in [(4096, 6144), (300, 520), (8192, 14336), (1000, 1032)]:
            tiles = ((M + 255) // 256) * ((N + 255) // 256)
            tail, split = _plan(lib, M, N, 4096, pairs)
            assert (tail, split) == (0, 0) or (tail == tiles % pairs and split in (2, 3, 4) and tail * split <= pairs
                                               and 2 * tail * split <= 160)
    assert lib.rl_plan_tail_split(0, 1, 1, 74, None, None) != 0


def test_argument_validation_needs_no_gpu(lib):
    f = lib.rl_rmsnorm_linear_bf16
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 15) // 16 * 16
    args = dict(M=128, N=128, K=64, ldx=64, ldw=64, ldy=128)

    def call(x=p, g=None, W=p, y=p, ws=None, ws_bytes=0, variant=0, **kw):
        a = {**args, **kw}
        return f(x, g, W, y, a["M"], a["N"], a["K"], a["ldx"], a["ldw"], a["ldy"], ctypes.c_float(1e-6), ws, ws_bytes,
                 variant, None)

    assert call(x=None) == _lib.RL_ERR_NULL_POINTER
    assert call(W=None) == _lib.RL_ERR_NULL_POINTER
    assert call(y=None) == _lib.RL_ERR_NULL_POINTER
    assert call(M=0) == _lib.RL_ERR_BAD_SHAPE
    assert call(N=-1) == _lib.RL_ERR_BAD_SHAPE
    assert call(ldx=32) == _lib.RL_ERR_BAD_SHAPE
    assert call(K=60, ldx=60, ldw=60) == _lib.RL_ERR_ALIGNMENT
    assert call(ldw=68) == _lib.RL_ERR_ALIGNMENT
    assert call(x=p + 2) == _lib.RL_ERR_ALIGNMENT
    assert call(g=p + 4) == _lib.RL_ERR_ALIGNMENT
    assert call(ldy=130) == _lib.RL_ERR_ALIGNMENT          # TMA store rows must start 16-byte aligned
    assert call(M=16, variant=0) == _lib.RL_ERR_WORKSPACE  # decode path needs its scratch
    assert call(M=16, ws=p, ws_bytes=256) == _lib.RL_ERR_WORKSPACE
    assert call(M=128, variant=20) == _lib.RL_ERR_BAD_VARIANT
    assert lib.rl_workspace_init(None, 0, None) == _lib.RL_ERR_NULL_POINTER
    assert lib.rl_read_status(None, None) == _lib.RL_ERR_NULL_POINTER


def test_check_maps_codes_to_exceptions(lib):
    with pytest.raises(ValueError):
        _lib.check(_lib.RL_ERR_ALIGNMENT, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.RL_ERR_WORKSPACE, "x")
    _lib.check(0, "x")
