"""Column-parallel use of the operator on several GPUs of one node.

W [N, K] is split into contiguous row blocks (= column blocks of y) over the
ranks; x and gamma are replicated; each rank runs the unmodified single-GPU
kernel on its block, so the hot path has no collective.  Only when the caller
asks for the assembled y is an all-gather issued (NCCL over NVLink on GPUs, in
place, into a buffer kept between calls), and it is timed separately by the
benchmark.  The reference project has no
multi-GPU code at all; this is the one distributed feature of the build.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(N: int, world: int, rank: int, multiple: int = 8) -> Tuple[int, int]:
    """Rows [n0, n1) of W owned by `rank`: blocks of `multiple` channels are dealt out as evenly as
    possible, earlier ranks taking the remainder, the last rank also taking a ragged tail."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    if N < 0:
        raise ValueError("N must be non-negative")
    blocks = N // multiple
    q, r = divmod(blocks, world)
    b0 = rank * q + min(rank, r)
    b1 = b0 + q + (1 if rank < r else 0)
    n0, n1 = b0 * multiple, b1 * multiple
    if rank == world - 1:
        n1 = N
    return n0, n1


def shard_rows(t: torch.Tensor, world: int, rank: int, multiple: int = 8) -> torch.Tensor:
    """The rank's slice of a per-output-channel tensor (W [N, K] or a scale vector [N])."""
    n0, n1 = shard_bounds(t.shape[0], world, rank, multiple)
    return t[n0:n1]


class ColumnParallelRMSNormLinear:
    """One rank's share of y = rmsnorm(x) * gamma @ W^T with W split along N.

    `local_fn(x, gamma, W_local, eps) -> y_local` is the single-device operator
    (the CUDA kernel by default; the tests pass a CPU stand-in to exercise the
    sharding and gather arithmetic over gloo).  With e4m3 weights the rank also
    holds its slice of the per-output-channel scales (`w_scale_local`, fp32
    [n1 - n0]) and `local_fn` is called with `w_scale=` as the operator takes it.

    Assembling y.  The ranks' column blocks are gathered into one buffer per rank
    of shape [G, M, Nb] (block r = rank r's columns, Nb = the widest block), kept
    between calls.  `forward` writes the rank's own block straight into its place
    in that buffer (the kernel takes any leading dimension), so `gather` is a
    single in-place all-gather with no copy before or after it and no allocation
    per call.  `gather(layout="blocked")` returns the result as it lies, a
    [M, G, Nb] view in which y[m, n0_r + j] is element [m, r, j]; a consumer that
    reads y tile by tile (the next GEMM's TMA descriptor) can take it like that.
    `gather(layout="row_major")` (the default) also returns the plain [M, N]
    matrix, at the price of one strided copy of the whole tensor.
    """

    def __init__(self, W_local: torch.Tensor, gamma: Optional[torch.Tensor], eps: float, N_total: int,
                 group: Optional[dist.ProcessGroup] = None, local_fn: Optional[Callable] = None,
                 multiple: int = 8, w_scale_local: Optional[torch.Tensor] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N_total = N_total
        self.multiple = multiple
        self.n0, self.n1 = shard_bounds(N_total, self.world, self.rank, multiple)
        if W_local.shape[0] != self.n1 - self.n0:
            raise ValueError(
                f"rank {self.rank} expects {self.n1 - self.n0} rows of W, got {W_local.shape[0]}")
        if w_scale_local is not None and w_scale_local.shape != (self.n1 - self.n0,):
            raise ValueError(
                f"rank {self.rank} expects {self.n1 - self.n0} weight scales, got {tuple(w_scale_local.shape)}")
        self.W_local = W_local
        self.w_scale_local = w_scale_local
        self.gamma = gamma
        self.eps = eps
        self._takes_out = local_fn is None       # the CUDA operator writes into a caller's buffer; stand-ins return a new one
        if local_fn is None:
            from .ops import rmsnorm_linear as local_fn
        self.local_fn = local_fn
        self.sizes = [b - a for a, b in (shard_bounds(N_total, self.world, r, multiple) for r in range(self.world))]
        self.block = -(-max(self.sizes) // 8) * 8   # rows of a block start on 16-byte boundaries (bf16)
        self._buf: Optional[torch.Tensor] = None    # [G, M, block]
        self._row_major: Optional[torch.Tensor] = None

    def _buffer(self, M: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        b = self._buf
        if b is None or b.shape[1] != M or b.dtype != dtype or b.device != device:
            b = torch.zeros((self.world, M, self.block), dtype=dtype, device=device)
            self._buf = b
            self._row_major = None
        return b

    def forward(self, x: torch.Tensor, into_gather_buffer: bool = True) -> torch.Tensor:
        """y[:, n0:n1] for this rank.  No communication.  With `into_gather_buffer` the result lives in this
        rank's block of the gather buffer (and is overwritten by the next call with the same M)."""
        kw = {} if self.w_scale_local is None else {"w_scale": self.w_scale_local}
        if self.world > 1 and into_gather_buffer and self._takes_out:
            mine = self._buffer(x.shape[0], torch.bfloat16, x.device)[self.rank, :, : self.n1 - self.n0]
            return self.local_fn(x, self.gamma, self.W_local, self.eps, out=mine, **kw)
        return self.local_fn(x, self.gamma, self.W_local, self.eps, **kw)

    def gather(self, y_local: torch.Tensor, layout: str = "row_major") -> torch.Tensor:
        """Assemble y on every rank from the ranks' column blocks: [M, N_total] (`row_major`), or the blocked
        [M, G, Nb] view of the gather buffer (`blocked`, no copy; columns beyond a block's width are padding)."""
        if layout not in ("row_major", "blocked"):
            raise ValueError("layout must be 'row_major' or 'blocked'")
        M = y_local.shape[0]
        if self.world == 1:
            return y_local if layout == "row_major" else y_local.unsqueeze(1)
        buf = self._buffer(M, y_local.dtype, y_local.device)
        mine = buf[self.rank, :, : self.n1 - self.n0]
        if y_local.data_ptr() != mine.data_ptr():
            mine.copy_(y_local)                    # a result that was not produced in place
        # in place: block `rank` of the output is this rank's contribution
        dist.all_gather_into_tensor(buf.view(self.world * M, self.block), buf[self.rank], group=self.group)
        if layout == "blocked":
            return buf.permute(1, 0, 2)
        out = self._row_major
        if out is None or out.shape[0] != M:
            out = torch.empty((M, self.N_total), dtype=y_local.dtype, device=y_local.device)
            self._row_major = out
        if len(set(self.sizes)) == 1 and self.block == self.sizes[0]:
            out.view(M, self.world, self.block).copy_(buf.permute(1, 0, 2))
        else:
            col = 0
            for r, sz in enumerate(self.sizes):
                out[:, col:col + sz] = buf[r, :, :sz]
                col += sz
        return out
