"""Column-parallel use of the operator on several GPUs of one node.

W [N, K] is split into contiguous row blocks (= column blocks of y) over the
ranks; x and gamma are replicated; each rank runs the unmodified single-GPU
kernel on its block, so the hot path has no collective.  Only when the caller
asks for the assembled y is an all-gather issued (NCCL over NVLink on GPUs),
and it is timed separately by the benchmark.  The reference project has no
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
        if local_fn is None:
            from .ops import rmsnorm_linear as local_fn
        self.local_fn = local_fn

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """y[:, n0:n1] for this rank.  No communication."""
        if self.w_scale_local is not None:
            return self.local_fn(x, self.gamma, self.W_local, self.eps, w_scale=self.w_scale_local)
        return self.local_fn(x, self.gamma, self.W_local, self.eps)

    def gather(self, y_local: torch.Tensor) -> torch.Tensor:
        """Assemble y [M, N_total] on every rank from the ranks' column blocks."""
        if self.world == 1:
            return y_local
        M = y_local.shape[0]
        sizes = [b - a for a, b in (shard_bounds(self.N_total, self.world, r, self.multiple)
                                    for r in range(self.world))]
        out = torch.empty((M, self.N_total), dtype=y_local.dtype, device=y_local.device)
        if len(set(sizes)) == 1:
            # equal blocks: one all-gather into [G, M, N/G], then one strided copy into place
            buf = torch.empty((self.world * M, sizes[0]), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(buf, y_local.contiguous(), group=self.group)
            out.view(M, self.world, sizes[0]).copy_(buf.view(self.world, M, sizes[0]).permute(1, 0, 2))
        else:
            # ragged blocks: pad every block to the widest, gather, then copy each block into place
            wmax = max(sizes)
            padded = torch.zeros((M, wmax), dtype=y_local.dtype, device=y_local.device)
            padded[:, : y_local.shape[1]] = y_local
            buf = torch.empty((self.world * M, wmax), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(buf, padded, group=self.group)
            buf = buf.view(self.world, M, wmax)
            col = 0
            for r, sz in enumerate(sizes):
                out[:, col:col + sz] = buf[r, :, :sz]
                col += sz
        return out
