"""Host-buffer front end: activations arrive in pinned host memory, results go back to it.

The reference moves its inputs to the device once, outside the timed region
(`ProfilingTensor._set_tensors`, python/profile_utils.py:296-308).  A serving loop cannot: every
step's activations come from the host and every step's result is read back.  This class keeps
the weights resident and pipelines the three stages of a step on three streams - copy-in of step
i+1, kernel of step i, copy-out of step i-1 - so a stream of steps runs at the speed of the
slowest stage (PCIe copy-out of y for the large-M shapes) instead of their sum.
"""
from __future__ import annotations

from typing import Optional

import torch

from .ops import rmsnorm_linear


class HostRMSNormLinear:
    """y_host = rmsnorm_linear(x_host, gamma, W, eps) with device-resident gamma / W (/ w_scale).

    `submit(x_host, y_host)` enqueues one step and returns immediately; `wait()` blocks until
    everything submitted so far has landed in its `y_host`.  Host tensors must be pinned.
    """

    def __init__(self, gamma: Optional[torch.Tensor], W: torch.Tensor, eps: float = 1e-6, *,
                 w_scale: Optional[torch.Tensor] = None, max_tokens: int, depth: int = 2, variant="auto"):
        if not W.is_cuda:
            raise ValueError("W must live on the device: there is no CPU path")
        self.gamma, self.W, self.eps, self.w_scale, self.variant = gamma, W, eps, w_scale, variant
        self.device = W.device
        self.depth = depth
        N, K = W.shape
        self.K, self.N = K, N
        with torch.cuda.device(self.device):
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream() for _ in range(3))
            self.x_dev = [torch.empty((max_tokens, K), dtype=torch.bfloat16, device=self.device) for _ in range(depth)]
            self.y_dev = [torch.empty((max_tokens, N), dtype=torch.bfloat16, device=self.device) for _ in range(depth)]
            self.ev_in = [torch.cuda.Event() for _ in range(depth)]
            self.ev_run = [torch.cuda.Event() for _ in range(depth)]
            self.ev_out = [torch.cuda.Event() for _ in range(depth)]
        self.step = 0

    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        if x_host.is_cuda or y_host.is_cuda:
            raise ValueError("submit() takes host tensors")
        if not (x_host.is_pinned() and y_host.is_pinned()):
            raise ValueError("host tensors must be pinned (torch.Tensor.pin_memory) for asynchronous copies")
        M = x_host.shape[0]
        if x_host.shape != (M, self.K) or y_host.shape != (M, self.N) or M > self.x_dev[0].shape[0]:
            raise ValueError("x_host must be [M, K] and y_host [M, N] with M <= max_tokens")
        i = self.step % self.depth
        reuse = self.step >= self.depth
        x_d, y_d = self.x_dev[i][:M], self.y_dev[i][:M]
        with torch.cuda.stream(self.s_in):
            if reuse:
                self.s_in.wait_event(self.ev_run[i])     # the kernel that last read this x slot is done
            x_d.copy_(x_host, non_blocking=True)
            self.ev_in[i].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[i])
            if reuse:
                self.s_run.wait_event(self.ev_out[i])    # the copy-out that last read this y slot is done
            rmsnorm_linear(x_d, self.gamma, self.W, self.eps, w_scale=self.w_scale, out=y_d, variant=self.variant)
            self.ev_run[i].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[i])
            y_host.copy_(y_d, non_blocking=True)
            self.ev_out[i].record(self.s_out)
        self.step += 1

    def wait(self) -> None:
        self.s_out.synchronize()
        self.s_run.synchronize()
        self.s_in.synchronize()
