"""Worker for the multi-GPU column-parallel test: one process per GPU (launched by torchrun)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import kernel_benchmarking_b200 as kb  # noqa: E402
from kernel_benchmarking_b200.sharding import ColumnParallelRMSNormLinear, shard_bounds, shard_rows  # noqa: E402
from oracle import rmsnorm_linear_oracle as orc  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    for (M, N, K) in [(300, 1024, 512), (16, 2048, 1024), (1000, 1032, 256)]:
        x, gm, W = orc.make_inputs(M, N, K, seed=7)           # identical on every rank
        op = ColumnParallelRMSNormLinear(shard_rows(W, world, rank).contiguous().to(dev), gm.to(dev), 1e-6, N)
        y_local = op.forward(x.to(dev))               # written straight into this rank's block of the gather buffer
        y = op.gather(y_local)
        torch.cuda.synchronize()
        kb.check_status()
        ref = orc.reference_fp32(x, gm, W, 1e-6)
        err = orc.rel_max_err(y.cpu(), ref)
        ok = ok and y.shape == (M, N) and err <= 1e-2
        yb = op.gather(y_local, layout="blocked")     # [M, G, Nb]: no copy behind the all-gather
        torch.cuda.synchronize()
        for r in range(world):
            a, b = shard_bounds(N, world, r)
            ok = ok and torch.equal(yb[:, r, : b - a], y[:, a:b])
        ok = ok and y_local.data_ptr() == yb[:, rank].data_ptr()
        # the single-GPU kernel on the whole weight gives the same columns: to one bf16 ulp (2^-7), since tiles of
        # the last round may be summed in k-slices and which tiles those are depends on the shard's tile count
        if M > 64 and rank == 0:
            y_full = kb.rmsnorm_linear(x.to(dev), gm.to(dev), W.to(dev), 1e-6)
            ok = ok and orc.rel_max_err(y_full[:, op.n0:op.n1], y_local.float()) <= 2.0 ** -7
    # e4m3 weights: each rank holds its rows of Wq and its slice of the per-channel scales
    M, N, K = 256, 1024, 1024
    x, gm, W = orc.make_inputs(M, N, K, seed=8)
    Wq, wsc = orc.quantize_weight_e4m3(W)
    op = ColumnParallelRMSNormLinear(shard_rows(Wq, world, rank).contiguous().to(dev), gm.to(dev), 1e-6, N,
                                     w_scale_local=shard_rows(wsc, world, rank).contiguous().to(dev))
    y = op.gather(op.forward(x.to(dev)))
    torch.cuda.synchronize()
    kb.check_status()
    ref = orc.reference_fp32(x, gm, Wq, 1e-6, w_scale=wsc)
    ok = ok and y.shape == (M, N) and orc.rel_max_err(y.cpu(), ref) <= 5e-2   # the FP8 tolerance at small K
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
