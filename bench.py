#!/usr/bin/env python
"""Benchmark of the fused RMSNorm -> Linear operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one pass of the operator over one batch of seeded synthetic input.
Default workload: the bf16 prefill QKV projection x [4096, 4096] @ W [6144, 4096]^T.
With N > 1 (launched by torchrun, one rank per GPU) W is column-sharded: every
rank holds its own [6144, 4096] block of a [6144 * N, 4096] weight, x is
replicated, no collective on the data path (weak scaling).  Rank 0 prints ONE
JSON line.

  value     whole-job TFLOP/s (2 M N K per step), inputs resident in HBM, timed
            with CUDA events on the launching stream, max over ranks
  e2e       the same through the host-buffer call: pinned host x -> device,
            kernel, y -> pinned host, all inside the timed region
  roofline  the kernel's achieved TFLOP/s (or GB/s for the M <= 64 workloads)
            against the measured peak of this GPU pool
  cpu_baseline  the reference's torch path (rms_norm then matmul) on the host
            cores, on a bounded row sample of the same workload

--impl reference times that CPU path alone, as the main value.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# name -> (M, N, K, bound).  "tensor": TFLOP/s against the bf16 tensor peak; "hbm": GB/s against copy bandwidth
WORKLOADS = {
    "prefill_qkv_4096x6144x4096": (4096, 6144, 4096, "tensor"),
    "decode_1x28672x4096": (1, 28672, 4096, "hbm"),
    "decode_4x28672x4096": (4, 28672, 4096, "hbm"),
    "decode_16x28672x4096": (16, 28672, 4096, "hbm"),
    "decode_64x28672x4096": (64, 28672, 4096, "hbm"),
    "mlp_shard8_16384x7168x8192": (16384, 7168, 8192, "tensor"),
    "mlp_shard4_16384x14336x8192": (16384, 14336, 8192, "tensor"),
    "bf16_8192x14336x4096": (8192, 14336, 4096, "tensor"),
    "fp8w_8192x14336x4096": (8192, 14336, 4096, "tensor"),   # e4m3 weights + per-channel scales
    # strong scaling: the weight is split along N over the ranks (N below is the whole layer)
    "strong_mlp_16384x57344x8192": (16384, 57344, 8192, "tensor"),
    "strong_fp8w_8192x14336x4096": (8192, 14336, 4096, "tensor"),
}
DEFAULT_WORKLOAD = "prefill_qkv_4096x6144x4096"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu summaries (profiles/)
NCU_TRAFFIC_BYTES = {
    "prefill_qkv_4096x6144x4096": 164.4e6,     # profiles/prefill_pair_kernel_4096x6144x4096_bf16.md
    "decode_16x28672x4096": 240.3e6,           # profiles/decode_kernel_16x28672x4096_bf16.md
    "fp8w_8192x14336x4096": 465.0e6,           # profiles/fp8_pair_kernel_8192x14336x4096_e4m3.md (GEMM kernel only)
}
L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(M, N, K, fp8=False):
    return 2 * M * K + (1 if fp8 else 2) * N * K + (4 * N if fp8 else 0) + 2 * K + 2 * M * N


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()   # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        for p in self.samples:
            try:
                clocks.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        # the busy half of the samples: idle samples before/after the region would drag the median down
        busy = clocks[len(clocks) // 2:] if clocks else []
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(clocks)}


def make_buffers(M, N, K, dev, sets, seed, fp8=False):
    """`sets` independent (x, gamma, W, y) groups so that consecutive steps never find their inputs in L2."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for _ in range(sets):
        x = torch.randn(M, K, generator=g, dtype=torch.float32).to(torch.bfloat16)
        gamma = (1.0 + 0.1 * torch.randn(K, generator=g, dtype=torch.float32)).to(torch.bfloat16)
        W = torch.empty(N, K, dtype=torch.bfloat16)
        # W is large: generate in slabs to bound host memory
        for n0 in range(0, N, 8192):
            n1 = min(N, n0 + 8192)
            W[n0:n1] = (torch.randn(n1 - n0, K, generator=g, dtype=torch.float32) * K ** -0.5).to(torch.bfloat16)
        Wd, wsc = W.to(dev), None
        if fp8:
            # per-output-channel absmax / 448 scales, weights stored as e4m3 codes
            wsc = (Wd.float().abs().amax(dim=1) / 448.0).clamp_min(1e-30)
            Wd = (Wd.float() / wsc[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
        out.append((x.to(dev), gamma.to(dev), Wd, torch.empty(M, N, dtype=torch.bfloat16, device=dev), x, wsc))
    return out


def cpu_reference_time(M, N, K, budget_s=15.0):
    """The reference's torch path on the host cores, fp32, on a row sample sized to ~budget_s."""
    from oracle import rmsnorm_linear_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    rows = min(M, 512)
    x, gm, W = orc.make_inputs(rows, N, K, seed=18, dtype=torch.float32)
    orc.torch_rmsnorm_linear(x, gm, W, 1e-6)   # warm-up
    times = []
    t_all = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_all < budget_s and len(times) < 20):
        t0 = time.perf_counter()
        orc.torch_rmsnorm_linear(x, gm, W, 1e-6)
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    return rows, med, len(times)


def run_reference_arm(args, rank):
    if rank != 0:
        return
    M, N, K, bound = WORKLOADS[args.workload]
    # all host cores (torchrun pins OMP_NUM_THREADS=1 for its workers; only rank 0 works here)
    torch.set_num_threads(os.cpu_count() or 1)
    # bounded sample per step: min(M, 512) rows of the workload, all N and K
    from oracle import rmsnorm_linear_oracle as orc
    rows = min(M, 512)
    x, gm, W = orc.make_inputs(rows, N, K, seed=18, dtype=torch.float32)
    for _ in range(max(args.warmup, 1)):
        orc.torch_rmsnorm_linear(x, gm, W, 1e-6)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.torch_rmsnorm_linear(x, gm, W, 1e-6)
    dt = (time.perf_counter() - t0) / args.steps
    if bound == "tensor":
        value, unit = 2.0 * rows * N * K / dt / 1e12, "TFLOP/s"
    else:
        value, unit = (4 * rows * K + 4 * N * K + 4 * K + 4 * rows * N) / dt / 1e9, "GB/s"
    cores = torch.get_num_threads()
    sample = f"{rows} of {M} rows x all N={N}, K={K}, fp32, torch CPU ({cores} threads of {os.cpu_count()} cpus)"
    print(json.dumps({
        "impl": "reference", "metric": metric_name(bound), "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "N": N, "K": K, "sample": sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def metric_name(bound):
    return ("fused RMSNorm+Linear TFLOP/s (% TC peak) at M>=4096" if bound == "tensor"
            else "fused RMSNorm+Linear HBM GB/s at M<=64")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--variant", default="auto", help="kernel variant name (see kernel_benchmarking_b200._lib.VARIANTS)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="M <= 64 workloads: time CUDA-graph replay instead of eager launches (measured: no faster, "
                         "the call costs 11 us of host time against a 43 us kernel)")
    ap.add_argument("--profile", action="store_true",
                    help="only warm-up + timed steps (no clock-sampling spin, no e2e, no CPU baseline): for ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    import torch.distributed as dist
    import kernel_benchmarking_b200 as kb

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    M, N, K, bound = WORKLOADS[args.workload]
    strong = args.workload.startswith("strong_")
    if strong:
        from kernel_benchmarking_b200.sharding import shard_bounds
        n0, n1 = shard_bounds(N, world, rank, multiple=256)
        N = n1 - n0          # this rank's block of output channels
    fp8 = "fp8w" in args.workload
    step_bytes = algorithmic_bytes(M, N, K, fp8)
    sets = max(2, -(-2 * L2_BYTES // step_bytes))   # rotate enough buffer sets to exceed 2x L2
    bufs = make_buffers(M, N, K, dev, sets, seed=18 + rank, fp8=fp8)
    stream = torch.cuda.current_stream()

    def step(i):
        x, g, W, y, _, wsc = bufs[i % sets]
        kb.rmsnorm_linear(x, g, W, 1e-6, w_scale=wsc, out=y, variant=args.variant)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-resident timing
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # keep the GPU busy long enough for nvidia-smi to sample it under load, then time exactly K steps
    t_spin = time.perf_counter()
    i = 0
    while not args.profile and time.perf_counter() - t_spin < 0.3:
        step(i)
        i += 1
        if i % 16 == 0:
            torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # optional: replay a CUDA graph that holds one step per buffer set, as a serving loop would
    use_graph = (bound == "hbm") and args.graph and not args.profile
    eager_ms = None
    if use_graph:
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        e1.record(stream)
        barrier()
        eager_ms = e0.elapsed_time(e1) / args.steps
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for i in range(sets):
                step(i)                      # workspace for this stream exists before capture starts
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(sets):
                    step(i)
        torch.cuda.current_stream().wait_stream(side)
        replays = max(1, args.steps // sets)
        for _ in range(3):
            graph.replay()
        barrier()
        e0.record(stream)
        for _ in range(replays):
            graph.replay()
        e1.record(stream)
        barrier()
        timed_steps = replays * sets
    else:
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        e1.record(stream)
        barrier()
        timed_steps = args.steps
    clocks = sampler.stop() if rank == 0 else None
    ms_total = e0.elapsed_time(e1)
    kb.check_status()
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / timed_steps
    flops = 2.0 * M * N * K
    if bound == "tensor":
        value, unit = world * flops / (ms_step * 1e-3) / 1e12, "TFLOP/s"
    else:
        value, unit = world * step_bytes / (ms_step * 1e-3) / 1e9, "GB/s"

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": args.workload, "ms_per_step": ms_step, "value": value,
                              "unit": unit}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- end to end: host buffers, copies inside the timed region
    # Through the package's host-buffer front end: every step copies its x from pinned host memory and
    # its y back to pinned host memory; the three stages of consecutive steps overlap on three streams.
    x_host = [b[4].pin_memory() for b in bufs[:2]]
    y_host = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    host_op = kb.HostRMSNormLinear(bufs[0][1], bufs[0][2], 1e-6, w_scale=bufs[0][5], max_tokens=M, depth=2,
                                   variant=args.variant)
    e2e_steps = max(3, min(args.steps, 20))
    for i in range(3):
        host_op.submit(x_host[i % 2], y_host[i % 2])
    host_op.wait()
    barrier()
    e0.record(host_op.s_in)
    for i in range(e2e_steps):
        host_op.submit(x_host[i % 2], y_host[i % 2])
    e1.record(host_op.s_out)
    host_op.wait()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_ms /= e2e_steps
    e2e_value = (world * flops / (e2e_ms * 1e-3) / 1e12) if bound == "tensor" else (world * step_bytes / (e2e_ms * 1e-3) / 1e9)

    # ---------------- optional assembled-y all-gather, timed on its own
    gather_ms = None
    if world > 1:
        from kernel_benchmarking_b200.sharding import ColumnParallelRMSNormLinear
        op = ColumnParallelRMSNormLinear(bufs[0][2], bufs[0][1], 1e-6, N * world)
        y_local = bufs[0][3]
        for _ in range(2):
            op.gather(y_local)
        barrier()
        e0.record(stream)
        for _ in range(5):
            op.gather(y_local)
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / 5], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_ms = float(t.item())

    if rank == 0:
        peaks = measured_peaks()
        per_gpu_ms = ms_step
        if bound == "tensor":
            achieved, peak, r_unit = flops / (per_gpu_ms * 1e-3) / 1e12, peaks["bf16_tflops"] * (2 if fp8 else 1), "TFLOP/s"
        else:
            achieved, peak, r_unit = step_bytes / (per_gpu_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
        line = {
            "metric": metric_name(bound), "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 (bf16 in/out)" if fp8 else "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "M": M, "N_per_gpu": N, "K": K, "eps": 1e-6, "gamma": True,
                       "sharding": f"column-parallel x{world}, x replicated, no collective",
                       "l2": f"inputs larger than L2: {sets} rotating buffer sets of {step_bytes / 1e6:.0f} MB",
                       "variant": args.variant,
                       "launch": "CUDA graph replay" if use_graph else "eager"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": 2 * M * K, "d2h_bytes_per_step": 2 * M * N,
                    "ms_per_step": e2e_ms, "note": "HostRMSNormLinear: x from pinned host memory and y back to pinned host "
                    "memory every step, copy-in / kernel / copy-out of consecutive steps overlapped on three streams; "
                    "W and gamma are weights, resident on the device"},
            # M > 128 and the FP8 path launch two kernels per step (row statistics / quantisation, then the GEMM)
            "gpu_launches": timed_steps * world * (2 if (fp8 or M > 128) else 1),
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": r_unit, "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_source": f"of {peaks['source']}" + (" bf16 x 2 (no FP8 peak was measured)" if fp8 else ""),
                         "algorithmic_bytes": step_bytes, "algorithmic_flops": flops},
        }
        if gather_ms is not None:
            line["gather_ms"] = gather_ms
        if eager_ms is not None:
            line["eager_ms_per_step"] = eager_ms
            line["steps"] = timed_steps
        if world == 1 and not args.no_cpu_baseline:
            rows, med, reps = cpu_reference_time(M, N, K)
            cores = torch.get_num_threads()
            if bound == "tensor":
                cv, cu = 2.0 * rows * N * K / med / 1e12, "TFLOP/s"
            else:
                cv, cu = (4 * rows * K + 4 * N * K + 4 * K + 4 * rows * N) / med / 1e9, "GB/s"
            line["cpu_baseline"] = {"value": cv, "unit": cu, "cores": cores, "kind": "port",
                                    "sample": f"{rows} of {M} rows x all N, K; fp32 torch CPU path of the reference "
                                              f"(rms_norm then matmul), median of {reps} runs, {cores} threads of "
                                              f"{os.cpu_count()} cpus"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
