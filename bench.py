#!/usr/bin/env python
"""Benchmark of the fused RMSNorm -> Linear operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--no-extra]

One step = one pass of the operator over one batch of seeded synthetic input.

Default workload, at every N: the bf16 prefill MLP gate+up layer x [16384, 8192] @ W [57344, 8192]^T with
gamma, W split along N over the N ranks (strong scaling: the whole job is the same at every N; N = 1 runs
the whole layer on one GPU), x replicated, no collective on the data path.  Launched by torchrun for
N > 1, one rank per GPU.  Rank 0 prints ONE JSON line.

  value       whole-job TFLOP/s (2 M N K per step over all ranks), inputs resident in HBM, CUDA events on
              the launching stream, max over ranks; `--steps` steps are timed in each of 5 windows and the
              median window is reported (all windows are listed)
  e2e         the same through the host-buffer call: pinned host x -> device, kernel, y -> pinned host,
              all inside the timed region
  roofline    the kernel's achieved TFLOP/s (GB/s for the M <= 64 workloads) against the measured peak
  parity      after the timed region every rank checks all of its y[:, n0:n1] against the reference's torch
              path in fp32 on its GPU; the line carries max |y - y_ref| / max |y_ref| over the whole tensor
  extra       further workloads, each with its own ms_per_step and roofline: the prefill QKV projection
              (4096 x 6144 x 4096), the M <= 64 sweep in GB/s, the 8192 x 14336 x 4096 shape with bf16 and
              e4m3 weights and their ratio; at N > 1 the e4m3 layer split along N
  cpu_baseline  the reference's torch path (rms_norm then matmul, fp32) on the host cores, on a bounded
              row sample of the same workload (N = 1 only)

--impl reference times that CPU path alone, on the same configuration and sample, as the main value.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# name -> (M, N, K, bound, fp8).  "tensor": TFLOP/s against the bf16 tensor peak; "hbm": GB/s against copy
# bandwidth.  N is the whole layer; with more than one rank it is split along N.
WORKLOADS = {
    "mlp_16384x57344x8192": (16384, 57344, 8192, "tensor", False),
    "prefill_qkv_4096x6144x4096": (4096, 6144, 4096, "tensor", False),
    "decode_1x28672x4096": (1, 28672, 4096, "hbm", False),
    "decode_4x28672x4096": (4, 28672, 4096, "hbm", False),
    "decode_16x28672x4096": (16, 28672, 4096, "hbm", False),
    "decode_64x28672x4096": (64, 28672, 4096, "hbm", False),
    "mlp_shard8_16384x7168x8192": (16384, 7168, 8192, "tensor", False),
    "mlp_shard4_16384x14336x8192": (16384, 14336, 8192, "tensor", False),
    "mlp_shard2_16384x28672x8192": (16384, 28672, 8192, "tensor", False),
    "bf16_8192x14336x4096": (8192, 14336, 4096, "tensor", False),
    "fp8w_8192x14336x4096": (8192, 14336, 4096, "tensor", True),   # e4m3 weights + per-channel scales
    "fp8w_decode_16x28672x4096": (16, 28672, 4096, "hbm", True),   # e4m3 weights at decode size: half the bytes
    "prefill_m128_128x6144x4096": (128, 6144, 4096, "tensor", False),  # half a row tile of tokens
    # the neighbouring operators of the reference's tables, for profiling (N = output channels)
    "swiglu_4096x14336x4096": (4096, 14336, 4096, "tensor", False),    # rmsnorm -> [gate; up] GEMM -> silu(gate) * up
    "lora_4096x4096x4096": (4096, 4096, 4096, "tensor", False),        # x W^T + (x A^T) B^T, lora_dim 16
}
LORA_DIM = 16
DEFAULT_WORKLOAD = "mlp_16384x57344x8192"
EXTRA_1GPU = ["prefill_qkv_4096x6144x4096", "decode_1x28672x4096", "decode_4x28672x4096", "decode_16x28672x4096",
              "decode_64x28672x4096", "bf16_8192x14336x4096", "fp8w_8192x14336x4096", "fp8w_decode_16x28672x4096"]
EXTRA_MULTI = ["fp8w_8192x14336x4096"]
# DRAM bytes (read + written) per launch of the dominant kernel, from one profiler capture each, keyed by the
# kernel variant and the per-GPU shape it was captured on.  A run whose variant or shape is not listed reports null.
MEASURED_DRAM_BYTES = {
    # 256 x 512 tiles on the gamma-folded copy of x (what AUTO runs on the default workload and its column shards);
    # the pre-pass that writes the copy adds up to 4 M K bytes
    ("prefill_pair_wide", 16384, 57344, 8192): 13150.0e6,   # the two DRAM byte counters alone: a one-pass capture, taken at full size
    ("prefill_pair_wide", 16384, 7168, 8192): 2116.6e6,
    ("prefill_pair_wide", 16384, 14336, 8192): 5276.3e6,
    ("prefill_pair_wide", 16384, 28672, 8192): 6705.4e6,    # (12.5 GB before the pairs re-aligned at tile boundaries)
    ("prefill_pair_wide", 8192, 14336, 4096): 682.3e6,
    # 256 x 256 tiles on the copy (by name on these shapes)
    ("prefill_pair_prescaled", 4096, 6144, 4096): 125.6e6,
    ("prefill_pair_prescaled", 16384, 7168, 8192): 2332.6e6,
    ("prefill_pair_prescaled", 16384, 14336, 8192): 4895.8e6,
    # gamma folded in the main loop (by name on these shapes; AUTO runs it for N < 6144)
    ("prefill_pair_prestats", 4096, 6144, 4096): 130.4e6,
    ("prefill_pair_prestats", 16384, 7168, 8192): 2230.5e6,
    ("prefill_pair_prestats", 16384, 14336, 8192): 4638.0e6,
    ("e4m3 pair kernel", 8192, 14336, 4096): 354.0e6,       # the GEMM kernel; the quantisation pre-pass adds 74 MB
    ("decode", 1, 28672, 4096): 240.3e6,
    ("decode", 16, 28672, 4096): 240.2e6,
    ("decode", 64, 28672, 4096): 242.4e6,
    ("e4m3 decode", 16, 28672, 4096): 122.0e6,
}
# The default workload's launches (3.4 GB on the device at N = 1) are too large for a multi-pass capture; the two DRAM
# byte counters on their own are one pass and were taken on it directly (13.15 GB per launch on 256 x 512 tiles).
# For the 256 x 256 kernels, which AUTO no longer runs on that shape, the captures of its column shards grow in
# proportion to the weight rows (x 2.10 for twice the rows), so a shard of N rows is given the 7168-row capture's
# bytes times N / 7168, and the line says that it is scaled.
SCALED_FROM = {"prefill_pair_prescaled": ("prefill_pair_prescaled", 16384, 7168, 8192),
               "prefill_pair_prestats": ("prefill_pair_prestats", 16384, 7168, 8192)}


def dram_traffic(kernel, M, N, K):
    """(bytes per launch or None, how it was obtained)."""
    v = MEASURED_DRAM_BYTES.get((kernel, M, N, K))
    if v is not None:
        return v, "one ncu capture of this kernel at this shape"
    base = SCALED_FROM.get(kernel)
    if base is not None:
        _, m0, n0, kk0 = base
        if (M, K) == (m0, kk0) and N % 256 == 0 and N > n0:
            return MEASURED_DRAM_BYTES[base] * N / n0, (f"scaled by N / {n0} from an ncu capture of {m0}x{n0}x{kk0} "
                                                        "(measured proportional to the weight rows)")
    return None, "no capture for this kernel and shape"


L2_BYTES = 126 * 1024 * 1024
WINDOWS = 5
EPS = 1e-6
CPU_SAMPLE_ROWS = 256      # rows of the default workload the CPU legs run (both arms use the same sample)


def algorithmic_bytes(M, N, K, fp8=False):
    return 2 * M * K + (1 if fp8 else 2) * N * K + (4 * N if fp8 else 0) + 2 * K + 2 * M * N


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def metric_name(bound):
    return ("fused RMSNorm+Linear TFLOP/s (% TC peak) at M>=4096" if bound == "tensor"
            else "fused RMSNorm+Linear HBM GB/s at M<=64")


class ClockSampler:
    """Samples nvidia-smi clocks, utilisation, power and throttle reasons of one GPU while a timed region runs.
    The SM clock reported is that of the samples taken under load (GPU utilisation >= 50 %, or, if the
    utilisation counter lags behind a short region, power draw within 40 % of the highest seen): on a
    power-capped part the loaded samples are the LOW clocks, so they cannot be picked by clock value."""

    Q = ("clocks.sm,clocks.max.sm,utilization.gpu,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 50):
        self.index, self.period_ms = index, period_ms
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(self.period_ms / 1000.0 + 0.02)
        self.proc.terminate()   # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        return summarize_clock_samples(self.samples)


def summarize_clock_samples(samples):
    rows, reasons, mx = [], set(), None
    for p in samples:
        try:
            clk, mx_, util, power = float(p[0]), float(p[1]), float(p[2]), float(p[3])
        except ValueError:
            continue
        mx = mx_
        rows.append((clk, util, power))
        for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[4:8]):
            if v.lower().startswith("active"):
                reasons.add(name)
    loaded = [r for r in rows if r[1] >= 50.0]
    how = "utilization.gpu >= 50"
    if not loaded and rows:
        pmax = max(r[2] for r in rows)
        loaded = [r for r in rows if r[2] >= 0.6 * pmax]
        how = "power.draw >= 0.6 x max"
    clocks = sorted(r[0] for r in loaded)
    return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_mhz_min": clocks[0] if clocks else None,
            "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(rows), "samples_under_load": len(loaded),
            "power_w_max": max((r[2] for r in rows), default=None), "loaded_by": how}


def shard_range(N, world, rank):
    from kernel_benchmarking_b200.sharding import shard_bounds
    return shard_bounds(N, world, rank, multiple=256)


W_CHUNK = 256   # weight rows generated per seeded chunk (shards are multiples of it)


def make_buffers(M, n0, n1, K, dev, sets, seed, fp8=False):
    """`sets` independent (x, gamma, W, y, w_scale) groups, generated on the device, so that consecutive steps never
    find their inputs in L2.  x and gamma depend only on (seed, set): every rank holds the same ones (x is
    replicated).  W is rows [n0, n1) of one layer whose rows are generated chunk by chunk from (seed, set, chunk):
    whatever the sharding, the ranks hold slices of the same weight matrix."""
    out = []
    N = n1 - n0
    for s in range(sets):
        g = torch.Generator(device=dev).manual_seed(seed + 7919 * s)
        x = torch.randn(M, K, generator=g, dtype=torch.float32, device=dev).to(torch.bfloat16)
        gamma = (1.0 + 0.1 * torch.randn(K, generator=g, dtype=torch.float32, device=dev)).to(torch.bfloat16)
        W = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        for c0 in range(n0 - n0 % W_CHUNK, n1, W_CHUNK):
            gw = torch.Generator(device=dev).manual_seed((seed + 7919 * s) * 100003 + c0 // W_CHUNK + 1)
            chunk = (torch.randn(W_CHUNK, K, generator=gw, dtype=torch.float32, device=dev) * K ** -0.5).to(torch.bfloat16)
            lo, hi = max(c0, n0), min(c0 + W_CHUNK, n1)
            W[lo - n0:hi - n0] = chunk[lo - c0:hi - c0]
        wsc = None
        if fp8:
            # per-output-channel absmax / 448 scales, weights stored as e4m3 codes
            wsc = (W.float().abs().amax(dim=1) / 448.0).clamp_min(1e-30)
            W = (W.float() / wsc[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
        out.append((x, gamma, W, torch.empty(M, N, dtype=torch.bfloat16, device=dev), wsc))
    return out


def parity_check(bufs, eps):
    """(max |y - y_ref|, max |y_ref|) over this rank's WHOLE y, y_ref = the reference's torch path (rms_norm then
    matmul) in fp32 on the GPU with TF32 off, computed block by block.  The caller takes the maxima over all ranks
    before dividing, so the figure is the metric of the tolerance - max |y - y_ref| / max |y_ref| over the whole
    tensor - however y is sharded."""
    import torch.nn.functional as F
    x, gamma, W, y, wsc = bufs
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        M, N = x.shape[0], W.shape[0]
        xn = F.rms_norm(x.float(), (x.shape[1],), weight=gamma.float(), eps=eps)
        max_err = torch.zeros((), device=x.device)
        max_ref = torch.zeros((), device=x.device)
        for n0 in range(0, N, 8192):
            n1 = min(N, n0 + 8192)
            Wf = W[n0:n1].float()
            if wsc is not None:
                Wf = Wf * wsc[n0:n1, None]
            for m0 in range(0, M, 2048):
                m1 = min(M, m0 + 2048)
                ref = xn[m0:m1] @ Wf.t()
                max_err = torch.maximum(max_err, (y[m0:m1, n0:n1].float() - ref).abs().max())
                max_ref = torch.maximum(max_ref, ref.abs().max())
        return max_err, max_ref
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def parity_over_ranks(bufs, eps, fp8, world):
    """max |y - y_ref| / max |y_ref| over the whole (sharded) tensor, and the tolerance it is held to."""
    max_err, max_ref = parity_check(bufs, eps)
    t = torch.stack([max_err, max_ref]).double()
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0] / t[1]), (3e-2 if fp8 else 1e-2)


def cpu_reference(M, N, K, rows, budget_s, steps=None, warmup=1):
    """The reference's torch path on the host cores, fp32, on `rows` rows of the workload (all N, all K).  Returns
    seconds per pass (median), passes, threads."""
    from oracle import rmsnorm_linear_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)     # torchrun pins OMP_NUM_THREADS=1 for its workers
    g = torch.Generator().manual_seed(18)
    x = torch.randn(rows, K, generator=g, dtype=torch.float32)
    gm = 1.0 + 0.1 * torch.randn(K, generator=g, dtype=torch.float32)
    W = torch.empty(N, K, dtype=torch.float32)
    for n0 in range(0, N, 8192):
        W[n0:min(N, n0 + 8192)].normal_(0.0, K ** -0.5, generator=g)
    for _ in range(max(warmup, 1)):
        orc.torch_rmsnorm_linear(x, gm, W, EPS)
    times, t_all = [], time.perf_counter()
    while (steps is not None and len(times) < steps) or (
            steps is None and (len(times) < 3 or (time.perf_counter() - t_all < budget_s and len(times) < 20))):
        t0 = time.perf_counter()
        orc.torch_rmsnorm_linear(x, gm, W, EPS)
        times.append(time.perf_counter() - t0)
    return statistics.median(times), sum(times) / len(times), len(times), torch.get_num_threads()


def cpu_sample_rows(workload):
    M = WORKLOADS[workload][0]
    return M if workload != DEFAULT_WORKLOAD else min(M, CPU_SAMPLE_ROWS)


def cpu_value(M_rows, N, K, bound, sec):
    if bound == "tensor":
        return 2.0 * M_rows * N * K / sec / 1e12, "TFLOP/s"
    return (4 * M_rows * K + 4 * N * K + 4 * K + 4 * M_rows * N) / sec / 1e9, "GB/s"


def cpu_sample_text(rows, M, N, K, threads):
    return (f"{rows} of {M} rows x all N={N}, K={K}; fp32 torch CPU path of the reference (rms_norm then matmul), "
            f"{threads} threads of {os.cpu_count()} cpus")


def run_reference_arm(args, rank):
    """The reference's own implementation of the path (its torch operator) on the host cores, same configuration,
    metric and sample as the other arm's `cpu_baseline`; rank 0 only."""
    if rank != 0:
        return
    M, N, K, bound, _ = WORKLOADS[args.workload]
    rows = cpu_sample_rows(args.workload)
    _, mean, n, threads = cpu_reference(M, N, K, rows, 0.0, steps=args.steps, warmup=args.warmup)
    value, unit = cpu_value(rows, N, K, bound, mean)
    sample = cpu_sample_text(rows, M, N, K, threads)
    line = {
        "impl": "reference", "metric": metric_name(bound), "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "N": N, "K": K, "eps": EPS, "gamma": True, "sample": sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_extra and args.workload == DEFAULT_WORKLOAD:
        m2, n2, k2, b2, _ = WORKLOADS["prefill_qkv_4096x6144x4096"]
        med, _, n, threads = cpu_reference(m2, n2, k2, m2, 8.0)
        v2, u2 = cpu_value(m2, n2, k2, b2, med)
        line["extra"] = {"prefill_qkv_4096x6144x4096": {
            "value": v2, "unit": u2, "ms_per_step": med * 1e3, "sample": cpu_sample_text(m2, m2, n2, k2, threads)}}
    print(json.dumps(line), flush=True)


class Runner:
    """One workload on this rank's GPU: buffers, the step, timing windows, parity."""

    def __init__(self, kb, name, dev, rank, world, variant="auto", gamma=True):
        self.kb, self.name, self.dev, self.rank, self.world, self.variant = kb, name, dev, rank, world, variant
        self.M, self.N_total, self.K, self.bound, self.fp8 = WORKLOADS[name]
        self.op = name.split("_")[0] if name.split("_")[0] in ("swiglu", "lora") else "linear"
        self.gamma = gamma
        n0, n1 = shard_range(self.N_total, world, rank) if world > 1 else (0, self.N_total)
        self.n0, self.n1, self.N = n0, n1, n1 - n0
        self.step_bytes = algorithmic_bytes(self.M, self.N, self.K, self.fp8)
        self.flops = 2.0 * self.M * self.N * self.K                    # this rank's share
        self.flops_total = 2.0 * self.M * self.N_total * self.K
        self.sets = max(2, -(-2 * L2_BYTES // self.step_bytes))        # rotate enough buffer sets to exceed 2x L2
        w0, w1 = (n0, n1) if self.op != "swiglu" else (0, 2 * self.N)
        self.bufs = make_buffers(self.M, w0, w1, self.K, dev, self.sets, seed=18, fp8=self.fp8)
        if self.op == "swiglu":      # W is [2N, K] (gate rows, then up rows), y [M, N]
            self.bufs = [(x, g, W, y[:, : self.N].contiguous(), w) for (x, g, W, y, w) in self.bufs]
        if self.op == "lora":
            gen = torch.Generator(device=dev).manual_seed(5 + rank)
            self.lA = (torch.randn(LORA_DIM, self.K, generator=gen, device=dev) * self.K ** -0.5).to(torch.bfloat16)
            self.lB = torch.randn(self.N, LORA_DIM, generator=gen, device=dev).to(torch.bfloat16)
        self.stream = torch.cuda.current_stream()
        self.kernel = "e4m3 pair kernel" if self.M > 64 else "e4m3 decode"
        if self.op != "linear":
            self.kernel = self.op
        elif not self.fp8:
            from kernel_benchmarking_b200 import _lib
            v = _lib.load().rl_select_variant(self.M, self.N, self.K, 1 if gamma else 0, 1)
            self.kernel = _lib.VARIANT_NAMES.get(v, str(v)) if variant == "auto" else str(variant)
        # kernels launched per step: the pre-pass (row statistics / quantisation) and the GEMM, or one fused kernel
        self.launches_per_step = 2 if (self.fp8 or any(t in self.kernel for t in ("prestats", "prescaled", "wide"))) else 1

    def step(self, i):
        x, g, W, y, wsc = self.bufs[i % self.sets]
        if self.op == "swiglu":
            self.kb.rmsnorm_swiglu(x, g, W, EPS, out=y)
        elif self.op == "lora":
            self.kb.lora_linear(x, W, self.lA, self.lB, out=y)
        else:
            self.kb.rmsnorm_linear(x, g if self.gamma else None, W, EPS, w_scale=wsc, out=y,
                                   variant="auto" if self.fp8 else self.variant)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def warm(self, warmup, spin_s=0.0):
        for i in range(warmup):
            self.step(i)
        t0, i = time.perf_counter(), 0
        while time.perf_counter() - t0 < spin_s:      # bring the part to its loaded state before the windows
            self.step(i)
            i += 1
            if i % 8 == 0:
                torch.cuda.synchronize()
        self.barrier()

    def windows(self, steps, n_windows):
        """ms per step of each window: `steps` steps bracketed by a barrier + synchronize, CUDA events on the
        launching stream, max over ranks."""
        out = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(n_windows):
            self.barrier()
            e0.record(self.stream)
            for i in range(steps):
                self.step(i)
            e1.record(self.stream)
            self.barrier()
            out.append(e0.elapsed_time(e1))
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor(out, device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out = t.tolist()
        return [ms / steps for ms in out]

    def value(self, ms_step):
        if self.bound == "tensor":
            return self.flops_total / (ms_step * 1e-3) / 1e12, "TFLOP/s"
        # HBM-bound workloads are not sharded here: every rank streams its own W
        return self.world * self.step_bytes / (ms_step * 1e-3) / 1e9, "GB/s"

    def roofline(self, ms_step, peaks):
        if self.bound == "tensor":
            achieved, unit = self.flops / (ms_step * 1e-3) / 1e12, "TFLOP/s"
            peak = peaks["bf16_tflops"] * (2 if self.fp8 else 1)
            sustained = peaks["bf16_tflops_sustained"] * (2 if self.fp8 else 1)
            src = f"of {peaks['source']} cuBLAS bf16 burst" + (" x 2 (no FP8 peak was measured)" if self.fp8 else "")
        else:
            achieved, unit = self.step_bytes / (ms_step * 1e-3) / 1e9, "GB/s"
            peak, sustained = peaks["hbm_gbs"], None
            src = f"of {peaks['source']} copy bandwidth"
        r = {"bound": "tensor" if self.bound == "tensor" else "hbm", "achieved": achieved, "peak": peak, "unit": unit,
             "frac": achieved / peak, "peak_source": src,
             "traffic": dram_traffic(self.kernel, self.M, self.N, self.K)[0],
             "traffic_source": dram_traffic(self.kernel, self.M, self.N, self.K)[1], "kernel": self.kernel,
             "algorithmic_bytes": self.step_bytes, "algorithmic_flops": self.flops}
        if sustained:
            r["peak_sustained"] = sustained
            r["frac_of_sustained"] = achieved / sustained
        return r

    def free(self):
        self.bufs = None
        torch.cuda.empty_cache()


def run_extra(kb, name, dev, rank, world, steps, warmup, peaks, cpu_leg):
    """One entry of the `extra` block."""
    r = Runner(kb, name, dev, rank, world)
    # short kernels: enough steps per window for a stable figure, and a short spin so clocks settle under load
    est_steps = max(steps, 20) if r.bound == "tensor" else max(steps, 100)
    sampler = ClockSampler(dev.index).start() if rank == 0 else None
    r.warm(warmup, spin_s=0.15)
    ms = r.windows(est_steps, 3)
    clocks = sampler.stop() if sampler else None
    kb.check_status()
    err, tol = parity_over_ranks(r.bufs[(est_steps - 1) % r.sets], EPS, r.fp8, world)
    med = statistics.median(ms)
    value, unit = r.value(med)
    entry = {"value": value, "unit": unit, "ms_per_step": med, "ms_per_step_windows": ms, "steps": est_steps,
             "M": r.M, "N_per_gpu": r.N, "K": r.K, "scaling": "strong" if (world > 1 and r.bound == "tensor") else "replicas",
             "dtype": "e4m3 x e4m3 -> f32 (bf16 in/out)" if r.fp8 else "bf16", "roofline": r.roofline(med, peaks),
             "parity_max_rel_err": err, "parity_ok": err <= tol,
             "clocks": None if clocks is None else {k: clocks[k] for k in ("sm_mhz", "sm_mhz_min", "reasons", "samples_under_load")}}
    r.free()
    if cpu_leg:
        sec, _, n, threads = cpu_reference(r.M, r.N_total, r.K, r.M, 8.0)
        cv, cu = cpu_value(r.M, r.N_total, r.K, r.bound, sec)
        entry["cpu_baseline"] = {"value": cv, "unit": cu, "cores": threads, "kind": "port",
                                 "sample": cpu_sample_text(r.M, r.M, r.N_total, r.K, threads) + f", median of {n} runs"}
    return entry


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--variant", default="auto", help="kernel variant name (see kernel_benchmarking_b200._lib.VARIANTS)")
    ap.add_argument("--no-extra", action="store_true", help="only the main workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gamma", action="store_true",
                    help="gamma = None, the reference operator's own form (profiling runs only)")
    ap.add_argument("--profile", action="store_true",
                    help="only warm-up + timed steps of the workload (no clock sampling, e2e, extras or CPU legs): "
                         "the command a profiler wraps")
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
    peaks = measured_peaks()

    if (args.no_gamma or args.workload.split("_")[0] in ("swiglu", "lora")) and not args.profile:
        raise SystemExit("--no-gamma and the swiglu / lora workloads are for --profile runs")
    run = Runner(kb, args.workload, dev, rank, world, variant=args.variant, gamma=not args.no_gamma)
    M, N, K = run.M, run.N, run.K

    if args.profile:
        run.warm(args.warmup)
        ms = run.windows(args.steps, 1)[0]
        if rank == 0:
            v, u = run.value(ms)
            print(json.dumps({"profile_run": True, "workload": args.workload, "kernel": run.kernel, "ms_per_step": ms,
                              "value": v, "unit": u}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- device-resident timing: 5 windows of --steps steps, clocks sampled throughout
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    run.warm(args.warmup, spin_s=0.3)
    win_ms = run.windows(args.steps, WINDOWS)
    clocks = sampler.stop() if sampler else None
    kb.check_status()
    ms_step = statistics.median(win_ms)
    value, unit = run.value(ms_step)

    # ---------------- parity of this rank's shard, outside the timed region
    parity_err, tol = parity_over_ranks(run.bufs[(args.steps - 1) % run.sets], EPS, run.fp8, world)

    # ---------------- end to end: host buffers, copies inside the timed region
    # Through the package's host-buffer front end: every step copies its x from pinned host memory and its y
    # (this rank's columns) back to pinned host memory; the three stages of consecutive steps overlap on three streams.
    x_host = [run.bufs[i][0].cpu().pin_memory() for i in range(2)]
    y_host = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    host_op = kb.HostRMSNormLinear(run.bufs[0][1], run.bufs[0][2], EPS, w_scale=run.bufs[0][4], max_tokens=M, depth=2,
                                   variant=args.variant)
    e2e_steps = max(3, min(args.steps, 8))
    for i in range(2):
        host_op.submit(x_host[i % 2], y_host[i % 2])
    host_op.wait()
    run.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(host_op.s_in)
    for i in range(e2e_steps):
        host_op.submit(x_host[i % 2], y_host[i % 2])
    e1.record(host_op.s_out)
    host_op.wait()
    run.barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_ms /= e2e_steps
    e2e_value = run.value(e2e_ms)[0]
    # the copied-back result is the kernel's: same bits as the device-resident run on the same inputs
    e2e_same = bool(torch.equal(y_host[(e2e_steps - 1) % 2], _rerun(kb, run, x_host[(e2e_steps - 1) % 2], args.variant)))
    del host_op, y_host, x_host
    torch.cuda.empty_cache()

    # ---------------- optional assembled-y all-gather, timed on its own
    gather = None
    if world > 1 and run.bound == "tensor" and not run.fp8:
        from kernel_benchmarking_b200.sharding import ColumnParallelRMSNormLinear
        x, g, W, _, _ = run.bufs[0]
        op = ColumnParallelRMSNormLinear(W, g, EPS, run.N_total, multiple=256)
        y_local = op.forward(x)                      # lands in this rank's block of the gather buffer
        res = {}
        for layout in ("blocked", "row_major"):
            for _ in range(2):
                op.gather(y_local, layout=layout)
            run.barrier()
            e0.record(run.stream)
            for _ in range(5):
                op.gather(y_local, layout=layout)
            e1.record(run.stream)
            run.barrier()
            t = torch.tensor([e0.elapsed_time(e1) / 5], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[layout] = float(t.item())
        recv = 2.0 * M * (run.N_total - N)           # bytes this rank receives
        gather = {"ms_blocked": res["blocked"], "ms_row_major": res["row_major"],
                  "received_gb_per_s_blocked": recv / (res["blocked"] * 1e-3) / 1e9,
                  "note": "NCCL all-gather of y [M, N] in place into a [G, M, N/G] buffer the kernel wrote its block "
                          "into (blocked); row_major adds one strided copy of the whole tensor"}
        del op, y_local
        torch.cuda.empty_cache()

    line = None
    if rank == 0:
        line = {
            "metric": metric_name(run.bound), "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if run.bound == "tensor" else "replicas",
            "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 (bf16 in/out)" if run.fp8 else "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "M": M, "N_total": run.N_total, "N_per_gpu": N, "K": K, "eps": EPS,
                       "gamma": True,
                       "sharding": f"W split along N over {world} rank(s), x replicated, no collective on the data path",
                       "l2": f"inputs larger than L2: {run.sets} rotating buffer sets of {run.step_bytes / 1e6:.0f} MB",
                       "variant": args.variant, "kernel": run.kernel, "windows": WINDOWS,
                       "timing": f"median of {WINDOWS} windows of {args.steps} steps, each bracketed by barrier + "
                                 "synchronize, CUDA events, max over ranks"},
            "ms_per_step_windows": win_ms,
            "ms_per_step_spread": (max(win_ms) - min(win_ms)) / ms_step,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": 2 * M * K, "d2h_bytes_per_step": 2 * M * N,
                    "ms_per_step": e2e_ms, "steps": e2e_steps, "same_bits_as_device_run": e2e_same,
                    "note": "HostRMSNormLinear: x from pinned host memory and this rank's y back to pinned host memory "
                            "every step (bytes are per rank), copy-in / kernel / copy-out of consecutive steps "
                            "overlapped on three streams; W and gamma are weights, resident on the device"},
            "gpu_launches": WINDOWS * args.steps * world * run.launches_per_step,
            "roofline": run.roofline(ms_step, peaks),
            "parity_checked": True, "parity_max_rel_err": parity_err, "parity_tolerance": tol,
            "parity_ok": parity_err <= tol,
            "parity_note": "max |y - y_ref| / max |y_ref| over the WHOLE tensor: every rank compares all of its "
                           "y[:, n0:n1] with rms_norm + matmul in fp32 (TF32 off) on its GPU, maxima taken over ranks",
        }
        if gather is not None:
            line["gather_ms"] = gather["ms_blocked"]
            line["gather"] = gather
    run.free()

    # ---------------- further workloads
    if not args.no_extra and args.workload == DEFAULT_WORKLOAD:
        extra = {}
        for name in (EXTRA_1GPU if world == 1 else EXTRA_MULTI):
            cpu_leg = (world == 1 and name == "prefill_qkv_4096x6144x4096" and not args.no_cpu_baseline)
            extra[name] = run_extra(kb, name, dev, rank, world, args.steps, args.warmup, peaks, cpu_leg and rank == 0)
        if rank == 0:
            b, f = extra.get("bf16_8192x14336x4096"), extra.get("fp8w_8192x14336x4096")
            if b and f:
                extra["fp8_over_bf16"] = f["value"] / b["value"]
            line["extra"] = extra

    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            rows = cpu_sample_rows(args.workload)
            sec, _, n, threads = cpu_reference(run.M, run.N_total, run.K, rows, 12.0)
            cv, cu = cpu_value(rows, run.N_total, run.K, run.bound, sec)
            line["cpu_baseline"] = {"value": cv, "unit": cu, "cores": threads, "kind": "port",
                                    "sample": cpu_sample_text(rows, run.M, run.N_total, run.K, threads) + f", median of {n} runs"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _rerun(kb, run, x_host, variant):
    """The device-resident result for one host batch (same weights as the end-to-end front end uses)."""
    _, g, W, _, wsc = run.bufs[0]
    y = kb.rmsnorm_linear(x_host.to(run.dev), g, W, EPS, w_scale=wsc, variant="auto" if run.fp8 else variant)
    torch.cuda.synchronize()
    return y.cpu()


if __name__ == "__main__":
    main()
