"""Measurement harness for the RMSNorm -> Linear workload, speaking the reference's CSV and CLI.

The reference's harness (python/profile_utils.py) cannot be imported without CuTeDSL and a live GPU
(`profile_utils.py:10` -> `cdsl_fn_utils.py:19`), so the pieces this one operator needs are provided
here to the same contract:

* rows `label,m,n,k,ms_median,ms_mean,ms_std,max_abs,max_rel,rmse,baseline_speedup,metadata,autotune_seconds`
  (field order of `ExperimentOutput`, profile_utils.py:76-88), label `"{workload}:{config}:{kernel}"`
  (profile_utils.py:419), rows appended to the CSV (profile_utils.py:114-125);
* timing: an L2 flush before every repetition, at least 10 warm-up and 100 timed repetitions, one pair of
  CUDA events per repetition on the kernel's stream (`do_bench_mod`, profile_utils.py:150-201);
* accuracy against the same operator run in fp64 on the same values (profile_utils.py:52-56,204-217,415);
* the shape table of `GEMM_SHAPES` (python/workload_shapes.py:19-33) and the N(0,1) + 10 N(0,1) Bernoulli
  input distribution (profile_utils.py:255-262).
"""
from __future__ import annotations

import argparse
import dataclasses
import statistics
import time
from typing import Callable, Dict, Optional, Sequence, Tuple

import torch

# (m, n, k) of python/workload_shapes.py:19-33, same order (config index = row)
RMSNORM_LINEAR_SHAPES: Tuple[Tuple[int, int, int], ...] = (
    (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
    (1024, 14336, 4096), (1024, 28672, 8192), (1024, 16384, 2048),
    (4096, 1024, 4096), (4096, 1024, 8192), (4096, 1536, 7168), (4096, 1024, 16384),
)
REFERENCE_EPS = 1e-5   # python/workload_shapes.py:42-47
CSV_FIELDS = ("label", "m", "n", "k", "ms_median", "ms_mean", "ms_std", "max_abs", "max_rel", "rmse",
              "baseline_speedup", "metadata", "autotune_seconds")


def rmse(ref: torch.Tensor, out: torch.Tensor) -> float:
    d = out.double().flatten() - ref.double().flatten()
    return float(d.pow(2).mean().sqrt())


def max_errors(ref: torch.Tensor, out: torch.Tensor) -> Tuple[float, float]:
    """(max |out-ref|, max |out-ref| / max(|ref|, 1)): profile_utils.py:211-217."""
    ref, out = ref.float(), out.float()
    diff = (out - ref).abs()
    return float(diff.max()), float((diff / ref.abs().clamp(min=1.0)).max())


def normal_bernoulli(shape, p: float = 0.001, dtype=torch.float64, device="cpu",
                     generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """N(0,1) + 10 N(0,1) Bernoulli(p): the reference's heavy-tailed test distribution."""
    base = torch.randn(shape, dtype=dtype, device=device, generator=generator)
    large = torch.randn(shape, dtype=dtype, device=device, generator=generator) * 10
    mask = torch.bernoulli(torch.full(shape, p, dtype=dtype, device=device), generator=generator)
    return base + large * mask


def bench_with_l2_flush(fn: Callable[[], object], warmup_ms: float = 25.0, rep_ms: float = 100.0,
                        min_reps: int = 100, stream: Optional[torch.cuda.Stream] = None) -> list:
    """Per-repetition device times in ms; L2 is flushed (a 256 MB buffer is zeroed) before each one."""
    stream = stream or torch.cuda.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.int8, device="cuda")
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(5):
        flush.zero_()
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    estimate = max(e0.elapsed_time(e1) / 5, 1e-3)
    n_warm = max(10, int(warmup_ms / estimate))
    n_rep = max(min_reps, int(rep_ms / estimate))
    for _ in range(n_warm):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_rep)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_rep)]
    for i in range(n_rep):
        flush.zero_()
        starts[i].record(stream)
        fn()
        ends[i].record(stream)
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


@dataclasses.dataclass
class ExperimentRow:
    """One CSV row, columns in the reference's order."""
    label: str
    m: Optional[int] = None
    n: Optional[int] = None
    k: Optional[int] = None
    ms_median: Optional[float] = None
    ms_mean: Optional[float] = None
    ms_std: Optional[float] = None
    max_abs: Optional[float] = None
    max_rel: Optional[float] = None
    rmse: Optional[float] = None
    baseline_speedup: Optional[float] = None
    metadata: Optional[str] = None
    autotune_seconds: Optional[float] = None

    @staticmethod
    def header() -> str:
        return ",".join(CSV_FIELDS)

    def csv(self) -> str:
        return ",".join(str(getattr(self, f)) for f in CSV_FIELDS)

    def measure(self, kernel: Callable, tensors: Sequence, ref: torch.Tensor, ncu: bool = False) -> None:
        stream = getattr(kernel, "_stream", None) or torch.cuda.current_stream()
        with torch.cuda.stream(stream):
            out = kernel(*tensors)
            if ncu:            # one launch, nothing else: the profiler wraps the process
                torch.cuda.synchronize()
                return
            torch.cuda.synchronize()
            self.rmse = rmse(ref, out)
            self.max_abs, self.max_rel = max_errors(out, ref)   # argument order as at profile_utils.py:56
            times = bench_with_l2_flush(lambda: kernel(*tensors), stream=stream)
        self.ms_median = statistics.median(times)
        self.ms_mean = statistics.fmean(times)
        self.ms_std = statistics.pstdev(times)


class ProfilingJob:
    """`kernels` maps a name to a callable; `arg_mask[name]` picks its arguments out of `args`
    (the reference's convention, demo/new_profiling/rmsnorm_linear_new.py:97-103).  The entry named
    `ref` is run on fp64 copies of the tensor arguments to produce the accuracy reference."""

    def __init__(self, workload: str, config: int, shape: Tuple[int, int, int], kernels: Dict[str, Callable],
                 args: Sequence, arg_mask: Dict[str, Sequence[int]], baseline: str, ref: str,
                 ref_args: Optional[Sequence] = None, ref_by_kernel: Optional[Dict[str, torch.Tensor]] = None):
        self.workload, self.config, self.shape = workload, config, shape
        self.kernels, self.args, self.arg_mask, self.baseline = kernels, args, arg_mask, baseline
        ra = ref_args if ref_args is not None else [a.double() if isinstance(a, torch.Tensor) and a.is_floating_point()
                                                    else a for a in args]
        self.ref_out = kernels[ref](*[ra[i] for i in arg_mask[ref]])
        self.ref_by_kernel = ref_by_kernel or {}   # e.g. the plain-GEMM lines are compared with a plain fp64 GEMM

    def run(self, ncu: bool = False, pause_s: float = 2.0) -> list:
        m, n, k = self.shape
        rows = []
        for name, fn in self.kernels.items():
            row = ExperimentRow(f"{self.workload}:{self.config}:{name}", m, n, k)
            row.measure(fn, [self.args[i] for i in self.arg_mask[name]], self.ref_by_kernel.get(name, self.ref_out),
                        ncu=ncu)
            rows.append(row)
            if not ncu:
                time.sleep(pause_s)     # let the part cool between kernels, as the reference does
        base = next((r for r in rows if r.label.endswith(":" + self.baseline)), None)
        if base is not None and base.ms_median:
            for r in rows:
                if r.ms_median:
                    r.baseline_speedup = base.ms_median / r.ms_median
        return rows


def write_rows(rows, path: Optional[str] = None) -> None:
    if path is None:
        for r in rows:
            print(r.csv())
        return
    with open(path, "a") as f:
        f.write("".join(r.csv() + "\n" for r in rows))


def rmsnorm_linear_job(config: int, seed: int = 18) -> ProfilingJob:
    """The job of demo/new_profiling/rmsnorm_linear_new.py for shape `config`, with the kernels that exist here:
    `b200` (this library), `torch` (eager rms_norm + matmul, the baseline) and `max` (plain matmul)."""
    from .ops import gemm_nt, rmsnorm_linear
    if not 0 <= config < len(RMSNORM_LINEAR_SHAPES):
        raise IndexError(f"config must be in [0, {len(RMSNORM_LINEAR_SHAPES)})")
    m, n, k = RMSNORM_LINEAR_SHAPES[config]
    g = torch.Generator().manual_seed(seed)
    a64 = normal_bernoulli((m, k), generator=g)
    b64 = normal_bernoulli((n, k), generator=g)
    a, b = a64.to(torch.bfloat16).cuda(), b64.to(torch.bfloat16).cuda()
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

    def torch_kernel(x, w, eps=REFERENCE_EPS):
        return torch.nn.functional.rms_norm(x, (x.shape[1],), eps=eps) @ w.t()

    kernels = {
        "b200": lambda x, w, eps: rmsnorm_linear(x, None, w, eps),
        "torch": torch_kernel,
        "max": lambda x, w: x @ w.t(),
        "max_b200": lambda x, w: gemm_nt(x, w),
    }
    masks = {"b200": (0, 1, 3), "torch": (0, 1, 3), "max": (0, 1), "max_b200": (0, 1)}
    ref_args = (a.double(), b.double(), None, REFERENCE_EPS)
    ref_gemm = a.double() @ b.double().t()     # demo/rmsnorm_linear.py:61,87
    return ProfilingJob("rmsnorm_linear", config, (m, n, k), kernels, (a, b, out, REFERENCE_EPS), masks,
                        baseline="torch", ref="torch", ref_args=ref_args,
                        ref_by_kernel={"max": ref_gemm, "max_b200": ref_gemm})


LORA_DIM = 16   # demo/new_profiling/lora_new.py:19


def lora_job(config: int, seed: int = 18) -> ProfilingJob:
    """The job of demo/new_profiling/lora_new.py for shape `config` (`LORA_NT_16`, python/workload_shapes.py:56-63:
    X [m, k], W [n, k], A [16, k], B [n, 16]) with `b200` (this library's fused kernel), `torch` (the reference's
    eager expression, the baseline) and `max` (the plain matmul without the low-rank term)."""
    from .ops import gemm_nt, lora_linear
    if not 0 <= config < len(RMSNORM_LINEAR_SHAPES):
        raise IndexError(f"config must be in [0, {len(RMSNORM_LINEAR_SHAPES)})")
    m, n, k = RMSNORM_LINEAR_SHAPES[config]
    g = torch.Generator().manual_seed(seed)
    x, w, la, lb = (normal_bernoulli(shape, generator=g).to(torch.bfloat16).cuda()
                    for shape in ((m, k), (n, k), (LORA_DIM, k), (n, LORA_DIM)))
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

    def torch_kernel(a, b, lA, lB):   # python/baselines/lora.py:4-13
        return (a @ b.t()) + ((a @ lA.t()) @ lB.t())

    kernels = {"b200": lora_linear, "torch": torch_kernel, "max": lambda a, b: a @ b.t(),
               "max_b200": lambda a, b: gemm_nt(a, b)}
    masks = {"b200": (0, 1, 2, 3), "torch": (0, 1, 2, 3), "max": (0, 1), "max_b200": (0, 1)}
    ref_gemm = x.double() @ w.double().t()
    return ProfilingJob("lora", config, (m, n, k), kernels, (x, w, la, lb, out), masks, baseline="torch", ref="torch",
                        ref_by_kernel={"max": ref_gemm, "max_b200": ref_gemm})


def main(argv=None) -> None:
    """`python -m kernel_benchmarking_b200.harness CONFIG [--workload rmsnorm_linear|lora] [--ncu] [--csv FILE]` - the
    new-style CLI of the reference (profile_utils.py:444-456); `--header` prints the CSV header (demo/gen_header.py)."""
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("config", type=int, nargs="?", default=0)
    ap.add_argument("--workload", default="rmsnorm_linear", choices=["rmsnorm_linear", "lora"])
    ap.add_argument("--ncu", action="store_true")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--header", action="store_true")
    ns = ap.parse_args(argv)
    if ns.header:
        print(ExperimentRow.header())
        return
    job = lora_job(ns.config) if ns.workload == "lora" else rmsnorm_linear_job(ns.config)
    write_rows(job.run(ncu=ns.ncu), ns.csv)


if __name__ == "__main__":
    main()
