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
# The reference's second shape list (res/cdsl_rmsnorm_shapes_m128n256.txt:1-7); the first three are also in the
# table above.  Its committed H100 timings for these shapes are in res/c2_kernels/results.json.
EXTRA_SHAPES: Tuple[Tuple[int, int, int], ...] = (
    (2048, 2048, 2048), (4096, 4096, 4096), (1024, 16384, 2048),
    (1024, 32768, 4096), (1024, 4096, 16384), (8192, 1024, 2048), (8192, 2048, 4096),
)
B200_DENSE_BF16_TFLOPS = 2250.0   # nominal dense bf16 tensor peak, the denominator of `pct_peak` in the metadata column
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
            torch.cuda.nvtx.range_push(self.label)     # lets a profiler pick this row's launches by name (--nvtx-include)
            try:
                out = kernel(*tensors)
            finally:
                torch.cuda.nvtx.range_pop()
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
        self.metadata = throughput_metadata(self.m, self.n, self.k, self.ms_median)


def throughput_metadata(m, n, k, ms_median, n_gpus: int = 1, elem_bytes: int = 2) -> Optional[str]:
    """The free-form `metadata` column (profile_utils.py:87): derived throughput figures, `;`-separated so the
    row stays one CSV record.  tflops = 2 m n k / time; pct_peak against the nominal dense bf16 tensor peak;
    gbps = bytes of x, W and y over time."""
    if not (m and n and k and ms_median):
        return None
    sec = ms_median * 1e-3
    tflops = 2.0 * m * n * k / sec / 1e12
    gbps = elem_bytes * (m * k + n * k + m * n) / sec / 1e9
    return (f"tflops={tflops:.1f};pct_peak={100.0 * tflops / (B200_DENSE_BF16_TFLOPS * n_gpus):.1f};"
            f"gbps={gbps:.0f};n_gpus={n_gpus}")


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


def rmsnorm_linear_job(config: int, seed: int = 18, shapes: Sequence[Tuple[int, int, int]] = RMSNORM_LINEAR_SHAPES,
                       shape: Optional[Tuple[int, int, int]] = None) -> ProfilingJob:
    """The job of demo/new_profiling/rmsnorm_linear_new.py for shape `config` of `shapes` (or an explicit `shape`,
    labelled with `config`), with the kernels that exist here: `b200` (this library), `torch` (eager rms_norm +
    matmul, the baseline), `max` (plain matmul) and `max_b200` (this library's plain GEMM)."""
    from .ops import gemm_nt, rmsnorm_linear
    if shape is None:
        if not 0 <= config < len(shapes):
            raise IndexError(f"config must be in [0, {len(shapes)})")
        shape = shapes[config]
    m, n, k = shape
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


def parse_new_style(argv=None) -> argparse.Namespace:
    """`CONFIG [--ncu] [--csv FILE]` (profile_utils.py:444-456) plus this harness's additions."""
    ap = argparse.ArgumentParser(description="Profiling program for the RMSNorm -> Linear workload (config = row of the shape table)")
    ap.add_argument("config", type=int, nargs="?", default=0, help="the config number")
    ap.add_argument("--ncu", action="store_true")
    ap.add_argument("--csv", default=None, help="append the results to csv file instead of stdout")
    ap.add_argument("--workload", default="rmsnorm_linear", choices=["rmsnorm_linear", "lora"])
    ap.add_argument("--shapes", default="gemm", choices=["gemm", "extra"],
                    help="gemm: python/workload_shapes.py GEMM_SHAPES; extra: res/cdsl_rmsnorm_shapes_m128n256.txt")
    ap.add_argument("--header", action="store_true", help="print the CSV header (demo/gen_header.py) and exit")
    ap.add_argument("--pause", type=float, default=2.0,
                    help="seconds of rest between kernels (the reference sleeps 2 s) and, with --all, 1.5 x that between configs")
    ap.add_argument("--all", action="store_true",
                    help="every config of the shape table, one process each, into --csv (run_scripts/profile_rmsnorm_linear.sh)")
    return ap.parse_args(argv)


def parse_old_style(argv) -> argparse.Namespace:
    """`m n k [--to_csv]` (`get_args`, profile_utils.py:219-234)."""
    ap = argparse.ArgumentParser(description="Profiling Program For Gemm-Based Kernel")
    ap.add_argument("m", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("--to_csv", action="store_true")   # doubles as the reference's print flag
    return ap.parse_args(argv)


def is_old_style(argv: Sequence[str]) -> bool:
    """Three leading integers select the old entry (demo/rmsnorm_linear.py), one (or none) the new one."""
    lead = []
    for a in argv:
        if a.startswith("-"):
            break
        lead.append(a)
    return len(lead) == 3 and all(x.lstrip("+").isdigit() for x in lead)


def run_old_style(ns: argparse.Namespace, out=print) -> list:
    """The old entry point (demo/rmsnorm_linear.py:40-104) for one explicit shape: rows for `torch`, `b200` and
    `max`; with --to_csv they are printed as CSV records, otherwise as the header, the value lists, the speed-up
    of the fused kernel over the baseline and the "max attainable speedup" line (baseline time over plain GEMM
    time, with the norm's own time beside it)."""
    job = rmsnorm_linear_job(0, shape=(ns.m, ns.n, ns.k))
    job.workload, job.config = "rmsnorm_linear", f"{ns.m}x{ns.n}x{ns.k}"
    rows = job.run()
    by = {r.label.split(":")[-1]: r for r in rows}
    order = [by["torch"], by["b200"], by["max"], by["max_b200"]]
    if ns.to_csv:
        for r in order:
            out(r.csv())
        return rows
    out(ExperimentRow.header())
    for r in order[:3]:
        out([getattr(r, f) for f in CSV_FIELDS])
    out(by["torch"].ms_median / by["b200"].ms_median)
    a = job.args[0]
    rmsnorm_ms = statistics.median(bench_with_l2_flush(
        lambda: torch.nn.functional.rms_norm(a, (a.shape[1],), eps=REFERENCE_EPS), min_reps=30))
    gemm_ms = by["max"].ms_median
    out(f"rmsnorm_ms={rmsnorm_ms}, gemm_ms={gemm_ms}. Max speedup = {by['torch'].ms_median / gemm_ms}")
    return rows


def run_all(csv_path: str, shapes: str = "gemm", workload: str = "rmsnorm_linear", pause_s: float = 3.0,
            runner=None, kernel_pause_s: float = 2.0) -> int:
    """The batch driver (run_scripts/profile_rmsnorm_linear.sh:6-17): write the header into the CSV (overwriting
    it), then one process per config appending its rows, a pause between them.  The reference's loop runs one
    index past its 10-row table; this one stops at the last row."""
    import os
    import subprocess
    import sys
    d = os.path.dirname(csv_path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(csv_path, "w") as f:
        f.write(ExperimentRow.header() + "\n")
    n = len(EXTRA_SHAPES if shapes == "extra" else RMSNORM_LINEAR_SHAPES)
    failed = 0
    for i in range(n):
        cmd = [sys.executable, "-m", "kernel_benchmarking_b200.harness", str(i), "--csv", csv_path, "--shapes", shapes,
               "--workload", workload, "--pause", str(kernel_pause_s)]
        rc = runner(cmd) if runner is not None else subprocess.run(cmd).returncode
        failed += 1 if rc else 0
        if runner is None and i + 1 < n:
            time.sleep(pause_s)
    return failed


def main(argv=None) -> None:
    """New style: `python -m kernel_benchmarking_b200.harness CONFIG [--workload rmsnorm_linear|lora] [--shapes gemm|extra]
    [--ncu] [--csv FILE] [--all] [--header]`; old style: `python -m kernel_benchmarking_b200.harness M N K [--to_csv]`."""
    import sys
    argv = list(sys.argv[1:] if argv is None else argv)
    if is_old_style(argv):
        run_old_style(parse_old_style(argv))
        return
    ns = parse_new_style(argv)
    if ns.header:
        print(ExperimentRow.header())
        return
    if ns.all:
        csv_path = ns.csv or time.strftime("results/rmsnorm_linear_%Y%m%d_%H%M%S.csv")
        print(f"writing csv to {csv_path}")
        raise SystemExit(1 if run_all(csv_path, ns.shapes, ns.workload, pause_s=1.5 * ns.pause, kernel_pause_s=ns.pause) else 0)
    shapes = EXTRA_SHAPES if ns.shapes == "extra" else RMSNORM_LINEAR_SHAPES
    job = lora_job(ns.config) if ns.workload == "lora" else rmsnorm_linear_job(ns.config, shapes=shapes)
    if ns.shapes == "extra":
        job.workload = "rmsnorm_linear_extra"
    write_rows(job.run(ncu=ns.ncu, pause_s=ns.pause), ns.csv)


if __name__ == "__main__":
    main()
