"""Host-side logic that needs no GPU: argument checks of the Python operator, shard arithmetic,
and the column-parallel gather run as two gloo ranks on the CPU with the oracle standing in for
the device kernel."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import kernel_benchmarking_b200 as kb
from kernel_benchmarking_b200.sharding import ColumnParallelRMSNormLinear, shard_bounds, shard_rows
from oracle import rmsnorm_linear_oracle as orc


def test_operator_rejects_cpu_tensors_and_bad_shapes():
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    W = torch.zeros(8, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        kb.rmsnorm_linear(x, None, W, 1e-6)   # no CPU path: must refuse, not fall back
    with pytest.raises(TypeError):
        kb.rmsnorm_linear([1, 2], None, W)


@pytest.mark.parametrize("N,world", [(57344, 1), (57344, 2), (57344, 4), (57344, 8), (14336, 8), (1000, 3), (8, 4), (7, 2)])
def test_shard_bounds_partition(N, world):
    prev = 0
    sizes = []
    for r in range(world):
        a, b = shard_bounds(N, world, r)
        assert a == prev and b >= a
        if r < world - 1:
            assert a % 8 == 0 and b % 8 == 0
        prev = b
        sizes.append(b - a)
    assert prev == N
    if N % (8 * world) == 0:
        assert len(set(sizes)) == 1 and sizes[0] == N // world


def test_shard_bounds_config_sizes():
    assert [shard_bounds(57344, g, 0)[1] for g in (1, 2, 4, 8)] == [57344, 28672, 14336, 7168]
    assert shard_bounds(14336, 8, 7) == (12544, 14336)
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, N, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K = 24, 128
        x, gm, W = orc.make_inputs(M, N, K, seed=5, dtype=torch.float32)

        def cpu_stand_in(x_, g_, W_, eps):
            return orc.torch_rmsnorm_linear(x_, g_, W_, eps)

        op = ColumnParallelRMSNormLinear(shard_rows(W, world, rank), gm, 1e-6, N, local_fn=cpu_stand_in)
        y_local = op.forward(x)
        n0, n1 = shard_bounds(N, world, rank)
        full = orc.torch_rmsnorm_linear(x, gm, W, 1e-6)
        ok_local = torch.allclose(y_local, full[:, n0:n1], rtol=1e-5, atol=1e-6)
        y = op.gather(y_local)
        ok_full = y.shape == full.shape and torch.allclose(y, full, rtol=1e-5, atol=1e-6)
        # the blocked layout is the gather buffer as it lies: element [m, r, j] is y[m, n0_r + j]
        yb = op.gather(y_local, layout="blocked")
        ok_full = ok_full and yb.shape[:2] == (M, world)
        for r in range(world):
            a, b = shard_bounds(N, world, r)
            ok_full = ok_full and torch.allclose(yb[:, r, : b - a], full[:, a:b], rtol=1e-5, atol=1e-6)
        ok_full = ok_full and op.gather(y_local).data_ptr() == y.data_ptr()     # buffers are kept between calls
        # e4m3 weights: the rank's slice of the per-channel scales travels with its rows of W
        Wq, wsc = orc.quantize_weight_e4m3(W)

        def cpu_stand_in_fp8(x_, g_, Wq_, eps, w_scale):
            return orc.torch_rmsnorm_linear(x_, g_, Wq_.float() * w_scale[:, None], eps)

        op8 = ColumnParallelRMSNormLinear(shard_rows(Wq, world, rank), gm, 1e-6, N, local_fn=cpu_stand_in_fp8,
                                          w_scale_local=shard_rows(wsc, world, rank))
        full8 = orc.torch_rmsnorm_linear(x, gm, Wq.float() * wsc[:, None], 1e-6)
        y8 = op8.gather(op8.forward(x))
        ok_full = ok_full and torch.allclose(y8, full8, rtol=1e-5, atol=1e-6)
        q.put((rank, bool(ok_local), bool(ok_full)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N", [64, 72])   # equal blocks (all_gather_into_tensor) and ragged blocks
def test_column_parallel_gather_two_gloo_ranks(N):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, N, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=10) for _ in procs)
    assert res == [(0, True, True), (1, True, True)]


def test_wrong_shard_size_is_rejected():
    W = torch.zeros(10, 16)
    with pytest.raises(ValueError, match="rows of W"):
        ColumnParallelRMSNormLinear(W, None, 1e-6, 64, local_fn=lambda *a: None)
    with pytest.raises(ValueError, match="weight scales"):
        ColumnParallelRMSNormLinear(torch.zeros(64, 16), None, 1e-6, 64, local_fn=lambda *a: None,
                                    w_scale_local=torch.zeros(10))


def test_harness_csv_contract(tmp_path):
    """Rows concatenate with the reference's CSVs: same columns, same order, appended."""
    from kernel_benchmarking_b200 import harness
    assert harness.ExperimentRow.header() == ("label,m,n,k,ms_median,ms_mean,ms_std,max_abs,max_rel,rmse,"
                                              "baseline_speedup,metadata,autotune_seconds")
    row = harness.ExperimentRow("rmsnorm_linear:1:b200", 4096, 4096, 4096, ms_median=0.1, ms_mean=0.11, ms_std=0.01)
    assert row.csv().startswith("rmsnorm_linear:1:b200,4096,4096,4096,0.1,0.11,0.01,None")
    p = tmp_path / "out.csv"
    harness.write_rows([row], str(p))
    harness.write_rows([row], str(p))
    assert p.read_text().count("\n") == 2
    assert len(harness.RMSNORM_LINEAR_SHAPES) == 10 and harness.RMSNORM_LINEAR_SHAPES[1] == (4096, 4096, 4096)
    with pytest.raises(IndexError):
        harness.rmsnorm_linear_job(10)       # the reference's run script walks off the table at index 10 too


def test_harness_metrics_and_distribution():
    from kernel_benchmarking_b200 import harness
    ref = torch.tensor([[1.0, -2.0], [0.5, 4.0]])
    out = torch.tensor([[1.5, -2.0], [0.5, 3.0]])
    assert abs(harness.rmse(ref, out) - (1.25 / 4) ** 0.5) < 1e-12
    max_abs, max_rel = harness.max_errors(ref, out)
    assert max_abs == 1.0 and abs(max_rel - 0.5) < 1e-7     # 0.5 / max(|1|, 1) vs 1 / 4
    g = torch.Generator().manual_seed(1)
    t = harness.normal_bernoulli((2000, 500), generator=g)
    assert 0.9 < float(t.std()) < 1.2 and float(t.abs().max()) > 8.0


def test_harness_command_lines(tmp_path):
    """Both of the reference's entry styles parse, the batch driver writes the header and visits every config once."""
    from kernel_benchmarking_b200 import harness
    assert harness.is_old_style(["4096", "1024", "4096"]) and harness.is_old_style(["2048", "2048", "2048", "--to_csv"])
    assert not harness.is_old_style(["3"]) and not harness.is_old_style(["3", "--csv", "x.csv"]) and not harness.is_old_style([])
    ns = harness.parse_old_style(["4096", "1536", "7168", "--to_csv"])
    assert (ns.m, ns.n, ns.k, ns.to_csv) == (4096, 1536, 7168, True)
    ns = harness.parse_new_style(["7", "--csv", "r.csv", "--ncu"])
    assert (ns.config, ns.csv, ns.ncu, ns.workload, ns.shapes) == (7, "r.csv", True, "rmsnorm_linear", "gemm")
    # the four shapes the second list adds to the table
    assert set(harness.EXTRA_SHAPES) - set(harness.RMSNORM_LINEAR_SHAPES) == {
        (1024, 32768, 4096), (1024, 4096, 16384), (8192, 1024, 2048), (8192, 2048, 4096)}
    seen = []
    csv = tmp_path / "res" / "all.csv"
    assert harness.run_all(str(csv), runner=lambda cmd: seen.append(cmd) or 0) == 0
    assert csv.read_text() == harness.ExperimentRow.header() + "\n"
    assert [c[3] for c in seen] == [str(i) for i in range(10)]           # stops at index 9
    assert all(c[1:3] == ["-m", "kernel_benchmarking_b200.harness"] and str(csv) in c for c in seen)
    seen.clear()
    harness.run_all(str(csv), shapes="extra", runner=lambda cmd: seen.append(cmd) or 0)
    assert len(seen) == 7 and all("extra" in c for c in seen)


def test_harness_metadata_column():
    from kernel_benchmarking_b200 import harness
    md = harness.throughput_metadata(4096, 4096, 4096, 0.1)
    assert md == "tflops=1374.4;pct_peak=61.1;gbps=1007;n_gpus=1"
    assert "," not in md                       # stays one CSV field
    assert harness.throughput_metadata(4096, 4096, 4096, None) is None
    row = harness.ExperimentRow("rmsnorm_linear:1:b200", 4096, 4096, 4096, ms_median=0.1, metadata=md)
    assert row.csv().split(",")[11] == md


def test_clock_summary_picks_the_samples_under_load():
    """On a power-capped part the loaded samples are the low clocks: they are chosen by utilisation (or power),
    never by clock value."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    idle = ["1965", "1965", "0", "180.0", "Not Active", "Not Active", "Not Active", "Not Active"]
    busy = [[str(c), "1965", "100", "990.0", "Not Active", "Not Active", "Not Active", "Active"] for c in (1320, 1350, 1290, 1410)]
    out = bench.summarize_clock_samples([idle] * 6 + busy + [idle] * 6)
    assert out["sm_mhz"] == 1335.0 and out["sm_mhz_min"] == 1290.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"] and out["samples_under_load"] == 4 and out["samples"] == 16
    # a region too short for the utilisation counter: fall back on power draw
    lag = [[str(c), "1965", "3", "950.0", "Not Active", "Not Active", "Not Active", "Active"] for c in (1500, 1480)]
    out = bench.summarize_clock_samples([idle] * 4 + lag)
    assert out["sm_mhz"] == 1490.0 and out["loaded_by"].startswith("power")
    assert bench.summarize_clock_samples([])["sm_mhz"] is None


def test_bench_ranks_hold_slices_of_one_layer():
    """bench.py's synthetic layer: every rank generates the same x and gamma, and its rows of W are a slice of one
    weight matrix whatever the sharding."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    dev = torch.device("cpu")
    full = bench.make_buffers(8, 0, 1024, 64, dev, 2, seed=18)
    parts = [bench.make_buffers(8, a, b, 64, dev, 2, seed=18) for a, b in ((0, 512), (512, 1024), (768, 1024))]
    for s in range(2):
        for part, (a, b) in zip(parts, ((0, 512), (512, 1024), (768, 1024))):
            assert torch.equal(part[s][0], full[s][0]) and torch.equal(part[s][1], full[s][1])     # x, gamma replicated
            assert torch.equal(part[s][2], full[s][2][a:b])                                          # W rows [a, b)
    assert not torch.equal(full[0][2], full[1][2])       # the rotating buffer sets differ
    x, gm, Wq, y, wsc = bench.make_buffers(8, 256, 768, 64, dev, 1, seed=18, fp8=True)[0]
    assert Wq.dtype == torch.float8_e4m3fn and wsc.shape == (512,) and y.shape == (8, 512)
    for kernel in ("prefill_pair_prescaled", "prefill_pair_prestats"):
        assert bench.dram_traffic(kernel, 16384, 57344, 8192)[0] == 8 * bench.dram_traffic(kernel, 16384, 7168, 8192)[0]
    assert bench.dram_traffic("decode", 3, 28672, 4096)[0] is None
