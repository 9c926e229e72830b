"""bench.py's host-side helpers (no GPU): roofline arithmetic, workload labels, thread count, CPU reference sample."""
import importlib.util
import os
from pathlib import Path

from oracle import oracle as O

ROOT = Path(__file__).resolve().parents[1]
spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)

PEAKS = {"hbm_gbs": 6553.6, "bf16_tflops": 1621.0, "bf16_tflops_sustained": 1347.5, "source": "measured"}


def test_roofline_entry_small_m_is_held_against_hbm():
    case = O.CONFIGS["c3"]
    r = bench.roofline_entry("c3", case, float(case.flops), 7.2e-6, PEAKS, False)
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["peak"] == 6553.6
    assert abs(r["achieved"] - case.algorithmic_bytes / 7.2e-6 / 1e9) < 1e-6
    assert abs(r["frac"] - r["achieved"] / 6553.6) < 1e-12
    assert r["traffic"] == bench.NCU_TRAFFIC_BYTES["c3"]


def test_roofline_entry_tensor_bound_picks_burst_or_sustained_peak():
    case = O.CONFIGS["c5"]
    burst = bench.roofline_entry("c5", case, float(case.flops), 5.7e-3, PEAKS, False)
    long_ = bench.roofline_entry("c5", case, float(case.flops), 6.0e-3, PEAKS, True)
    assert burst["bound"] == long_["bound"] == "tensor"
    assert burst["peak"] == 1621.0 and "burst" in burst["peak_source"]
    assert long_["peak"] == 1347.5 and "sustained" in long_["peak_source"]
    assert abs(burst["achieved"] - case.flops / 5.7e-3 / 1e12) < 1e-6
    # a sharded run's per-launch traffic was never captured: it reports none rather than the whole GEMM's
    shard = bench.roofline_entry("c5_nshard", case, float(case.flops) / 8, 0.69e-3, PEAKS, False)
    assert shard["traffic"] is None


def test_workload_label_is_the_same_in_both_arms():
    case = O.CONFIGS["c2"]
    assert bench.workload_label("c2", case) == "c2: bf16 'nt' M=2048 N=4096 K=4096 +bias -> bf16"
    assert bench.workload_label("c3", O.CONFIGS["c3"]).endswith("-> fp32")


def test_host_threads_ignores_omp_num_threads(monkeypatch):
    monkeypatch.setenv("OMP_NUM_THREADS", "1")  # what torch.distributed.run sets for every rank
    assert bench.host_threads() == max(1, len(os.sched_getaffinity(0)))


def test_cpu_reference_sample_is_bounded_and_described():
    r = bench.cpu_reference_run(O.CONFIGS["c1"], seconds_budget=0.5, max_reps=3)
    assert r["rows"] == 256 and r["tflops"] > 0 and r["cores"] == bench.host_threads()
    assert "256 of 256 rows" in r["sample"] and r["flops_full"] == O.CONFIGS["c1"].flops
