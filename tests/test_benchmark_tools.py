"""Benchmark tooling on CPU: shape suite, case keys, suite runner (gloo ranks, resumable) and report renderer."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "benchmark"))

from universal_gemm_b200.models import MethodCase, build_shape_suite, case_key, gpt3_expansion  # noqa: E402


def test_shape_suite_and_case_key():
    suite = build_shape_suite(gpt3_m_values=[1024], square_sizes=[2048], odd_large_values=[4096], odd_small_value=1024)
    groups = [s.experiment_group for s in suite]
    assert groups == ["gpt3_expansion", "gpt3_shrinking", "square", "odd_m_large", "odd_n_large", "odd_k_large"]
    up, down = suite[0], suite[1]
    assert (up.m, up.n, up.k) == (1024, 49152, 12288) and (down.m, down.n, down.k) == (1024, 12288, 49152)
    assert suite[3].experiment_label == "Odd-dimension: large m (n=k=1024)" and (suite[5].m, suite[5].k) == (1024, 4096)
    key = case_key(gpt3_expansion(8192), MethodCase("stationary_b", "row", "column", "row", 2))
    assert key == "gpt3_expansion_m8192_n49152_k12288_stationary_b_ArowBcolumnCrow_rep2"


def test_partition_triple_parsing():
    import run_matmul_experiments as R

    assert R.parse_partition_triples("row,col,row; block,block,block") == [("row", "column", "row"), ("block",) * 3]
    with pytest.raises(ValueError):
        R.parse_partition_triples("row,diag,row")
    args = R.parse_args(["--nproc-per-node", "8", "--device", "cpu"])
    cases = R.enumerate_cases(args)
    assert len(cases) == (4 + 4 + 4 + 12) * 3 * 2 * 3     # shapes x methods x reps x triples


def test_suite_runner_resume_and_report(tmp_path):
    out = tmp_path / "suite"
    cmd = [sys.executable, os.path.join(ROOT, "benchmark", "run_matmul_experiments.py"), "--nproc-per-node", "2",
           "--device", "cpu", "--warmup-iters", "1", "--measure-iters", "2", "--methods", "dtensor,stationary_c,auto",
           "--replication-factors", "1", "--partition-triples", "row,column,row", "--gpt3-m-values", "",
           "--square-sizes", "48,64", "--odd-large-values", "", "--output-dir", str(out), "--verify",
           "--master-port-base", "29720"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    payload = json.loads((out / "results.json").read_text())
    assert len(payload["results"]) == 6 and not payload["failures"]
    row = payload["results"][0]
    for field in ("experiment_group", "experiment_label", "varied_dim", "varied_value", "case_key", "m", "n", "k",
                  "method", "a_partition", "b_partition", "c_partition", "replication_factor", "warmup_iters",
                  "measure_iters", "world_size", "median_seconds", "min_seconds", "max_seconds", "median_tflops",
                  "max_tflops", "flops", "theoretical_tflops"):
        assert field in row
    assert all(r["max_abs_error"] is None or r["max_abs_error"] < 1e-3 for r in payload["results"])
    assert (out / "results.csv").read_text().splitlines()[0].startswith("a_partition,")
    # resume: results are reused, no worker is launched (finishes within seconds)
    proc = subprocess.run(cmd + ["--resume"], capture_output=True, text=True, timeout=60)
    assert proc.returncode == 0
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "benchmark", "render_benchmark_report.py"),
                           "--results-json", str(out / "results.json")], capture_output=True, text=True, timeout=60)
    assert proc.returncode == 0
    html = (out / "report.html").read_text()
    assert "stationary_c | A=row B=column C=row | rep=1" in html and "method-toggle" in html and "<svg" not in html[:100]


def test_trace_summary_on_a_synthetic_timeline():
    """utils.trace.summarize / to_chrome_trace on a hand-made two-CTA timeline (no GPU involved)."""
    import numpy as np

    from universal_gemm_b200.utils import trace as TR

    arr = np.zeros((2, 3, 8), dtype=np.int64)          # 2 CTAs, 2 tile slots + summary
    base = 1_000_000
    for cta in range(2):
        arr[cta, 2, TR.S_START] = base + 100 * cta
        arr[cta, 2, TR.S_END] = base + 50_000
        arr[cta, 2, TR.S_FETCH_END] = base + 9_000
        arr[cta, 2, TR.S_PIECES] = 3 + cta
        for i in range(2):
            t = base + 1_000 + i * 20_000
            arr[cta, i] = [cta + 2 * i + 1, t, 500 * i, t + 15_000, t + 1_000, t + 16_000, t + 18_000, t + 19_000 + cta * 1_000]
    s = TR.summarize(arr)
    assert s["recorded_tiles"] == 4 and s["pieces_copied"] == 7
    assert abs(s["kernel_us"] - 50.0) < 1e-9 and abs(s["cta_start_spread_us"] - 0.1) < 1e-9
    assert abs(s["main_us_mean"] - 17.0) < 1e-9 and s["main_us_by_iteration"] == [17.0, 17.0]
    assert s["flagwait_us_by_iteration"] == [0.0, 0.5] and abs(s["flagwait_us_max_per_cta"] - 0.5) < 1e-9
    assert abs(s["cta_finish_spread_us"] - 1.0) < 1e-9 and abs(s["fetch_end_us"] - 9.0) < 1e-9
    ev = TR.to_chrome_trace(arr, pid=3)
    assert {e["name"] for e in ev} == {"load", "main", "epilogue", "fetch"} and all(e["pid"] == 3 for e in ev)
    assert TR.summarize(np.zeros((2, 3, 8), dtype=np.int64)) == {"grid": 2, "recorded_tiles": 0}


def test_trace_device_breakdown_adds_up_to_the_kernel_time():
    from universal_gemm_b200.utils import trace as TR

    s = {"grid": 148, "pair": False, "recorded_tiles": 148 * 10, "kernel_us": 1000.0, "flagwait_us_mean_per_cta": 20.0,
         "main_loop_share_of_kernel": 0.9, "epilogue_us_mean": 7.0}
    b = TR.device_breakdown(s)
    assert abs(sum(b.values()) - 1000e-6) < 1e-12
    assert abs(b["comm_sync"] - 20e-6) < 1e-12 and abs(b["compute"] - 880e-6) < 1e-12 and abs(b["epilogue"] - 70e-6) < 1e-12
    assert TR.device_breakdown({"grid": 2, "recorded_tiles": 0}) == {"comm_sync": 0.0, "compute": 0.0, "epilogue": 0.0,
                                                                    "other": 0.0}


@pytest.mark.parametrize("method", ["dtensor", "stationary_c", "stationary_b"])
def test_plumbing_config_cpu_gloo_1024(tmp_path, method):
    """The CPU plumbing configuration: C = A @ B, M = N = K = 1024 fp32, A / B / C row-partitioned, replication 1,
    two gloo ranks, seed 0; the plain-DTensor baseline and both stationary methods give the fp64 product."""
    result = tmp_path / "result.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29760 + ["dtensor", "stationary_c", "stationary_b"].index(method)),
           os.path.join(ROOT, "benchmark", "matmul_bench_worker.py"), "--method", method, "--dim-m", "1024",
           "--dim-n", "1024", "--dim-k", "1024", "--a-partition", "row", "--b-partition", "row", "--c-partition", "row",
           "--replication-factor", "1", "--warmup-iters", "1", "--measure-iters", "2", "--seed", "0", "--dtype", "fp32",
           "--device", "cpu", "--verify", "--result-file", str(result)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    rec = json.loads(result.read_text())
    assert rec["method"] == method and rec["world_size"] == 2 and (rec["m"], rec["n"], rec["k"]) == (1024, 1024, 1024)
    assert rec["max_abs_error"] is not None and rec["max_abs_error"] < 1e-2 and rec["median_tflops"] > 0


def test_sweep_summary_tables(tmp_path):
    """summarize_sweep.py: ratio against the dtensor comparator, best-of columns, odd-shape win count."""
    import summarize_sweep as S

    def row(method, tflops, group="gpt3_expansion", m=8192, n=49152, k=12288, c_dtype="fp32", triple=("row", "column", "row"), **kw):
        base = {"experiment_group": group, "m": m, "n": n, "k": k, "a_partition": triple[0], "b_partition": triple[1],
                "c_partition": triple[2], "replication_factor": 1, "world_size": 8, "method": method,
                "median_tflops": tflops, "c_dtype": c_dtype, "max_abs_error": 1e-5, "roofline_fraction": 0.8,
                "executed_method": "stationary_b", "tile_variant": "pair"}
        base.update(kw)
        return base

    rows = [row("dtensor", 4000.0), row("stationary_c", 5000.0), row("stationary_b", 9000.0),
            row("stationary_b", 9500.0, c_dtype="bf16"),
            row("dtensor", 100.0, group="skinny", m=64, n=16383, k=16383), row("auto", 250.0, group="skinny", m=64, n=16383, k=16383)]
    path = tmp_path / "results.json"
    path.write_text(json.dumps({"results": rows}))
    text = S.summarize(S.load([str(path)]))
    assert "### 8 GPUs" in text
    big = [ln for ln in text.splitlines() if ln.startswith("| 8192 x 49152 x 12288")][0]
    cells = [c.strip() for c in big.strip("|").split("|")]
    assert cells[3:8] == ["4000", "5000", "9000", "-", "9500"] and cells[8] == "2.25" and cells[9] == "2.38"
    assert "auto >= dtensor bf16 on 1 of 1 odd / skinny cases." in text
    assert S.main([str(path), "--output", str(tmp_path / "t.md")]) == 0 and (tmp_path / "t.md").read_text().startswith("### 8 GPUs")


def test_bench_reference_arm_without_gpu_reports_unavailable_and_arms_share_the_metric():
    """``bench.py --impl reference`` on a machine without CUDA prints the one-line ``unavailable`` record and exits 0;
    both arms take their ``metric`` string from ``bench.METRIC``; the reference arm imports nothing of the package."""
    import torch

    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    if not torch.cuda.is_available():
        line = json.loads([ln for ln in proc.stdout.splitlines() if ln.startswith("{")][-1])
        assert line["impl"] == "reference" and "unavailable" in line
    src = open(os.path.join(ROOT, "baseline", "run_reference.py"), encoding="utf-8").read()
    assert '"metric": metric' in src and "import universal_gemm_b200" not in src and "from universal_gemm_b200" not in src
    bench_src = open(os.path.join(ROOT, "bench.py"), encoding="utf-8").read()
    assert '"metric": METRIC' in bench_src and "run_reference.main(args, METRIC)" in bench_src
