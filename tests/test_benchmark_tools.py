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
