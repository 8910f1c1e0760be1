#!/usr/bin/env python3
"""Run the distributed-GEMM experiment suite: every shape case x (method, partition triple,
replication factor), one ``torchrun`` launch per case, and merge the per-case records into
``results.json`` / ``results.csv`` (the format ``render_benchmark_report.py`` reads).

Command line and output schema follow the reference's runner
(benchmark/run_matmul_experiments.py:288-312, :255-285, :404-413).  Additions: ``--dtype`` /
``--device`` are forwarded to the worker, each case has a ``--case-timeout``, and ``--resume``
skips cases whose ``result.json`` already exists in the output directory.
"""
from __future__ import annotations

import argparse
import csv
import datetime as dt
import json
import os
import pathlib
import socket
import subprocess
import sys
from dataclasses import asdict

THIS_DIR = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(THIS_DIR.parent))

from universal_gemm_b200.models.workloads import (  # noqa: E402
    MethodCase, ShapeCase, build_shape_suite, case_key, merged_row,
)

WORKER = THIS_DIR / "matmul_bench_worker.py"
METHODS = ("dtensor", "stationary_c", "stationary_b", "auto")
PARTS = {"row": "row", "column": "column", "col": "column", "block": "block"}


def parse_csv_list(value: str) -> list[str]:
    return [x.strip() for x in value.split(",") if x.strip()]


def parse_int_list(value: str) -> list[int]:
    return [int(x) for x in parse_csv_list(value)]


def parse_partition_triples(value: str) -> list[tuple[str, str, str]]:
    triples = []
    for item in (x.strip() for x in value.split(";")):
        if not item:
            continue
        parts = [p.strip() for p in item.split(",")]
        if len(parts) != 3 or any(p not in PARTS for p in parts):
            raise ValueError("Partition triples must be formatted as 'a,b,c;a,b,c;...' with each value in "
                             "{row,column,block}")
        triples.append(tuple(PARTS[p] for p in parts))
    return triples


def default_output_dir() -> pathlib.Path:
    return THIS_DIR / "results" / f"matmul_suite_{dt.datetime.now().strftime('%Y%m%d_%H%M%S')}"


def worker_command(args, shape: ShapeCase, method: MethodCase, port: int, result_file: pathlib.Path, seed: int) -> list[str]:
    cmd = [args.python, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.nproc_per_node}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(WORKER),
           "--method", method.method, "--dim-m", str(shape.m), "--dim-n", str(shape.n), "--dim-k", str(shape.k),
           "--a-partition", method.a_partition, "--b-partition", method.b_partition,
           "--c-partition", method.c_partition, "--replication-factor", str(method.replication_factor),
           "--warmup-iters", str(args.warmup_iters), "--measure-iters", str(args.measure_iters),
           "--seed", str(seed), "--result-file", str(result_file), "--device", args.device]
    if args.dtype:
        cmd += ["--dtype", args.dtype]
    if args.verify:
        cmd += ["--verify"]
    if args.theoretical_tflops is not None:
        cmd += ["--theoretical-tflops", str(args.theoretical_tflops)]
    return cmd


def run_case(args, shape: ShapeCase, method: MethodCase, index: int, output_dir: pathlib.Path) -> dict:
    case_dir = output_dir / "runs" / case_key(shape, method)
    case_dir.mkdir(parents=True, exist_ok=True)
    result_file, log_file = case_dir / "result.json", case_dir / "torchrun.log"
    if not (args.resume and result_file.exists()):
        if result_file.exists():
            result_file.unlink()
        cmd = worker_command(args, shape, method, args.master_port_base + index % 1000, result_file, args.seed + index)
        env = dict(os.environ, MASTER_ADDR="127.0.0.1")
        try:
            proc = subprocess.run(cmd, cwd=str(THIS_DIR.parent), env=env, text=True, capture_output=True,
                                  timeout=args.case_timeout or None)
            out, err, code = proc.stdout, proc.stderr, proc.returncode
        except subprocess.TimeoutExpired as exc:
            out, err, code = (exc.stdout or ""), (exc.stderr or ""), -9
            out = out.decode() if isinstance(out, bytes) else out
            err = err.decode() if isinstance(err, bytes) else err
        log_file.write_text((out or "") + ("\n" if out and err else "") + (err or ""), encoding="utf-8")
        if code != 0:
            raise RuntimeError(f"Benchmark case failed (exit={code}): {' '.join(cmd)}\nSee log: {log_file}")
        if not result_file.exists():
            raise RuntimeError(f"Worker completed without result file: {result_file}")
    return merged_row(shape, method, json.loads(result_file.read_text(encoding="utf-8")))


def write_results(output_dir: pathlib.Path, payload: dict) -> None:
    (output_dir / "results.json").write_text(json.dumps(payload, indent=2), encoding="utf-8")
    rows = payload["results"]
    with open(output_dir / "results.csv", "w", encoding="utf-8", newline="") as f:
        if not rows:
            csv.writer(f).writerow(["no_results"])
            return
        columns = sorted({k for r in rows for k in r})
        writer = csv.DictWriter(f, fieldnames=columns)
        writer.writeheader()
        writer.writerows(rows)


def parse_args(argv=None) -> argparse.Namespace:
    import torch

    p = argparse.ArgumentParser(description="Run the distributed GEMM experiment suite")
    p.add_argument("--python", type=str, default=sys.executable)
    p.add_argument("--nproc-per-node", type=int, default=max(torch.cuda.device_count(), 1))
    p.add_argument("--master-port-base", type=int, default=29600)
    p.add_argument("--warmup-iters", type=int, default=3)
    p.add_argument("--measure-iters", type=int, default=10)
    p.add_argument("--seed", type=int, default=20260218)
    p.add_argument("--methods", type=str, default="dtensor,stationary_c,stationary_b")
    p.add_argument("--replication-factors", type=str, default="1,2")
    p.add_argument("--partition-triples", type=str, default="row,row,row;row,column,row;block,block,block",
                   help="Semicolon-separated 'a,b,c' triples")
    p.add_argument("--gpt3-m-values", type=str, default="1024,2048,4096,8192")
    p.add_argument("--square-sizes", type=str, default="1024,2048,4096,8192")
    p.add_argument("--odd-large-values", type=str, default="4096,8192,16384,32768")
    p.add_argument("--odd-small-value", type=int, default=1024)
    p.add_argument("--max-cases", type=int, default=0, help="0 means run all")
    p.add_argument("--theoretical-tflops", type=float, default=None)
    p.add_argument("--continue-on-error", action="store_true")
    p.add_argument("--output-dir", type=str, default=str(default_output_dir()))
    p.add_argument("--dtype", choices=["bf16", "fp32"], default=None)
    p.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--case-timeout", type=float, default=900.0, help="seconds per case; 0 disables")
    p.add_argument("--resume", action="store_true", help="skip cases that already have a result.json")
    p.add_argument("--verify", action="store_true")
    return p.parse_args(argv)


def enumerate_cases(args) -> list[tuple[ShapeCase, MethodCase]]:
    methods = parse_csv_list(args.methods)
    for method in methods:
        if method not in METHODS:
            raise ValueError(f"Unsupported method {method!r}")
    shapes = build_shape_suite(gpt3_m_values=parse_int_list(args.gpt3_m_values),
                               square_sizes=parse_int_list(args.square_sizes),
                               odd_large_values=parse_int_list(args.odd_large_values),
                               odd_small_value=args.odd_small_value)
    method_cases = [MethodCase(method, a, b, c, rep)
                    for method in methods
                    for rep in parse_int_list(args.replication_factors) if args.nproc_per_node % rep == 0
                    for (a, b, c) in parse_partition_triples(args.partition_triples)]
    if not method_cases:
        raise RuntimeError("No runnable method/partition/replication combinations generated.")
    cases = [(s, mc) for s in shapes for mc in method_cases]
    return cases[: args.max_cases] if args.max_cases > 0 else cases


def main(argv=None) -> None:
    args = parse_args(argv)
    if args.nproc_per_node <= 0:
        raise ValueError("--nproc-per-node must be positive")
    cases = enumerate_cases(args)
    output_dir = pathlib.Path(args.output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    results, failures = [], []
    for idx, (shape, method) in enumerate(cases):
        print(f"[{idx + 1}/{len(cases)}] {shape.experiment_group} (m={shape.m}, n={shape.n}, k={shape.k}) "
              f"method={method.method} parts={method.a_partition}/{method.b_partition}/{method.c_partition} "
              f"rep={method.replication_factor}", flush=True)
        try:
            results.append(run_case(args, shape, method, idx, output_dir))
        except Exception as exc:  # noqa: BLE001
            failures.append({"index": idx, "shape_case": asdict(shape), "method_case": asdict(method), "error": str(exc)})
            print(f"  FAILED: {exc}", flush=True)
            if not args.continue_on_error:
                break
    write_results(output_dir, {
        "created_at": dt.datetime.now().isoformat(), "host": socket.gethostname(),
        "nproc_per_node": args.nproc_per_node, "warmup_iters": args.warmup_iters, "measure_iters": args.measure_iters,
        "theoretical_tflops": args.theoretical_tflops, "results": results, "failures": failures})
    print(f"Wrote {len(results)} successful results and {len(failures)} failures to {output_dir}", flush=True)
    if failures and not args.continue_on_error:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
