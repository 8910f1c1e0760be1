#!/usr/bin/env python3
"""Run many benchmark cases inside ONE ``torchrun`` launch (process group and symmetric memory are
set up once), and write the same ``results.json`` / ``results.csv`` as ``run_matmul_experiments.py``.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmark/run_matmul_sweep.py --preset baseline --output-dir out/sweep

The per-case records come from the same ``bench_case`` as the one-launch-per-case worker; the suite
runner remains the isolated (one process group per case) way to run them.  ``--preset baseline`` is
the configuration list this repository reports against: square 8192, the two GPT-3 MLP GEMMs at
M in {2048, 8192, 32768} with their natural partition triples and replication factors, and the odd /
skinny shapes with ``auto`` over all 27 partition triples.
"""
from __future__ import annotations

import argparse
import csv
import datetime as dt
import itertools
import json
import os
import pathlib
import socket
import sys
import traceback

import torch
import torch.distributed as dist

THIS_DIR = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(THIS_DIR.parent))
sys.path.insert(0, str(THIS_DIR))

import universal_gemm_b200 as ug  # noqa: E402
from universal_gemm_b200.models.workloads import (  # noqa: E402
    MethodCase, ShapeCase, build_shape_suite, gpt3_expansion, gpt3_shrinking, merged_row, square,
)
import matmul_bench_worker as worker  # noqa: E402
from run_matmul_experiments import parse_csv_list, parse_int_list, parse_partition_triples  # noqa: E402

PARTS = ("row", "column", "block")


def preset_baseline(world_size: int, full: bool) -> list[tuple[ShapeCase, MethodCase]]:
    cases: list[tuple[ShapeCase, MethodCase]] = []
    methods = ("dtensor", "stationary_c", "stationary_b")

    def add(shape, triples, reps, meths=methods):
        for meth, rep, (a, b, c) in itertools.product(meths, reps, triples):
            if world_size % rep == 0 and rep <= world_size:
                cases.append((shape, MethodCase(meth, a, b, c, rep)))

    add(square(8192), [("row", "row", "row")], [1])
    for m in (2048, 8192, 32768):
        add(gpt3_expansion(m), [("row", "column", "row"), ("row", "row", "row")], [1, 2])
        add(gpt3_shrinking(m), [("column", "row", "row")], [1, 2, 4])
    odd_shapes = [ShapeCase("odd_cube", "Odd cube (m=n=k)", "size", s, s, s, s) for s in (3001, 12289)]
    odd_shapes.append(ShapeCase("skinny", "Skinny (m=64, n=k=16383)", "m", 64, 64, 16383, 16383))
    triples = list(itertools.product(PARTS, repeat=3)) if full else \
        [("row", "row", "row"), ("row", "column", "row"), ("column", "row", "row"), ("block", "block", "block"),
         ("block", "row", "column")]
    for shape in odd_shapes:
        add(shape, triples, [1], ("dtensor", "auto"))
    return cases


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", choices=["baseline", "baseline-full", "none"], default="none")
    ap.add_argument("--methods", default="dtensor,stationary_c,stationary_b")
    ap.add_argument("--replication-factors", default="1,2")
    ap.add_argument("--partition-triples", default="row,row,row;row,column,row;block,block,block")
    ap.add_argument("--gpt3-m-values", default="1024,2048,4096,8192")
    ap.add_argument("--square-sizes", default="1024,2048,4096,8192")
    ap.add_argument("--odd-large-values", default="4096,8192,16384,32768")
    ap.add_argument("--odd-small-value", type=int, default=1024)
    ap.add_argument("--warmup-iters", type=int, default=3)
    ap.add_argument("--measure-iters", type=int, default=10)
    ap.add_argument("--seed", type=int, default=20260218)
    ap.add_argument("--dtype", choices=["bf16", "fp32"], default=None)
    ap.add_argument("--c-dtype", choices=["bf16", "fp32"], default="fp32")
    ap.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--theoretical-tflops", type=float, default=None)
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--verify-rows", type=int, default=0, help="verify sampled rows only (0 = every row)")
    ap.add_argument("--verify-tolerance", type=float, default=None, help="fail a case above this relative error")
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="bf16 GEMM peak of one GPU (roofline fields)")
    ap.add_argument("--link-gbs", type=float, default=0.0, help="NVLink GB/s per direction per GPU (roofline fields)")
    ap.add_argument("--only-groups", default="", help="comma-separated experiment groups to keep (e.g. odd_cube,skinny)")
    ap.add_argument("--dtensor-skip-mixed-block", action="store_true",
                    help="skip dtensor cases that mix block with row / column partitions (torch refuses most of them: "
                         "operands on different device meshes; each also costs new NCCL sub-groups)")
    ap.add_argument("--cuda-graph", action="store_true", help="replay each stationary GEMM from a captured CUDA graph")
    ap.add_argument("--max-cases", type=int, default=0)
    ap.add_argument("--only-methods", default="", help="comma-separated filter applied to the case list")
    ap.add_argument("--max-m", type=int, default=0, help="skip shapes with more rows than this (0 = no limit)")
    ap.add_argument("--output-dir", default=str(THIS_DIR / "results" / f"sweep_{dt.datetime.now():%Y%m%d_%H%M%S}"))
    args = ap.parse_args()

    world = ug.init(device=args.device)
    size, rank = world.size, world.rank
    if args.preset.startswith("baseline"):
        cases = preset_baseline(size, args.preset == "baseline-full")
    else:
        shapes = build_shape_suite(gpt3_m_values=parse_int_list(args.gpt3_m_values),
                                   square_sizes=parse_int_list(args.square_sizes),
                                   odd_large_values=parse_int_list(args.odd_large_values),
                                   odd_small_value=args.odd_small_value)
        mcs = [MethodCase(meth, a, b, c, rep) for meth in parse_csv_list(args.methods)
               for rep in parse_int_list(args.replication_factors) if size % rep == 0
               for (a, b, c) in parse_partition_triples(args.partition_triples)]
        cases = [(s, mc) for s in shapes for mc in mcs]
    if args.only_methods:
        keep = set(parse_csv_list(args.only_methods))
        cases = [(s, mc) for s, mc in cases if mc.method in keep]
    if args.only_groups:
        keep_groups = set(parse_csv_list(args.only_groups))
        cases = [(s, mc) for s, mc in cases if s.experiment_group in keep_groups]
    if args.dtensor_skip_mixed_block:
        def mixed(mc):
            parts = {mc.a_partition, mc.b_partition, mc.c_partition}
            return "block" in parts and len(parts) > 1
        cases = [(s, mc) for s, mc in cases if not (mc.method == "dtensor" and mixed(mc))]
    if args.max_m > 0:
        cases = [(s, mc) for s, mc in cases if s.m <= args.max_m]
    if args.max_cases > 0:
        cases = cases[: args.max_cases]

    results, failures = [], []
    for idx, (shape, mc) in enumerate(cases):
        ns = argparse.Namespace(
            method=mc.method, m=shape.m, n=shape.n, k=shape.k, a_partition=mc.a_partition,
            b_partition=mc.b_partition, c_partition=mc.c_partition, replication_factor=mc.replication_factor,
            warmup_iters=args.warmup_iters, measure_iters=args.measure_iters, seed=args.seed + idx,
            theoretical_tflops=args.theoretical_tflops, dtype=args.dtype or ("bf16" if args.device == "cuda" else "fp32"),
            c_dtype=args.c_dtype, device=args.device, b_scale=1.0 / max(shape.k, 1) ** 0.5, verify=args.verify,
            result_file="", cuda_graph=args.cuda_graph, verify_rows=args.verify_rows,
            verify_tolerance=args.verify_tolerance, peak_tflops=args.peak_tflops, link_gbs=args.link_gbs)
        ok = torch.ones(1, device=world.device)
        try:
            rec = worker.bench_case(world, ns)
        except Exception as exc:  # noqa: BLE001
            rec = None
            ok.zero_()
            err_text = f"{type(exc).__name__}: {exc}"
            if world.is_cuda:
                try:
                    from universal_gemm_b200.ops.device import DeviceState

                    DeviceState.get(world.device).clear_status()
                except Exception:  # noqa: BLE001
                    pass
            traceback.print_exc()
        if dist.is_initialized():
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if rank == 0:
            if ok.item() > 0 and rec is not None:
                from dataclasses import asdict

                row = merged_row(shape, mc, asdict(rec))
                results.append(row)
                print(f"[{idx + 1}/{len(cases)}] {row['case_key']}: {row['median_tflops']:.1f} TFLOP/s "
                      f"({row['median_seconds'] * 1e3:.3f} ms)" +
                      (f" err={row['max_abs_error']:.2e}" if row.get("max_abs_error") is not None else ""), flush=True)
            else:
                failures.append({"index": idx, "shape_case": shape.__dict__, "method_case": mc.__dict__,
                                 "error": err_text if rec is None and ok.item() == 0 and "err_text" in dir() else "failed on another rank"})
                print(f"[{idx + 1}/{len(cases)}] FAILED {shape.experiment_group} {mc}", flush=True)
    if rank == 0:
        out = pathlib.Path(args.output_dir)
        out.mkdir(parents=True, exist_ok=True)
        payload = {"created_at": dt.datetime.now().isoformat(), "host": socket.gethostname(), "nproc_per_node": size,
                   "warmup_iters": args.warmup_iters, "measure_iters": args.measure_iters,
                   "theoretical_tflops": args.theoretical_tflops, "results": results, "failures": failures}
        (out / "results.json").write_text(json.dumps(payload, indent=2), encoding="utf-8")
        with open(out / "results.csv", "w", encoding="utf-8", newline="") as f:
            if results:
                cols = sorted({k for r in results for k in r})
                w = csv.DictWriter(f, fieldnames=cols)
                w.writeheader()
                w.writerows(results)
            else:
                csv.writer(f).writerow(["no_results"])
        print(f"Wrote {len(results)} results and {len(failures)} failures to {out}", flush=True)
    world.close()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
