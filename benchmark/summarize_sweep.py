#!/usr/bin/env python3
"""Turn the ``results.json`` files of ``run_matmul_sweep.py`` (one per GPU count and C dtype) into the markdown
tables this repository reports: per shape / partition triple / replication factor the whole-box TFLOP/s of the
plain-DTensor baseline (bf16 operands) and of this framework's methods, their ratio, and the achieved fraction of
the roofline (the slower of the case's FLOPs at the measured bf16 GEMM peak and its remote bytes at the measured
NVLink rate; the fields come from the worker).

    python benchmark/summarize_sweep.py out/n8_fp32/results.json out/n8_bf16/results.json --output table.md

The same result files feed ``render_benchmark_report.py`` (plots); this script only writes text.
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import defaultdict


def load(paths: list[str]) -> list[dict]:
    rows = []
    for path in paths:
        with open(path, encoding="utf-8") as f:
            payload = json.load(f)
        for row in payload.get("results", []):
            row = dict(row)
            row["_file"] = path
            rows.append(row)
    return rows


def fmt(x: float | None, digits: int = 0) -> str:
    if x is None:
        return "-"
    return f"{x:.{digits}f}"


def summarize(rows: list[dict]) -> str:
    by_world: dict[int, list[dict]] = defaultdict(list)
    for r in rows:
        by_world[int(r["world_size"])].append(r)
    out: list[str] = []
    for world in sorted(by_world):
        cases: dict[tuple, dict] = {}
        for r in by_world[world]:
            key = (r["experiment_group"], r["m"], r["n"], r["k"], r["a_partition"], r["b_partition"], r["c_partition"],
                   r["replication_factor"])
            slot = cases.setdefault(key, {})
            name = r["method"] if r["method"] == "dtensor" else f"{r['method']}/{r.get('c_dtype', 'fp32')}"
            best = slot.get(name)
            if best is None or r["median_tflops"] > best["median_tflops"]:
                slot[name] = r
        out.append(f"### {world} GPU{'s' if world > 1 else ''}\n")
        big = [k for k in cases if k[0] in ("square", "gpt3_expansion", "gpt3_shrinking")]
        if big:
            out.append("| M x N x K | A,B,C | rep | dtensor bf16 | St-C fp32 C | St-B fp32 C | St-C bf16 C | St-B bf16 C | "
                       "best fp32 C / dtensor | best / dtensor | roofline fraction (best fp32 C) | max abs err (fp32 C) |")
            out.append("|---|---|---|---|---|---|---|---|---|---|---|---|")
            for key in big:
                slot = cases[key]
                g = lambda name: slot.get(name, {}).get("median_tflops")  # noqa: E731
                ours32 = [slot[n_] for n_ in ("stationary_c/fp32", "stationary_b/fp32") if n_ in slot]
                ours = ours32 + [slot[n_] for n_ in ("stationary_c/bf16", "stationary_b/bf16") if n_ in slot]
                dt = g("dtensor")
                b32 = max(ours32, key=lambda r: r["median_tflops"]) if ours32 else None
                ball = max(ours, key=lambda r: r["median_tflops"]) if ours else None
                errs = [r.get("max_abs_error") for r in ours32 if r.get("max_abs_error") is not None]
                out.append("| {} x {} x {} | {},{},{} | {} | {} | {} | {} | {} | {} | {} | {} | {} | {} |".format(
                    key[1], key[2], key[3], key[4], key[5], key[6], key[7], fmt(dt), fmt(g("stationary_c/fp32")),
                    fmt(g("stationary_b/fp32")), fmt(g("stationary_c/bf16")), fmt(g("stationary_b/bf16")),
                    fmt(b32["median_tflops"] / dt, 2) if b32 and dt else "-",
                    fmt(ball["median_tflops"] / dt, 2) if ball and dt else "-",
                    fmt(b32.get("roofline_fraction"), 2) if b32 else "-",
                    f"{max(errs):.1e}" if errs else "-"))
            out.append("")
        odd = [k for k in cases if k not in big]
        if odd:
            out.append("| M x N x K | A,B,C | dtensor bf16 | auto (fp32 C) | method / tile | auto / dtensor | max abs err |")
            out.append("|---|---|---|---|---|---|---|")
            wins = total = 0
            for key in odd:
                slot = cases[key]
                auto = slot.get("auto/fp32")
                dt = slot.get("dtensor", {}).get("median_tflops")
                if auto is None:
                    continue
                if dt:
                    total += 1
                    wins += auto["median_tflops"] >= dt
                err = auto.get("max_abs_error")
                out.append("| {} x {} x {} | {},{},{} | {} | {} | {} / {} | {} | {} |".format(
                    key[1], key[2], key[3], key[4], key[5], key[6], fmt(dt), fmt(auto["median_tflops"]),
                    auto.get("executed_method", ""), auto.get("tile_variant", ""),
                    fmt(auto["median_tflops"] / dt, 2) if dt else "-", f"{err:.1e}" if err is not None else "-"))
            out.append("")
            if total:
                out.append(f"auto >= dtensor bf16 on {wins} of {total} odd / skinny cases.\n")
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("results", nargs="+", help="results.json files of run_matmul_sweep.py / run_matmul_experiments.py")
    ap.add_argument("--output", default="", help="write the markdown here (default: standard output)")
    args = ap.parse_args(argv)
    text = summarize(load(args.results))
    if args.output:
        with open(args.output, "w", encoding="utf-8") as f:
            f.write(text + "\n")
    else:
        sys.stdout.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
