#!/usr/bin/env python3
"""Run ONE rank of a multi-rank Stationary-B / Stationary-C plan on a single GPU.

All ranks' shards live on this GPU (an emulated cluster), so the kernel that is launched is exactly
the fused kernel a real rank runs - fetch warps pulling "remote" operand slices through peer pointers
into staging, tcgen05 tiles, and the epilogue storing / adding into other ranks' C - only that the
peers' memory is local.  Meant for profiler captures of the fused paths and for quick timing.

    python benchmark/fused_emulated_microbench.py --method stationary_b --a-partition row \
        --b-partition column --c-partition row --world 8 --rank 3 --dim-m 8192 --dim-n 8192 --dim-k 8192
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402
from universal_gemm_b200.ops.device import DeviceState  # noqa: E402
from universal_gemm_b200.parallel import exec as X, plan as P  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--rank", type=int, default=3)
    ap.add_argument("--method", choices=["stationary_c", "stationary_b", "auto"], default="stationary_b")
    ap.add_argument("--dim-m", type=int, default=8192)
    ap.add_argument("--dim-n", type=int, default=8192)
    ap.add_argument("--dim-k", type=int, default=8192)
    ap.add_argument("--a-partition", default="row")
    ap.add_argument("--b-partition", default="row")
    ap.add_argument("--c-partition", default="row")
    ap.add_argument("--replication", type=int, default=1)
    ap.add_argument("--c-dtype", choices=["fp32", "bf16"], default="fp32")
    ap.add_argument("--beta", type=int, default=0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--trace-dir", default="", help="after timing, run one traced launch and write its timeline here")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    m, n, k = args.dim_m, args.dim_n, args.dim_k
    cluster = ug.EmulatedCluster(args.world, dev)
    mats = []
    g = torch.Generator(device=dev).manual_seed(1)
    for w in cluster.worlds():
        a = ug.empty(w, (m, k), args.a_partition, torch.bfloat16, args.replication)
        b = ug.empty(w, (k, n), args.b_partition, torch.bfloat16, args.replication)
        c = ug.zeros(w, (m, n), args.c_partition, torch.float32 if args.c_dtype == "fp32" else torch.bfloat16,
                     args.replication)
        a.local_padded.zero_()
        b.local_padded.zero_()
        a.local.copy_(torch.randn(a.local.shape, generator=g, device=dev) * 0.02)
        b.local.copy_(torch.randn(b.local.shape, generator=g, device=dev) * 0.02)
        mats.append((a, b, c))
    a, b, c = mats[args.rank]
    kind = "b" if P.select_method(args.method, b.layout, c.layout) == "stationary_b" else "c"
    build = P.build_stationary_b_ops if kind == "b" else P.build_stationary_c_ops
    ops = build(a.layout, b.layout, c.layout, rank=args.rank)

    def run():
        X._run_fused(kind, a, b, c, ops, beta=args.beta)

    for _ in range(args.warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    DeviceState.get(dev).check()
    ms = e0.elapsed_time(e1) / args.iters
    prog, _ = X._program(kind, a, b, c, ops, True, args.beta)
    flops = 2.0 * m * n * k / args.world
    timeline = None
    if args.trace_dir:
        from universal_gemm_b200.utils import trace as TR

        prog.enable_trace()
        run()
        arr = prog.read_trace()
        timeline = TR.summarize(arr, pair=bool(prog.params.cta_pair))
        os.makedirs(args.trace_dir, exist_ok=True)
        tag = f"{kind}_w{args.world}_r{args.rank}_{m}x{n}x{k}_{prog.stats['tile_m']}"
        with open(os.path.join(args.trace_dir, f"timeline_{tag}.json"), "w", encoding="utf-8") as f:
            json.dump({"summary": timeline, "stats": prog.stats,
                       "traceEvents": TR.to_chrome_trace(arr, pid=args.rank, label=tag)}, f)
        prog.disable_trace()
    print(json.dumps({"world": args.world, "rank": args.rank, "method": "stationary_" + kind, "m": m, "n": n, "k": k,
                      "ms_per_call": ms, "rank_tflops": flops / ms / 1e9, "program": prog.stats, "timeline": timeline}))


if __name__ == "__main__":
    main()
