#!/usr/bin/env python3
"""Single-GPU micro-benchmark of the fused tcgen05 GEMM kernel against ``torch.matmul``.

    python benchmark/kernel_microbench.py --m 8192 --n 8192 --k 8192 --iters 20
    python benchmark/kernel_microbench.py --m 4096 --n 4096 --k 4096 --stage-b   # B through the fetch warps

Times with CUDA events after warm-up; prints one JSON line.  ``--iters 1 --no-torch`` gives a
short run suited to a profiler capture of one launch.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from universal_gemm_b200.ops import native  # noqa: E402
from universal_gemm_b200.ops.device import DeviceState  # noqa: E402
from universal_gemm_b200.ops.gemm import build_gemm_program, run_program  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--segments", type=int, default=1, help="split K into this many segments")
    ap.add_argument("--stage-a", action="store_true")
    ap.add_argument("--stage-b", action="store_true")
    ap.add_argument("--mode", choices=["store", "add", "atomic"], default="store")
    ap.add_argument("--c-dtype", choices=["fp32", "bf16"], default="fp32")
    ap.add_argument("--no-torch", action="store_true")
    ap.add_argument("--trace", action="store_true", help="add the in-kernel timeline summary of one more launch")
    ap.add_argument("--tile-m", type=lambda v: v if v.startswith("pair") else int(v), default=None, help="rows per output tile (default: model)")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    m, n, k = args.m, args.n, args.k
    a = torch.randn(m, k, device=dev).bfloat16()
    b = (torch.randn(k, n, device=dev) / k ** 0.5).bfloat16()
    c = torch.zeros(m, n, device=dev, dtype=torch.float32 if args.c_dtype == "fp32" else torch.bfloat16)
    cuts = [k * i // args.segments // 64 * 64 for i in range(args.segments)] + [k]
    mode = {"store": native.C_STORE, "add": native.C_ADD, "atomic": native.C_ATOMIC}[args.mode]
    prog = build_gemm_program([a[:, cuts[i]:cuts[i + 1]] for i in range(args.segments)],
                              [b[cuts[i]:cuts[i + 1]] for i in range(args.segments)], c, mode=mode,
                              stage_a=args.stage_a, stage_b=args.stage_b, tile_m=args.tile_m)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.iters

    ours = timed(lambda: run_program(prog, dev))
    DeviceState.get(dev).check()
    flops = 2.0 * m * n * k
    out = {"m": m, "n": n, "k": k, "ours_ms": ours, "ours_tflops": flops / ours / 1e9, "stats": prog.stats,
           "mode": args.mode, "c_dtype": args.c_dtype}
    if args.trace:
        from universal_gemm_b200.utils import trace as TR

        prog.enable_trace()
        run_program(prog, dev)
        tl = TR.summarize(prog.read_trace(), pair=bool(prog.params.cta_pair))
        out["timeline"] = {k_: (round(v, 2) if isinstance(v, float) else v) for k_, v in tl.items()}
        prog.disable_trace()
    if not args.no_torch:
        ref = timed(lambda: torch.matmul(a, b))
        out.update({"torch_ms": ref, "torch_tflops": flops / ref / 1e9})
    print(json.dumps(out))


if __name__ == "__main__":
    main()
