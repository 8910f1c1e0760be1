#!/usr/bin/env python3
"""Bandwidth of the stand-alone tile kernels on one GPU: zero, copy (pull), accumulate (red.add) and
dtype conversion, on a 2-D slice larger than L2.  Prints one JSON line with GB/s of bytes read + written.

    python benchmark/tile_ops_microbench.py --rows 16384 --cols 16384
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    st = DeviceState.get(dev)
    rows, cols = args.rows, args.cols
    ld = cols + 64                                   # strided slices, as tiles in symmetric memory are
    f32_a = torch.randn(rows, ld, device=dev)
    f32_b = torch.zeros(rows, ld, device=dev)
    bf_a = torch.randn(rows, ld, device=dev).bfloat16()
    bf_b = torch.zeros(rows, ld, device=dev, dtype=torch.bfloat16)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.iters * 1e-3

    n = rows * cols
    out = {"rows": rows, "cols": cols}
    t = timed(lambda: st.zero_2d(f32_b.data_ptr(), ld * 4, rows, cols * 4))
    out["zero_f32_gbs"] = n * 4 / t / 1e9
    t = timed(lambda: st.pull_2d(f32_b.data_ptr(), ld * 4, f32_a.data_ptr(), ld * 4, rows, cols * 4, 4))
    out["copy_f32_gbs"] = 2 * n * 4 / t / 1e9
    t = timed(lambda: st.pull_2d(bf_b.data_ptr(), ld * 2, bf_a.data_ptr(), ld * 2, rows, cols * 2, 2))
    out["copy_bf16_gbs"] = 2 * n * 2 / t / 1e9
    t = timed(lambda: st.accumulate_2d(f32_b.data_ptr(), ld, f32_a.data_ptr(), ld, rows, cols, native.DT_F32))
    out["accumulate_f32_gbs"] = 3 * n * 4 / t / 1e9       # read src, read-modify-write dst
    t = timed(lambda: st.accumulate_2d(bf_b.data_ptr(), ld, bf_a.data_ptr(), ld, rows, cols, native.DT_BF16))
    out["accumulate_bf16_gbs"] = 3 * n * 2 / t / 1e9
    t = timed(lambda: st.convert_2d(bf_b.data_ptr(), ld, native.DT_BF16, f32_a.data_ptr(), ld, native.DT_F32, rows, cols))
    out["convert_f32_to_bf16_gbs"] = n * 6 / t / 1e9
    t = timed(lambda: f32_b.copy_(f32_a))
    out["torch_copy_f32_gbs"] = 2 * rows * ld * 4 / t / 1e9
    st.check()
    print(json.dumps({k: (round(v, 1) if isinstance(v, float) else v) for k, v in out.items()}))


if __name__ == "__main__":
    main()
