#!/usr/bin/env python3
"""Peer-to-peer micro-benchmark over NVLink: one-sided pull (``ug_pull_2d``), one-sided
accumulate (``ug_accumulate_2d``) and the fetch path of the fused kernel in isolation.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmark/p2p_microbench.py --mib 256

Every rank r reads from / adds into rank (r + 1) % size at the same time, so each link carries
traffic in both directions.  Device-timed with CUDA events, max over ranks; prints one JSON line.
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
from universal_gemm_b200.utils.benchmarking import max_over_ranks, sync_all  # noqa: E402


def timed(world, fn, iters, warmup=2):
    for _ in range(warmup):
        fn()
    sync_all(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    sync_all(world)
    return max_over_ranks(e0.elapsed_time(e1) / iters, world.device)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=256, help="payload per transfer")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--cols", type=int, default=8192, help="row length in bf16 elements")
    args = ap.parse_args()
    world = ug.init()
    dev, rank, size = world.device, world.rank, world.size
    st = DeviceState.get(dev)
    cols = args.cols
    rows = args.mib * 2 ** 20 // (cols * 2)
    nbytes = rows * cols * 2
    peer = (rank + 1) % size
    out = {"world": size, "payload_mib": nbytes / 2 ** 20}

    src = ug.empty(world, (rows * size, cols), "row", torch.bfloat16)       # one [rows, cols] tile per rank
    src.local.normal_()
    dst = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
    sync_all(world)
    ms = timed(world, lambda: st.pull_2d(dst.data_ptr(), cols * 2, src.tile_ptr(peer), src.ld * 2, rows, cols * 2, 2),
               args.iters)
    out["pull_kernel_gbs"] = nbytes / ms / 1e6
    ms = timed(world, lambda: st.pull_2d(dst.data_ptr(), cols * 2, src.tile_ptr(rank), src.ld * 2, rows, cols * 2, 2),
               args.iters)
    out["local_copy_kernel_gbs"] = nbytes / ms / 1e6

    acc = ug.zeros(world, (rows * size // 2, cols), "row", torch.float32)   # fp32: same bytes as above
    part = torch.ones(rows // 2, cols, dtype=torch.float32, device=dev)
    sync_all(world)
    ms = timed(world, lambda: st.accumulate_2d(acc.tile_ptr(peer), acc.ld, part.data_ptr(), cols, rows // 2, cols, 0),
               args.iters)
    out["accumulate_kernel_gbs"] = nbytes / ms / 1e6

    # Fetch path of the fused kernel: a GEMM with 128 rows whose B operand is the peer's tile, so the
    # run time is the time the fetch warps need to stage B.
    k = rows
    a = ug.empty(world, (128 * size, k), "row", torch.bfloat16)
    a.local.normal_()
    c = ug.zeros(world, (128 * size, cols * size), "block" if False else "row", torch.float32)
    bmat = ug.empty(world, (k, cols * size), "column", torch.bfloat16)
    bmat.local.normal_()
    sync_all(world)
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.fused import FusedProgramBuilder, OperandSlice, TaskSpec

    # Second case: the A operand remote with rows of 24 KiB (the shape of the staged activations of a
    # row / column / row GEMM with K = 12288): every copy piece is a single long row.
    wide_k = 12288
    wide_rows = max(256, (nbytes // (wide_k * 2)) // 256 * 256)
    a2 = ug.empty(world, (wide_rows * size, wide_k), "row", torch.bfloat16)
    a2.local.normal_()
    b2 = ug.empty(world, (wide_k, 256 * size), "column", torch.bfloat16)
    b2.local.normal_()
    c2 = ug.zeros(world, (wide_rows * size, 256), "row", torch.float32)
    sync_all(world)
    # Both for every tile variant: the copy loop is compiled into each kernel instantiation separately.
    for variant in (128, 256, "pair", "pair512"):
        builder = FusedProgramBuilder(dev, num_sms=st.num_sms, tile_m=variant)
        builder.add_task(TaskSpec(c_ptr=c.tile_ptr(rank), ldc=c.ld, m=128, n=cols, c_mode=native.C_STORE, c_dtype=0,
                                  segments=[(OperandSlice(a.tile_ptr(rank), a.ld, 0, 0, 128, k),
                                             OperandSlice(bmat.tile_ptr(peer), bmat.ld, 0, 0, k, cols, remote=True))]))
        prog = builder.build(st.status_ptr)

        def fused(prog=prog):
            prog.reset_flags(st.stream())
            prog.launch(st.stream())

        ms = timed(world, fused, args.iters)
        st.check()
        out[f"fused_fetch_gbs_{variant}"] = round(k * cols * 2 / ms / 1e6, 1)

        builder = FusedProgramBuilder(dev, num_sms=st.num_sms, tile_m=variant)
        builder.add_task(TaskSpec(c_ptr=c2.tile_ptr(rank), ldc=c2.ld, m=wide_rows, n=256, c_mode=native.C_STORE, c_dtype=0,
                                  segments=[(OperandSlice(a2.tile_ptr(peer), a2.ld, 0, 0, wide_rows, wide_k, remote=True),
                                             OperandSlice(b2.tile_ptr(rank), b2.ld, 0, 0, wide_k, 256))]))
        prog2 = builder.build(st.status_ptr)

        def fused_wide(prog2=prog2):
            prog2.reset_flags(st.stream())
            prog2.launch(st.stream())

        ms = timed(world, fused_wide, args.iters)
        st.check()
        out[f"fused_fetch_wide_rows_gbs_{variant}"] = round(wide_rows * wide_k * 2 / ms / 1e6, 1)
    # redistribute (block -> column partition, and row -> column with a bf16 -> fp32 change) into an existing matrix:
    # one-sided pulls of the overlapping pieces plus two device barriers per call
    if size > 1:
        side = 8192
        src_m = ug.empty(world, (side, side), "block", torch.bfloat16)
        src_m.local.normal_()
        dst_m = ug.empty(world, (side, side), "column", torch.bfloat16)
        sync_all(world)
        ms = timed(world, lambda: ug.redistribute(src_m, "column", out=dst_m), args.iters)
        moved = side * side * 2 / size                      # bytes every rank receives
        out["redistribute_block_to_column_gbs_per_gpu"] = round(moved / ms / 1e6, 1)
        out["redistribute_block_to_column_ms"] = round(ms, 4)
        row_m = ug.empty(world, (side, side), "row", torch.bfloat16)
        row_m.local.normal_()
        dst32 = ug.empty(world, (side, side), "column", torch.float32)
        sync_all(world)
        ms = timed(world, lambda: ug.redistribute(row_m, "column", dtype=torch.float32, out=dst32), args.iters)
        out["redistribute_row_to_column_bf16_to_fp32_ms"] = round(ms, 4)
        st.check()
    if rank == 0:
        print(json.dumps(out), flush=True)
    world.close()
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
