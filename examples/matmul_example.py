#!/usr/bin/env python3
"""Distributed matrix multiplication example with a correctness check.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/matmul_example.py \
        --a-partition row --b-partition column --c-partition row --stationary-method auto

Every rank builds the same random A, B from a seed, shards them into symmetric memory, runs
``C += A @ B`` ten times through the ``torch.addmm(c, a, b, out=c)`` hook (or directly with
``--no-hook``), prints the profiler breakdown and the max / median GFLOP/s against a single-GPU
``torch.addmm`` of the full matrices, and checks the gathered result.  Command line of the
reference's dtensor_example.py:184-268 (sizes, partitions, replication flags, method).
"""
from __future__ import annotations

import argparse
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Distributed matrix multiplication example")
    p.add_argument("--rows-m", "--m", dest="m", type=int, default=8 * 1024, help="Number of rows in matrix A")
    p.add_argument("--cols-n", "--n", dest="n", type=int, default=8 * 1024, help="Number of columns in matrix B")
    p.add_argument("--inner-k", "--k", dest="k", type=int, default=8 * 1024, help="Columns of A / rows of B")
    for name in "abc":
        p.add_argument(f"--{name}-partition", choices=["row", "column", "col", "block"], default="row")
        p.add_argument(f"--{name}-replication", type=int, default=None)
    p.add_argument("--replication", type=int, default=None,
                   help="Replication factor for A, B and C (exclusive with the per-matrix flags)")
    p.add_argument("--stationary-method", choices=["auto", "stationary_c", "stationary_b"], default="auto")
    p.add_argument("--dtype", choices=["bf16", "fp32"], default=None)
    p.add_argument("--iterations", type=int, default=10)
    p.add_argument("--no-hook", action="store_true", help="call ug.matmul instead of torch.addmm on DTensors")
    args = p.parse_args()
    per_matrix = [args.a_replication, args.b_replication, args.c_replication]
    if args.replication is not None and any(v is not None for v in per_matrix):
        p.error("Cannot pass --replication together with --a-replication/--b-replication/--c-replication.")
    if any(v is not None and v <= 0 for v in per_matrix + [args.replication]):
        p.error("replication factors must be >= 1.")
    base = args.replication or 1
    args.reps = [base if v is None else v for v in per_matrix]
    return args


def main() -> None:
    args = parse_args()
    world = ug.init()
    dev, rank = world.device, world.rank
    on_gpu = world.is_cuda
    in_dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, None: torch.bfloat16 if on_gpu else torch.float32}[args.dtype]
    m, n, k = args.m, args.n, args.k
    print(f"Rank {rank}/{world.size} running on {dev}")
    torch.manual_seed(0)
    full_a = torch.randn(m, k, device=dev)
    full_b = torch.randn(k, n, device=dev) / k ** 0.5
    full_c = torch.full((m, n), 0.5, device=dev)
    a = ug.distribute_tensor(full_a, world, args.a_partition, args.reps[0], dtype=in_dtype)
    b = ug.distribute_tensor(full_b, world, args.b_partition, args.reps[1], dtype=in_dtype)
    c = ug.distribute_tensor(full_c, world, args.c_partition, args.reps[2], dtype=torch.float32)
    if rank == 0:
        print(f"Multiply A {a.shape} by B {b.shape} -> C {c.shape}")
        print(f"Tile grids are A {ug.grid_shape(a)}, B {ug.grid_shape(b)}, and C {ug.grid_shape(c)}")
    use_hook = not args.no_hook and world.size > 0 and torch.distributed.is_initialized()
    if use_hook:
        ug.mm_handler.enable(args.stationary_method)
        da, db, dc = a.to_dtensor(), b.to_dtensor(), c.to_dtensor()
    ug.profile.reset_stats()
    ug.profile.enable(on_gpu)

    def run_once():
        if use_hook:
            torch.addmm(dc, da, db, out=dc)
        else:
            ug.matmul(a, b, c, method=args.stationary_method)

    def timed(fn):
        if on_gpu:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            world.barrier()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            world.barrier()
            return e0.elapsed_time(e1) * 1e-3
        import time

        world.barrier()
        t0 = time.perf_counter()
        fn()
        world.barrier()
        return time.perf_counter() - t0

    durations = [timed(run_once) for _ in range(args.iterations)]
    if on_gpu:
        ug.check_status(dev)
    if rank == 0:
        ug.profile.print_stats(runtime_total_s=sum(durations))

    ref_c = full_c.clone()
    ra, rb = full_a.to(in_dtype), full_b.to(in_dtype)
    ref_durations = []
    for _ in range(args.iterations):
        ref_durations.append(timed(lambda: ref_c.addmm_(ra.float() if not on_gpu else ra.to(torch.float32), rb.float())
                                   if in_dtype == torch.float32 else ref_c.add_(torch.matmul(ra, rb).float())))
    got = c.full_tensor(replica=0)
    if on_gpu:
        torch.cuda.synchronize()
    if rank == 0:
        tol = 1e-4 if in_dtype == torch.float32 else 2e-2
        torch.testing.assert_close(got.cpu(), ref_c.cpu(), rtol=tol, atol=tol * 10)
        gflop = 1e-9 * (2 * m * n * k + 3 * m * n)
        ours = [gflop / d for d in durations]
        ref = [gflop / d for d in ref_durations]
        print(f"Max Distributed GFLOPs: {max(ours)}")
        print(f"Median Distributed GFLOPs: {statistics.median(ours)}")
        print(f"Max Reference (Single GPU) GFLOPs: {max(ref)}")
        print(f"Median Reference (Single GPU) GFLOPs: {statistics.median(ref)}")
        print(f"Median speedup is {statistics.median(ours) / statistics.median(ref)} over a single GPU.")
        print("result check passed")
    if use_hook:
        ug.mm_handler.disable()
    world.close()
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
