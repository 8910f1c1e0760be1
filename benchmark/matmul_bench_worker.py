#!/usr/bin/env python3
"""One benchmark case: (shape, method, partition triple, replication factor) on all ranks of a
``torchrun`` launch.  Rank 0 writes a JSON record with the same fields as the reference's worker
(benchmark/matmul_bench_worker.py:66-85) plus a few extra ones.

Methods: ``dtensor`` (stock torch DTensor matmul + redistribute: the library baseline),
``stationary_c``, ``stationary_b`` and ``auto`` (this framework).  Differences from the
reference's worker: the dtype is a flag (bf16 operands with fp32 accumulation by default on GPU),
iterations are timed on the device with CUDA events (host clock on CPU), C is zeroed before the
cross-rank barrier that precedes the first remote accumulate, and the result can be verified.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from dataclasses import asdict, dataclass

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402
from universal_gemm_b200.utils.benchmarking import max_over_ranks, sync_all  # noqa: E402

METHODS = ("dtensor", "stationary_c", "stationary_b", "auto", "min_traffic")
DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32}


@dataclass
class BenchResult:
    method: str
    m: int
    n: int
    k: int
    a_partition: str
    b_partition: str
    c_partition: str
    replication_factor: int
    warmup_iters: int
    measure_iters: int
    world_size: int
    median_seconds: float
    min_seconds: float
    max_seconds: float
    median_tflops: float
    max_tflops: float
    flops: float
    theoretical_tflops: float | None
    dtype: str = "bf16"
    c_dtype: str = "fp32"
    device: str = "cuda"
    timing: str = "cuda_events_max_over_ranks"
    executed_method: str = ""
    max_abs_error: float | None = None
    verified_rows: int | None = None
    # bytes rank 0 moves over NVLink per iteration (staged remote operand slices in, partial C out), the tile variant
    # its plan was lowered to, and the roofline time of the case: the slower of its FLOPs at the measured bf16 GEMM
    # peak of one GPU and its remote bytes at the measured peer-copy rate per direction
    remote_in_bytes: int | None = None
    remote_out_bytes: int | None = None
    tile_variant: str = ""
    roofline_seconds: float | None = None
    roofline_fraction: float | None = None


def _dtensor_iteration(dt_a, dt_b):
    out = torch.matmul(dt_a, dt_b)
    need, placements = ug.materialized_placements(out.placements)
    if need:
        out = out.redistribute(out.device_mesh, placements)
    return out.to_local()


def bench_case(world, args: argparse.Namespace) -> BenchResult | None:
    """Run one case on an existing world; returns the record on rank 0 (None elsewhere)."""
    dev = world.device
    rank, size = world.rank, world.size
    in_dtype, c_dtype = DTYPES[args.dtype], DTYPES[args.c_dtype]
    torch.manual_seed(args.seed)          # same full matrices on every rank; each keeps its shard
    m, n, k = args.m, args.n, args.k
    mats = None
    try:
        full_a = torch.randn(m, k, device=dev, dtype=torch.float32).to(in_dtype)
        full_b = (torch.randn(k, n, device=dev, dtype=torch.float32) * args.b_scale).to(in_dtype)
        executed = args.method
        if args.method == "dtensor":
            from torch.distributed.tensor import DTensor

            pa = ug.get_partitioning(args.a_partition, args.replication_factor, size)
            pb = ug.get_partitioning(args.b_partition, args.replication_factor, size)

            def shard(full, part):
                lay = part.layout(tuple(full.shape))
                mesh, placements = part.to_torch(dev.type)
                from universal_gemm_b200.parallel import tiles as T

                b = T.tile_bounds(lay, T.local_tile_coord(lay, rank))
                local = full[b.rows.as_slice(), b.cols.as_slice()].contiguous()
                return DTensor.from_local(local, mesh, placements, run_check=False, shape=full.shape,
                                          stride=(full.shape[1], 1))

            dt_a, dt_b = shard(full_a, pa), shard(full_b, pb)
            iteration = lambda: _dtensor_iteration(dt_a, dt_b)  # noqa: E731
        else:
            a = ug.distribute_tensor(full_a, world, args.a_partition, args.replication_factor)
            b = ug.distribute_tensor(full_b, world, args.b_partition, args.replication_factor)
            c = ug.zeros(world, (m, n), args.c_partition, c_dtype, args.replication_factor)
            executed = ug.select_method(args.method, b.layout, c.layout, a.layout, in_bytes=a.itemsize,
                                        c_bytes=c.itemsize)
            mats = (a, b, c)

            if world.is_cuda and getattr(args, "cuda_graph", False) and in_dtype == torch.bfloat16:
                plan = ug.prepare_matmul(a, b, c, method=executed, beta=0).capture()
                iteration = plan.run                              # barrier + fused GEMM + barrier from a CUDA graph
            else:
                def iteration():
                    ug.matmul(a, b, c, method=executed, beta=0)  # C = A @ B, like "zero C; C += A @ B"

        for _ in range(args.warmup_iters):
            iteration()
        sync_all(world)
        durations = []
        for _ in range(args.measure_iters):
            sync_all(world)
            if world.is_cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                iteration()
                e1.record()
                sync_all(world)
                local = e0.elapsed_time(e1) * 1e-3
            else:
                t0 = time.perf_counter()
                iteration()
                world.barrier()
                local = time.perf_counter() - t0
            durations.append(max_over_ranks(local, dev))
        if world.is_cuda:
            ug.check_status(dev)

        err, verified_rows = None, None
        if args.verify:
            if mats is not None:
                got = mats[2].full_tensor(replica=0)
            else:                          # plain-DTensor baseline: one more product, gathered (collective)
                got = torch.matmul(dt_a, dt_b).full_tensor()
            nrows = int(getattr(args, "verify_rows", 0) or 0)
            if 0 < nrows < m:              # sampled rows (a different sample per case): cheap enough for every case
                rows = (torch.arange(nrows, device=dev) * (m // nrows) + (args.seed * 7919) % max(m // nrows, 1)) % m
                want = full_a[rows].double() @ full_b.double()
                got = got[rows]
                verified_rows = nrows
            else:
                want = full_a.double() @ full_b.double()
                verified_rows = m
            if world.is_cuda:
                torch.cuda.synchronize()
            err = float((got.double() - want).abs().max().item())
            limit = getattr(args, "verify_tolerance", None)
            if limit is not None and got.dtype == torch.bfloat16:
                limit = max(limit, 3e-2)          # the result itself is rounded to 8 bits of mantissa
            if limit is not None and not err <= limit * max(1.0, float(want.abs().max().item())):
                raise RuntimeError(f"result differs from the fp64 product: max abs error {err:.3e}")
        stats = {}
        if mats is not None and world.is_cuda:
            from universal_gemm_b200.parallel.exec import cached_programs

            progs = cached_programs()
            if progs:
                stats = max((p.stats for _, p in progs), key=lambda st: st.get("tiles", 0))
        if rank != 0:
            return None
        flops = float(2.0 * m * n * k)
        tflops = [flops / d / 1e12 for d in durations]
        peak = float(getattr(args, "peak_tflops", 0) or 0)
        link = float(getattr(args, "link_gbs", 0) or 0)
        roof = None
        if peak > 0:
            roof = flops / size / (peak * 1e12)
            if link > 0 and stats:
                roof = max(roof, stats.get("remote_bytes", 0) / (link * 1e9), stats.get("push_bytes", 0) / (link * 1e9))
        med = statistics.median(durations)
        return BenchResult(
            verified_rows=verified_rows, remote_in_bytes=stats.get("remote_bytes"), remote_out_bytes=stats.get("push_bytes"),
            tile_variant=str(stats.get("tile_m", "")), roofline_seconds=roof,
            roofline_fraction=(roof / med) if roof else None,
            method=args.method, m=m, n=n, k=k, a_partition=args.a_partition, b_partition=args.b_partition,
            c_partition=args.c_partition, replication_factor=args.replication_factor,
            warmup_iters=args.warmup_iters, measure_iters=args.measure_iters, world_size=size,
            median_seconds=statistics.median(durations), min_seconds=min(durations), max_seconds=max(durations),
            median_tflops=statistics.median(tflops), max_tflops=max(tflops), flops=flops,
            theoretical_tflops=args.theoretical_tflops, dtype=args.dtype, c_dtype=args.c_dtype, device=dev.type,
            timing="cuda_events_max_over_ranks" if world.is_cuda else "host_clock_max_over_ranks",
            executed_method=executed, max_abs_error=err)
    finally:
        if mats is not None:
            world.barrier()
            for mat in mats:
                mat.free()
            from universal_gemm_b200.parallel.exec import clear_program_cache

            clear_program_cache()


def run_worker(args: argparse.Namespace) -> None:
    world = ug.init(device=args.device)
    try:
        result = bench_case(world, args)
        if result is not None:
            os.makedirs(os.path.dirname(os.path.abspath(args.result_file)), exist_ok=True)
            with open(args.result_file, "w", encoding="utf-8") as f:
                json.dump(asdict(result), f, indent=2, sort_keys=True)
    finally:
        try:
            world.close()
        except Exception:  # noqa: BLE001
            pass
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Single-case distributed GEMM benchmark")
    p.add_argument("--method", choices=METHODS, required=True)
    # --dim-* are aliases that survive torchrun's own option parser (it rejects "--m" as an
    # ambiguous abbreviation of its --master-* / --max-* options).
    p.add_argument("--m", "--dim-m", dest="m", type=int, required=True)
    p.add_argument("--n", "--dim-n", dest="n", type=int, required=True)
    p.add_argument("--k", "--dim-k", dest="k", type=int, required=True)
    for name in ("a", "b", "c"):
        p.add_argument(f"--{name}-partition", choices=["row", "column", "col", "block"], required=True)
    p.add_argument("--replication-factor", type=int, required=True)
    p.add_argument("--warmup-iters", type=int, default=3)
    p.add_argument("--measure-iters", type=int, default=10)
    p.add_argument("--seed", type=int, default=20260218)
    p.add_argument("--result-file", type=str, required=True)
    p.add_argument("--theoretical-tflops", type=float, default=None)
    p.add_argument("--dtype", choices=list(DTYPES), default=None, help="operand dtype (default bf16 on GPU, fp32 on CPU)")
    p.add_argument("--c-dtype", choices=list(DTYPES), default="fp32")
    p.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--b-scale", type=float, default=1.0)
    p.add_argument("--verify", action="store_true", help="compare the result with an fp64 matmul of the full matrices")
    p.add_argument("--verify-rows", type=int, default=0, help="verify only this many sampled rows (0 = all rows)")
    p.add_argument("--verify-tolerance", type=float, default=None,
                   help="fail the case when the max abs error exceeds this times max(1, max |C|)")
    p.add_argument("--peak-tflops", type=float, default=0.0, help="bf16 GEMM peak of one GPU for the roofline fields")
    p.add_argument("--link-gbs", type=float, default=0.0, help="NVLink rate per direction per GPU for the roofline fields")
    p.add_argument("--cuda-graph", action="store_true", help="replay each stationary GEMM from a captured CUDA graph")
    args = p.parse_args(argv)
    for name in ("a_partition", "b_partition", "c_partition"):
        setattr(args, name, ug.parallel.partition.normalize_partition(getattr(args, name)))
    if args.dtype is None:
        args.dtype = "bf16" if args.device == "cuda" else "fp32"
    return args


def main(argv=None) -> None:
    run_worker(parse_args(argv))


if __name__ == "__main__":
    main()
