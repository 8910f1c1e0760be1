#!/usr/bin/env python3
"""Headline benchmark: whole-box TFLOP/s of one distributed GEMM ``C = A @ B``.

Default configuration: the GPT-3-175B MLP up-projection, A = [8192, 12288] activations,
B = [12288, 49152] weights, bf16 inputs with fp32 accumulation and fp32 C, partition triple
row / column / row, replication 1, method ``auto``; random-init synthetic data.  The total
problem is fixed, so the scaling over 1 / 2 / 4 / 8 GPUs is strong scaling.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

One step = one distributed GEMM C = A @ B (entry barrier, fused tcgen05 kernel with in-kernel tile
fetch / remote store or accumulate, exit barrier).  After the warm-up the bench times ``--rounds``
rounds (at least 5) of exactly ``--steps`` steps each, every round bracketed by a barrier and a device
synchronisation on both sides and timed with CUDA events; the time of a round is the maximum over
ranks, ``value`` is 2*M*N*K over the median round's time per step and ``rounds_ms`` lists all of them.

``e2e`` repeats the measurement through the same public call but with, every step, the
host-to-device copy of that step's activations from pinned memory and a device-to-host read of a
checksum of the result.  After the timed regions the product is checked: sampled rows of C against
an fp32 product of the same bf16 operands, and every end-to-end checksum against the checksum of
the verified C (``verified``, ``max_abs_err``).  On more than one GPU a per-rank breakdown
(barriers / fused kernel) and a summary of the in-kernel timeline of one extra step are added, and
``context.dtensor_bf16_tflops`` gives stock DTensor + NCCL + cuBLAS on the same bf16 operands in the
same launch.

``--impl reference`` runs the unmodified reference benchmark worker instead (see baseline/).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# Both arms print this string, so that their values can be divided.
METRIC = "whole-box TFLOP/s (2*M*N*K / time per step, max over ranks)"


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rounds", type=int, default=5, help="timed rounds of --steps steps each (at least 5); the "
                    "median round is reported")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    # --dim-* spellings pass through torchrun's own parser ("--m" is an ambiguous prefix there)
    ap.add_argument("--m", "--dim-m", dest="m", type=int, default=8192)
    ap.add_argument("--n", "--dim-n", dest="n", type=int, default=49152)
    ap.add_argument("--k", "--dim-k", dest="k", type=int, default=12288)
    ap.add_argument("--a-partition", default="row")
    ap.add_argument("--b-partition", default="column")
    ap.add_argument("--c-partition", default="row")
    ap.add_argument("--replication", type=int, default=1)
    ap.add_argument("--method", default="auto", choices=["auto", "stationary_c", "stationary_b"])
    ap.add_argument("--c-dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--operand-dtype", default="bf16", choices=["bf16", "fp32"],
                    help="fp32: A and B are fp32 like the reference worker's; the kernel runs them as three bf16 products")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-context", action="store_true", help="skip the stock-DTensor bf16 comparator")
    ap.add_argument("--profile", action="store_true", help="add the per-rank breakdown on one GPU too")
    ap.add_argument("--trace-dir", default="", help="write the in-kernel timeline of one extra step there "
                    "(trace_rank<r>_*.json)")
    ap.add_argument("--master-port", type=int, default=29517)
    return ap.parse_args(argv)


def _relaunch_under_torchrun(args) -> int:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(args.master_port), os.path.abspath(__file__)] + sys.argv[1:]
    return subprocess.call(cmd)


def _gather_floats(values, world, dev):
    """``values`` (list of floats) of every rank, as a list of lists on every rank."""
    import torch
    import torch.distributed as dist

    mine = torch.tensor(values, dtype=torch.float64, device=dev)
    if world.size == 1:
        return [mine.tolist()]
    allv = [torch.zeros_like(mine) for _ in range(world.size)]
    dist.all_gather(allv, mine)
    return [v.tolist() for v in allv]


def _verify(ug, world, a, b, c, c_dtype, rows_per_rank: int = 64):
    """Compare ``rows_per_rank`` sampled rows of the distributed C (a different sample on every rank) with an fp32
    product of the same bf16 operands.  Returns (ok, max_abs_err, tolerance, sum and sum of squares of this rank's C shard)."""
    import torch

    dev = world.device
    full_a, full_b, full_c = a.full_tensor(), b.full_tensor(), c.full_tensor()
    torch.cuda.synchronize(dev)
    m = full_a.shape[0]
    step = max(m // rows_per_rank, 1)
    rows = (torch.arange(rows_per_rank, device=dev) * step + (world.rank * 7919) % step) % m
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        want = (full_a[rows].double() @ full_b.double()).float() if full_a.dtype == torch.float32 \
            else full_a[rows].float() @ full_b.float()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    got = full_c[rows].float()
    err = float((got - want).abs().max().item())
    scale = float(want.abs().max().item())
    tol = (2e-2 if c_dtype == torch.bfloat16 else 2e-3) * max(scale, 1e-6)
    checksum = float(c.local.sum(dtype=torch.float64).item())
    sumsq = float(c.local.float().square().sum(dtype=torch.float64).item())
    del full_a, full_b, full_c, want, got
    return err <= tol, err, tol, checksum, sumsq


def run_ours(args) -> dict:
    import torch

    import universal_gemm_b200 as ug
    from universal_gemm_b200.ops.device import DeviceState
    from universal_gemm_b200.utils.benchmarking import ClockSampler, max_over_ranks, sync_all

    world = ug.init()
    if not world.is_cuda:
        raise RuntimeError("bench.py needs a CUDA device")
    if world.size != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but the launcher started {world.size} rank(s)")
    dev = world.device
    state = DeviceState.get(dev)
    m, n, k = args.m, args.n, args.k
    c_dtype = torch.float32 if args.c_dtype == "fp32" else torch.bfloat16
    warmup = max(args.warmup, 3)
    rounds = max(args.rounds, 5)

    in_dtype = torch.bfloat16 if args.operand_dtype == "bf16" else torch.float32
    a = ug.empty(world, (m, k), args.a_partition, in_dtype, args.replication)
    b = ug.empty(world, (k, n), args.b_partition, in_dtype, args.replication)
    c = ug.zeros(world, (m, n), args.c_partition, c_dtype, args.replication)
    # Every rank draws the same full matrices from one seed and keeps its shards (replicas hold equal copies).
    g = torch.Generator(device=dev).manual_seed(20260218)
    a.local_padded.zero_()
    b.local_padded.zero_()
    a.fill_from_full((torch.randn(m, k, generator=g, device=dev) * 0.02).to(in_dtype))
    b.fill_from_full((torch.randn(k, n, generator=g, device=dev) * 0.02).to(in_dtype))
    method = ug.select_method(args.method, b.layout, c.layout)

    def step():
        # C = A @ B (beta = 0): same result as the reference's "zero C, then C += A @ B" iteration; C is only
        # zeroed by the executor when several ranks have to add into the same elements.
        ug.matmul(a, b, c, method=method, beta=0)

    for _ in range(warmup):
        step()
    sync_all(world)
    ug.check_status(dev)

    sampler = ClockSampler(dev.index or 0) if world.rank == 0 else None
    if sampler:
        sampler.start()
    rounds_ms, launches = [], 0
    for _ in range(rounds):
        launches0 = state.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all(world)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        sync_all(world)
        rounds_ms.append(max_over_ranks(e0.elapsed_time(e1) / args.steps, dev))
        launches = state.launches - launches0
    ms_per_step = statistics.median(rounds_ms)
    ug.check_status(dev)

    # End to end through the public API: every step copies that step's activations from pinned host memory
    # into the (double-buffered) symmetric A shard and reads a checksum of that step's C back to the host.
    # The copy for step i+1 runs on a copy stream while step i computes, and the host waits for the checksum
    # of step i-1 while step i runs; all K copies and K read-backs happen inside the timed region.
    e2e, checks = None, []
    if not args.no_e2e:
        a_alt = ug.empty(world, (m, k), args.a_partition, in_dtype, args.replication)
        a_alt.local_padded.zero_()
        bufs = (a, a_alt)
        host_a = torch.empty(a.local.shape, dtype=in_dtype).pin_memory()
        host_a.copy_(a.local)
        # The kernel's epilogue adds this rank's share of sum(C) of every step to one running double (never reset);
        # the host reads the running value back every step and takes differences.
        running = torch.zeros(1, dtype=torch.float64, device=dev)
        host_out = [torch.zeros(1, dtype=torch.float64).pin_memory() for _ in range(2)]
        copy_stream = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        copied = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        read_back = [torch.cuda.Event() for _ in range(2)]

        def issue_copy(i):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[i % 2])          # the GEMM that last read this buffer is done
                bufs[i % 2].local.copy_(host_a, non_blocking=True)
                copied[i % 2].record(copy_stream)

        def run_e2e(steps):
            for ev in consumed + read_back:
                ev.record(main)
            issue_copy(0)
            out = []
            for i in range(steps):
                main.wait_event(copied[i % 2])
                if i + 1 < steps:
                    issue_copy(i + 1)
                ug.matmul(bufs[i % 2], b, c, method=method, beta=0, checksum=running)
                consumed[i % 2].record(main)
                read_back[(i + 1) % 2].synchronize()            # host reads the checksum of step i-1
                if i > 0:
                    out.append(float(host_out[(i + 1) % 2][0]))
                host_out[i % 2].copy_(running, non_blocking=True)
                read_back[i % 2].record(main)
            read_back[(steps - 1) % 2].synchronize()
            out.append(float(host_out[(steps - 1) % 2][0]))
            shares = [out[0] - run_e2e.last] + [out[j] - out[j - 1] for j in range(1, len(out))]
            run_e2e.last = out[-1]
            return shares

        run_e2e.last = 0.0

        run_e2e(3)
        e2e_rounds = []
        for _ in range(rounds):
            sync_all(world)
            t0 = time.perf_counter()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            checks += run_e2e(args.steps)
            s1.record()
            sync_all(world)
            wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
            # the region ends with a host synchronisation, so device time and host wall time agree; take the larger
            e2e_rounds.append(max(max_over_ranks(s0.elapsed_time(s1) / args.steps, dev), max_over_ranks(wall_ms, dev)))
        e2e_ms = statistics.median(e2e_rounds)
        # The same host-to-device copy alone (all ranks at once, nothing else on the GPUs): what the platform gives.
        shard_bytes = host_a.numel() * host_a.element_size()
        sync_all(world)
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record()
        for i in range(8):
            bufs[1].local.copy_(host_a, non_blocking=True)
        h1.record()
        sync_all(world)
        h2d_alone_ms = max_over_ranks(h0.elapsed_time(h1) / 8, dev)
        bufs[1].local.copy_(a.local)
        e2e = {"value": 2.0 * m * n * k / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "rounds_ms": [round(x, 4) for x in e2e_rounds],
               "h2d_bytes_per_step": shard_bytes * world.size,
               "d2h_bytes_per_step": 8 * world.size, "checksums_read": len(checks),
               # rate at which each rank's copy stream had to deliver its activations to keep this step time, and
               # the rate of the same copy with the GPUs otherwise idle (all ranks copying at once)
               "h2d_gb_per_s_per_gpu": shard_bytes / (e2e_ms * 1e-3) / 1e9,
               "h2d_alone_ms": round(h2d_alone_ms, 4),
               "h2d_alone_gb_per_s_per_gpu": shard_bytes / (h2d_alone_ms * 1e-3) / 1e9,
               "result_read_back": "each rank's share of sum(C), accumulated by the kernel's epilogue into a running "
                                   "double; 8 bytes per rank and step",
               "pipelining": "copy of step i+1 overlaps compute of step i; checksum of step i is read during step i+1"}
        a_alt.free()
    clocks = sampler.stop() if sampler else None
    ug.check_status(dev)

    # ------------------------------------------------------------------ untimed: what was computed, and where the time goes
    verified = None
    if not args.no_verify:
        step()
        sync_all(world)
        ok, err, tol, checksum, sumsq = _verify(ug, world, a, b, c, c_dtype)
        # every end-to-end step multiplied the same operands: the ranks' shares of its checksum must add up to the
        # sum of the verified C
        # (atomic accumulation orders differ between steps, hence a small relative tolerance)
        if checks:
            import torch.distributed as dist

            totals = torch.tensor(checks + [checksum, sumsq], dtype=torch.float64, device=dev)
            if world.size > 1:
                dist.all_reduce(totals)                 # per step: sum of the ranks' shares; then sum and sum of squares of C
            checksum, sumsq = float(totals[-2]), float(totals[-1])
            checks = totals[:-2].tolist()
        # the kernel sums its fp32 accumulators, C holds them rounded to its dtype and summed in another order: allow
        # the rounding noise of that many elements (a random walk) on top of a relative term
        noise = (1e-2 if c_dtype == torch.bfloat16 else 1e-5) * sumsq ** 0.5
        bad = [x for x in checks if abs(x - checksum) > 1e-4 * abs(checksum) + noise + 1e-3]
        per_rank = _gather_floats([float(ok), err, tol, float(len(bad))], world, dev)
        verified = {"ok": all(r[0] > 0 for r in per_rank) and all(r[3] == 0 for r in per_rank),
                    "max_abs_err": max(r[1] for r in per_rank), "tolerance": max(r[2] for r in per_rank),
                    "rows_checked": 64 * world.size, "against": "fp32 product of the same bf16 operands (torch, no TF32)",
                    "e2e_checksums_compared": len(checks) * world.size,
                    "e2e_checksum_mismatches": int(sum(r[3] for r in per_rank))}

    breakdown = None
    if world.size > 1 or args.profile:
        ug.profile.reset_stats()
        ug.profile.enable(True)
        sync_all(world)
        for _ in range(args.steps):
            step()
        sync_all(world)
        snap = ug.profile.snapshot()
        ug.profile.enable(False)
        per_rank = _gather_floats([snap["comm_sync"] * 1e3 / args.steps, snap["compute"] * 1e3 / args.steps], world, dev)
        breakdown = {"barrier_ms_per_rank": [round(v[0], 4) for v in per_rank],
                     "fused_kernel_ms_per_rank": [round(v[1], 4) for v in per_rank]}
        # in-kernel timeline of one more step: how long producers waited for staged (remote) chunks, when the
        # fetch warps ran dry, how far apart the CTAs finished
        ug.trace.attach_cached()
        sync_all(world)
        step()
        sync_all(world)
        keys = ("kernel_us", "flagwait_us_mean_per_cta", "flagwait_us_max_per_cta", "fetch_end_us", "main_us_mean",
                "epilogue_us_mean", "cta_finish_spread_us", "main_loop_share_of_kernel", "sm_clock_ghz")
        items = ug.trace.collect()
        summ = max((it["summary"] for it in items), key=lambda s: s.get("kernel_us", 0.0), default={})
        per_rank = _gather_floats([float(summ.get(key, 0.0) or 0.0) for key in keys], world, dev)
        breakdown["timeline"] = {key: [round(v[i], 3) for v in per_rank] for i, key in enumerate(keys)}
        if items:
            breakdown["program"] = {kk: items[0]["stats"].get(kk) for kk in ("tile_m", "tiles", "pieces", "grid",
                                                                              "remote_bytes", "model_us")}
        if args.trace_dir:
            ug.trace.dump(args.trace_dir, rank=world.rank, chrome=world.rank == 0)
        ug.trace.detach_all()
        ug.check_status(dev)

    context = None
    if not args.no_context and in_dtype == torch.bfloat16:
        # Stock DTensor (sharding propagation + NCCL redistribute + cuBLAS) on the same bf16 shards, same launch,
        # same timing.  This is a library baseline measured by this script, not the reference arm.
        try:
            import torch.distributed as dist

            if not dist.is_initialized():       # one GPU without a launcher: DTensor still wants a process group
                import socket

                with socket.socket() as sock:
                    sock.bind(("127.0.0.1", 0))
                    port = sock.getsockname()[1]
                dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
            from benchmark.matmul_bench_worker import _dtensor_iteration

            dt_a, dt_b = a.to_dtensor(), b.to_dtensor()
            for _ in range(3):
                _dtensor_iteration(dt_a, dt_b)
            dt_rounds = []                     # same protocol as the timed region above: rounds of --steps steps
            for _ in range(rounds):
                d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                sync_all(world)
                d0.record()
                for _ in range(args.steps):
                    _dtensor_iteration(dt_a, dt_b)
                d1.record()
                sync_all(world)
                dt_rounds.append(max_over_ranks(d0.elapsed_time(d1) / args.steps, dev))
            dt_ms = statistics.median(dt_rounds)
            context = {"dtensor_bf16_tflops": 2.0 * m * n * k / (dt_ms * 1e-3) / 1e12, "dtensor_bf16_ms_per_step": dt_ms,
                       "rounds_ms": [round(x, 4) for x in dt_rounds],
                       "what": "torch DTensor matmul + redistribute of Partial results (NCCL + cuBLAS), bf16 operands, "
                               "output placement chosen by DTensor; CUDA events, max over ranks, median of the same "
                               "number of rounds and steps as `value`"}
        except Exception as exc:  # noqa: BLE001
            context = {"dtensor_bf16_tflops": None, "error": f"{type(exc).__name__}: {str(exc)[:160]}"}

    flops = 2.0 * m * n * k
    value = flops / (ms_per_step * 1e-3) / 1e12
    shard_bytes = min(a.nbytes, b.nbytes, c.nbytes)
    result = {
        "metric": METRIC,
        "value": value, "unit": "TFLOP/s", "n_gpus": world.size, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16" if in_dtype == torch.bfloat16 else "fp32 operands as three bf16 products (hi x hi + hi x lo + lo x hi)",
        "data": "synthetic (random-init N(0, 0.02) weights and activations)",
        "impl": "ours", "gpu_launches": launches, "rounds": rounds, "rounds_ms": [round(x, 4) for x in rounds_ms],
        "clocks": clocks, "e2e": e2e, "verified": verified, "breakdown": breakdown, "context": context,
        "config": {"model": "GPT-3-175B MLP up-projection GEMM" if (n, k) == (49152, 12288) else "GEMM",
                   "m": m, "n": n, "k": k, "global_batch": m, "seq_len": None,
                   "parallelism": f"{args.a_partition},{args.b_partition},{args.c_partition} rep{args.replication} "
                                  f"{method} x{world.size}",
                   "c_dtype": args.c_dtype, "accumulate": "fp32 (TMEM)",
                   "timing": f"CUDA events around {rounds} rounds of {args.steps} steps, each round max over ranks; "
                             "value = median round; gpu_launches = kernels of this package per round",
                   "l2": f"inputs larger than L2 (B shard {b.nbytes >> 20} MiB, C shard {c.nbytes >> 20} MiB per rank)"
                         if max(a.nbytes, b.nbytes, c.nbytes) > 126 * 2 ** 20 else
                         f"smallest shard {shard_bytes >> 20} MiB; C is rewritten every step",
                   "step": "C = A @ B: barrier + fused GEMM + barrier (C zeroed first only when K is split across ranks)"},
    }
    rank = world.rank
    world.close()
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()
    if rank == 0 and verified is not None and not verified["ok"]:
        print(json.dumps(result), flush=True)
        raise SystemExit("bench.py: the distributed product does not match the fp32 check")
    return result if rank == 0 else {}


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(REPO, "baseline"))
        import run_reference

        return run_reference.main(args, METRIC)
    if args.gpus > 1 and "RANK" not in os.environ:
        return _relaunch_under_torchrun(args)
    result = run_ours(args)
    if result:
        print(json.dumps(result), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
