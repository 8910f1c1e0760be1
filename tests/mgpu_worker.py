"""Multi-process worker for the multi-GPU (or multi-process CPU) tests.

Launched by ``torch.distributed.run`` with one rank per GPU (``--device cuda``) or as gloo
ranks on CPU (``--device cpu``).  Every rank builds the same full matrices from a seed,
distributes them into symmetric memory, runs the requested methods and compares the gathered
result against an fp64 oracle.  Exit code 0 means every case passed on every rank.
"""
from __future__ import annotations

import argparse
import itertools
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402


def large_cases(world) -> tuple[int, int]:
    """Shapes on which the machinery of the fused kernel runs for real on several GPUs: several waves of tiles per
    rank, megabytes of staged remote operands, remote stores / red.add of whole tiles, every tile variant with static
    and dynamic tile order, replication 1 and 2, fp32 and bf16 C; then redistribute and put + signal between GPUs.
    The status word is checked after every case.  Returns (failures, cases)."""
    from universal_gemm_b200.parallel.exec import clear_program_cache

    dev, rank, size = world.device, world.rank, world.size
    failures = ncases = 0
    configs = [((2048, 3072, 4096), t) for t in (("row", "row", "row"), ("row", "column", "row"),
                                                 ("column", "row", "row"), ("block", "block", "block"))]
    configs += [((2048, 12288, 3072), ("row", "column", "row")), ((2048, 3072, 12288), ("column", "row", "row"))]
    saved = {key: os.environ.get(key) for key in ("UGEMM_TILE_M", "UGEMM_DYNAMIC_TILES")}
    for (m, n, k), triple in configs:
        g = torch.Generator().manual_seed(99 + m + n + k)
        full_a = torch.randn(m, k, generator=g).to(dev)
        full_b = (torch.randn(k, n, generator=g) / k ** 0.5).to(dev)
        want = full_a.bfloat16().double() @ full_b.bfloat16().double()
        scale = max(1.0, want.abs().max().item())
        for rep, c_dtype in itertools.product([r for r in (1, 2) if size % r == 0], (torch.float32, torch.bfloat16)):
            a = ug.distribute_tensor(full_a, world, triple[0], rep, dtype=torch.bfloat16)
            b = ug.distribute_tensor(full_b, world, triple[1], rep, dtype=torch.bfloat16)
            c = ug.zeros(world, (m, n), triple[2], c_dtype, rep)
            for variant, dyn, method in itertools.product(("128", "256", "pair", "pair512"), ("0", "1"),
                                                          ("stationary_c", "stationary_b")):
                os.environ["UGEMM_TILE_M"], os.environ["UGEMM_DYNAMIC_TILES"] = variant, dyn
                clear_program_cache()
                c.local_padded.fill_(7.0)                        # beta = 0 must not depend on what C held
                torch.cuda.synchronize()
                world.barrier()
                for _ in range(2):                               # second call: counters and claims were re-armed
                    ug.matmul(a, b, c, method=method, beta=0)
                torch.cuda.synchronize()
                what = f"{m}x{n}x{k} {triple} rep={rep} {c_dtype} tile={variant} dyn={dyn} {method}"
                try:
                    ug.check_status(dev)
                except Exception as exc:  # noqa: BLE001
                    failures += 1
                    print(f"[rank {rank}] status error in {what}: {exc}", flush=True)
                world.barrier()
                got = c.full_tensor(replica=0).double()
                torch.cuda.synchronize()
                err = (got - want).abs().max().item()
                tol = (3e-3 if c_dtype == torch.float32 else 3e-2) * scale
                ncases += 1
                if not err <= tol:
                    failures += 1
                    print(f"[rank {rank}] FAIL {what}: max err {err:.3e} (tolerance {tol:.1e})", flush=True)
                world.barrier()
            for mat in (a, b, c):
                mat.free()
    for key, val in saved.items():
        if val is None:
            os.environ.pop(key, None)
        else:
            os.environ[key] = val
    clear_program_cache()

    # redistribute between partitions over real peers (one-sided pulls), with and without a dtype change
    full = torch.randn(1531, 2045, generator=torch.Generator().manual_seed(5)).to(dev)
    src = ug.distribute_tensor(full, world, "block")
    for part, dtype in (("column", None), ("row", torch.bfloat16)):
        out = ug.redistribute(src, part, dtype=dtype)
        torch.cuda.synchronize()
        world.barrier()
        got = out.full_tensor()
        torch.cuda.synchronize()
        ncases += 1
        if not torch.equal(got.float(), full if dtype is None else full.bfloat16().float()):
            failures += 1
            print(f"[rank {rank}] FAIL redistribute block -> {part} {dtype}", flush=True)
        world.barrier()
        out.free()
    src.free()

    # put + signal: every rank writes a row into its neighbour's window and signals; the receiver's stream waits
    window = ug.zeros(world, (size, 4096), "row", torch.float32)
    pad = ug.SignalPad(world, slots=4)
    dst = (rank + 1) % size
    payload = torch.full((1, 4000), float(rank + 1), device=dev)
    ug.put_tile(window, (dst, 0), payload, slice_=ug.Slice2D(ug.Slice1D(0, 1), ug.Slice1D(8, 4008)))
    pad.signal(dst, slot=1)
    pad.wait(slot=1, value=1)
    torch.cuda.synchronize()
    ncases += 1
    try:
        ug.check_status(dev)
        row = window.local[0]
        src_rank = (rank - 1) % size
        if not (bool((row[8:4008] == float(src_rank + 1)).all()) and float(row[:8].abs().sum()) == 0.0
                and float(row[4008:].abs().sum()) == 0.0):
            raise AssertionError("window contents differ from what the neighbour put")
    except Exception as exc:  # noqa: BLE001
        failures += 1
        print(f"[rank {rank}] FAIL put + signal: {exc}", flush=True)
    world.barrier()
    window.free()
    return failures, ncases


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--cases", default="small")
    ap.add_argument("--world", default="", help='"symm_mem": symmetric allocations from torch symmetric memory')
    args = ap.parse_args()
    world = ug.init(device=args.device, world=args.world or None)
    dev = world.device
    in_dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    rank, size = world.rank, world.size
    parts = ("row", "column", "block")
    if args.cases == "small":
        shapes = [(301, 203, 157)]
        triples = list(itertools.product(parts, repeat=3))
        reps = [r for r in (1, 2) if size % r == 0]
    elif args.cases == "tiny":
        shapes = [(64, 48, 40)]
        triples = [("row", "row", "row"), ("row", "column", "row"), ("column", "row", "row"), ("block", "block", "block")]
        reps = [r for r in (1, 2) if size % r == 0]
    else:
        shapes = [(2048, 3072, 4096)]
        triples = [("row", "row", "row"), ("row", "column", "row"), ("column", "row", "row"), ("block", "block", "block")]
        reps = [r for r in (1, 2) if size % r == 0]
    failures = 0
    ncases = 0
    if args.cases == "large":
        f, nc = large_cases(world)
        failures += f
        ncases += nc
        shapes = []
    for (m, n, k), triple, rep, method in itertools.product(shapes, triples, reps, ("stationary_c", "stationary_b")):
        g = torch.Generator().manual_seed(1234 + m + n + k)
        full_a = torch.randn(m, k, generator=g).to(dev)
        full_b = (torch.randn(k, n, generator=g) / k ** 0.5).to(dev)
        full_c = torch.randn(m, n, generator=g).to(dev)
        a = ug.distribute_tensor(full_a, world, triple[0], rep, dtype=in_dtype)
        b = ug.distribute_tensor(full_b, world, triple[1], rep, dtype=in_dtype)
        c = ug.distribute_tensor(full_c, world, triple[2], rep, dtype=torch.float32)
        iters = 2
        ug.matmul(a, b, c, method=method, beta=0)                # C = A @ B, whatever C held
        if dev.type == "cuda":
            torch.cuda.synchronize()
        world.barrier()
        got0 = c.full_tensor(replica=0).double()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        want0 = full_a.to(in_dtype).double() @ full_b.to(in_dtype).double()
        err0 = (got0 - want0).abs().max().item()
        if err0 > 3e-3 * max(1.0, want0.abs().max().item()):
            failures += 1
            print(f"[rank {rank}] FAIL beta=0 {m}x{n}x{k} {triple} rep={rep} {method}: max err {err0:.3e}", flush=True)
        world.barrier()
        c.local.copy_(full_c[ug.tile_bounds(c.layout, c.coord).rows.as_slice(), ug.tile_bounds(c.layout, c.coord).cols.as_slice()])
        if dev.type == "cuda":
            torch.cuda.synchronize()
        world.barrier()
        for _ in range(iters):
            ug.matmul(a, b, c, method=method)
        if dev.type == "cuda":
            torch.cuda.synchronize()
            try:
                ug.check_status(dev)
            except Exception as exc:  # noqa: BLE001
                print(f"[rank {rank}] status error in {triple} rep={rep} {method}: {exc}", flush=True)
                failures += 1
        world.barrier()
        got = c.full_tensor(replica=0).double()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        want = full_c.double() + iters * (full_a.to(in_dtype).double() @ full_b.to(in_dtype).double())
        err = (got - want).abs().max().item()
        ok = err <= 3e-3 * max(1.0, want.abs().max().item())
        ncases += 1
        if not ok:
            failures += 1
            print(f"[rank {rank}] FAIL {m}x{n}x{k} {triple} rep={rep} {method}: max err {err:.3e}", flush=True)
        world.barrier()
        for mat in (a, b, c):
            mat.free()
    # prepared plan replayed from a CUDA graph (GPU only): barriers keep their round counter on the device
    if dev.type == "cuda":
        m, n, k = 384, 512, 448
        g = torch.Generator().manual_seed(11)
        full_a, full_b = torch.randn(m, k, generator=g).to(dev), (torch.randn(k, n, generator=g) / 20).to(dev)
        a = ug.distribute_tensor(full_a, world, "row", dtype=in_dtype)
        b = ug.distribute_tensor(full_b, world, "row", dtype=in_dtype)          # K split: Stationary-B adds atomically
        c = ug.zeros(world, (m, n), "row", torch.float32)
        plan = ug.prepare_matmul(a, b, c, method="stationary_b", beta=1).capture()
        torch.cuda.synchronize()
        world.barrier()
        c.local_padded.zero_()
        torch.cuda.synchronize()
        world.barrier()
        for _ in range(4):
            plan()
        torch.cuda.synchronize()
        ug.check_status(dev)
        world.barrier()
        got = c.full_tensor().double()
        torch.cuda.synchronize()
        want = 4 * (full_a.to(in_dtype).double() @ full_b.to(in_dtype).double())
        ncases += 1
        if (got - want).abs().max().item() > 3e-3 * max(1.0, want.abs().max().item()):
            failures += 1
            print(f"[rank {rank}] FAIL cuda-graph replay", flush=True)
        world.barrier()

    # torch.addmm(c, a, b, out=c) on DTensors through the dispatch hook
    m, n, k = 96, 80, 72
    g = torch.Generator().manual_seed(7)
    full_a, full_b = torch.randn(m, k, generator=g).to(dev), (torch.randn(k, n, generator=g) / 8).to(dev)
    a = ug.distribute_tensor(full_a, world, "row", dtype=in_dtype)
    b = ug.distribute_tensor(full_b, world, "column", dtype=in_dtype)
    c = ug.zeros(world, (m, n), "block" if size > 1 else "row", torch.float32)
    ug.mm_handler.enable("auto")
    try:
        dc = c.to_dtensor()
        out = torch.addmm(dc, a.to_dtensor(), b.to_dtensor(), out=dc)
        assert out is dc
    finally:
        ug.mm_handler.disable()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    world.barrier()
    got = c.full_tensor().double()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    want = full_a.to(in_dtype).double() @ full_b.to(in_dtype).double()
    ncases += 1
    if (got - want).abs().max().item() > 3e-3 * max(1.0, want.abs().max().item()):
        failures += 1
        print(f"[rank {rank}] FAIL addmm hook", flush=True)
    world.barrier()

    try:                                         # guard regions (UGEMM_GUARD_BYTES): nothing wrote outside a shard
        guarded = world.check_guards()
    except ug.GuardViolation as exc:
        guarded = -1
        failures += 1
        print(f"[rank {rank}] FAIL {exc}", flush=True)
    if rank == 0:
        print(f"mgpu_worker: guarded allocations checked on rank 0: {guarded}", flush=True)

    t = torch.tensor([failures], device=dev, dtype=torch.int64)
    dist.all_reduce(t)
    if rank == 0:
        print(f"mgpu_worker: world={size} device={dev.type} cases={ncases} failures={int(t.item())}", flush=True)
    world.close()
    dist.destroy_process_group()
    return 1 if int(t.item()) else 0


if __name__ == "__main__":
    sys.exit(main())
