"""Reference arm of ``bench.py``: run the reference's own benchmark worker, unmodified.

``baseline/_ref`` holds a verbatim copy of the reference tree (it has no ``setup.py`` /
``pyproject.toml``, so ``pip install --target baseline/_ref`` refuses it; the files are copied
instead).  This module runs ``baseline/_ref/benchmark/matmul_bench_worker.py`` in-process with its
own command line, for the reference's ``dtensor`` method (sharding propagation + NCCL
redistribute + cuBLAS).  The worker is fp32-only and times with the host clock between
barriers; both are the reference's stock behaviour and are reported as such.  ``value`` is what
that unmodified run wrote into its result file.

``e2e`` is measured afterwards with the worker's own set-up functions and the same call sequence
as its ``dtensor`` iteration (the worker's ``_execute_one_iteration`` discards the product, so the
sequence is repeated here to be able to read a checksum of it): every step copies the rank's A
shard from pinned host memory into the DTensor's local tensor, multiplies, and reads a 4-byte
checksum of the local result back to the host; timed like the worker times, host clock between
barriers, max over ranks, median of the steps.

Nothing of the ``universal_gemm_b200`` package is imported here.

The reference's ``stationary_b`` / ``stationary_c`` methods need nvshmem4py, ``cuda.core`` and a
patched PyTorch that provides ``DTensor.nvshmem_base()``; none exists on this image, so they are
reported as unavailable rather than emulated.
"""
from __future__ import annotations

import json
import os
import runpy
import statistics
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
WORKER = os.path.join(REF, "benchmark", "matmul_bench_worker.py")


def _unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def _e2e(g: dict, parts: tuple[str, str, str], args, steps: int, seed: int = 20260218) -> dict:
    """End-to-end step time of the reference's ``dtensor`` method (see the module docstring).  ``g`` are the
    globals of the executed worker module: its partition helper, its ``bench_util`` and torch."""
    import torch
    import torch.distributed as dist
    from torch.distributed.tensor import distribute_tensor

    bench_util = g["bench_util"]
    dist.init_process_group(backend="nccl")
    try:
        rank = dist.get_rank()
        gpu_id = rank % torch.cuda.device_count()
        torch.cuda.set_device(gpu_id)
        device = torch.device(f"cuda:{gpu_id}")
        torch.manual_seed(seed + rank)
        a_p = g["_get_partitioning"](parts[0], args.replication)
        b_p = g["_get_partitioning"](parts[1], args.replication)
        full_a = torch.randn(args.m, args.k, dtype=torch.float32, device=device)
        full_b = torch.randn(args.k, args.n, dtype=torch.float32, device=device)
        dt_a = distribute_tensor(full_a, *a_p)
        dt_b = distribute_tensor(full_b, *b_p)
        del full_a, full_b
        local_a = dt_a.to_local()
        host_a = torch.empty(local_a.shape, dtype=local_a.dtype).pin_memory()
        host_a.copy_(local_a)

        def iteration() -> float:
            local_a.copy_(host_a, non_blocking=True)                     # this step's activations
            dt_out = torch.matmul(dt_a, dt_b)
            need, placements = bench_util.materialized_placements(dt_out.device_mesh, dt_out.placements)
            if need:
                dt_out = dt_out.redistribute(dt_out.device_mesh, placements)
            return float(dt_out.to_local().sum(dtype=torch.float32).item())   # 4 bytes back to the host

        for _ in range(2):
            iteration()
            dist.barrier()
        durations = []
        for _ in range(steps):
            dist.barrier()
            t0 = time.perf_counter()
            iteration()
            dist.barrier()
            elapsed = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
            durations.append(float(elapsed.item()))
        sec = statistics.median(durations)
        world = dist.get_world_size()
        return {"value": 2.0 * args.m * args.n * args.k / sec / 1e12, "unit": "TFLOP/s", "ms_per_step": sec * 1e3,
                "h2d_bytes_per_step": host_a.numel() * host_a.element_size() * world, "d2h_bytes_per_step": 4 * world,
                "pipelining": "none (copy, multiply and read-back run one after the other; the reference has no "
                              "asynchronous entry point for its dtensor method)"}
    finally:
        try:
            dist.barrier()
        except Exception:  # noqa: BLE001
            pass
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def main(args, metric: str) -> int:
    if not os.path.exists(WORKER):
        return _unavailable("baseline/_ref is missing: the reference tree is not pip-installable (no setup.py / "
                            "pyproject.toml) and its copy was not found")
    try:
        import torch
    except Exception as exc:  # noqa: BLE001
        return _unavailable(f"torch import failed: {exc}")
    if not torch.cuda.is_available():
        return _unavailable("no CUDA device")
    part = {"col": "column"}
    a_p, b_p, c_p = (part.get(p, p) for p in (args.a_partition, args.b_partition, args.c_partition))
    if "RANK" not in os.environ:
        if args.gpus != 1:
            return _unavailable("launch with torch.distributed.run for more than one GPU")
        os.environ.update({"RANK": "0", "WORLD_SIZE": "1", "LOCAL_RANK": "0", "MASTER_ADDR": "127.0.0.1",
                           "MASTER_PORT": str(args.master_port)})
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    if world != args.gpus:
        return _unavailable(f"--gpus {args.gpus} but the launcher started {world} rank(s)")
    out_dir = os.environ.get("UGEMM_REF_OUT") or os.path.join(tempfile.gettempdir(), f"ugemm_ref_{os.environ.get('MASTER_PORT', '0')}")
    result_file = os.path.join(out_dir, "result.json")
    if rank == 0 and os.path.exists(result_file):
        os.unlink(result_file)

    sys.path.insert(0, HERE)
    import ref_stubs
    from clock_sampler import ClockSampler

    ref_stubs.install()
    sampler = None
    if rank == 0:
        sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
        if not sampler.start():
            sampler = None
    warmup = max(args.warmup, 3)
    argv = [WORKER, "--method", "dtensor", "--m", str(args.m), "--n", str(args.n), "--k", str(args.k),
            "--a-partition", a_p, "--b-partition", b_p, "--c-partition", c_p,
            "--replication-factor", str(args.replication), "--warmup-iters", str(warmup),
            "--measure-iters", str(args.steps), "--result-file", result_file]
    saved = sys.argv
    sys.argv = argv
    try:
        worker_globals = runpy.run_path(WORKER, run_name="__main__")
    except SystemExit as exc:
        if exc.code not in (None, 0):
            return _unavailable(f"reference worker exited with {exc.code}")
        worker_globals = None
    except Exception as exc:  # noqa: BLE001
        return _unavailable(f"reference worker raised {type(exc).__name__}: {str(exc)[:200]}")
    finally:
        sys.argv = saved
    e2e = None
    if worker_globals is not None and not getattr(args, "no_e2e", False):
        try:
            e2e = _e2e(worker_globals, (a_p, b_p, c_p), args, args.steps)
        except Exception as exc:  # noqa: BLE001
            e2e = {"value": None, "error": f"{type(exc).__name__}: {str(exc)[:200]}"}
    clocks = sampler.stop() if sampler else None
    if rank != 0:
        return 0
    if not os.path.exists(result_file):
        return _unavailable("reference worker wrote no result file")
    with open(result_file, encoding="utf-8") as f:
        res = json.load(f)
    line = {
        "metric": metric,
        "value": res["median_tflops"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": res["median_seconds"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 (hard-coded by the reference worker; cuBLAS without TF32)", "data": "synthetic (torch.randn)",
        "impl": "reference", "clocks": clocks, "e2e": e2e,
        "config": {"model": "GPT-3-175B MLP up-projection GEMM" if (args.n, args.k) == (49152, 12288) else "GEMM",
                   "m": args.m, "n": args.n, "k": args.k, "global_batch": args.m, "seq_len": None,
                   "parallelism": f"{a_p},{b_p},{c_p} rep{args.replication} dtensor x{world}",
                   "method": "dtensor (reference's plain DTensor matmul: NCCL redistribute + cuBLAS); its "
                             "stationary_b / stationary_c need nvshmem4py, cuda.core and a patched PyTorch and are "
                             "unavailable on this image",
                   "timing": "host wall clock between NCCL barriers, max over ranks, median of the steps "
                             "(the reference's own timing)",
                   "max_tflops": res["max_tflops"]},
    }
    print(json.dumps(line), flush=True)
    return 0
