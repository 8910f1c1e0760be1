"""Reference arm of ``bench.py``: run the reference's own benchmark worker, unmodified.

``baseline/_ref`` holds a verbatim copy of the reference tree (it has no ``setup.py`` /
``pyproject.toml``, so ``pip install --target baseline/_ref`` refuses it; the files are copied
instead).  This module runs ``baseline/_ref/benchmark/matmul_bench_worker.py`` in-process with its
own command line, for the reference's ``dtensor`` method (sharding propagation + NCCL
redistribute + cuBLAS).  The worker is fp32-only and times with the host clock between
barriers; both are the reference's stock behaviour and are reported as such.

The reference's ``stationary_b`` / ``stationary_c`` methods need nvshmem4py, ``cuda.core`` and a
patched PyTorch that provides ``DTensor.nvshmem_base()``; none exists on this image, so they are
reported as unavailable rather than emulated.
"""
from __future__ import annotations

import json
import os
import runpy
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
WORKER = os.path.join(REF, "benchmark", "matmul_bench_worker.py")


def _unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def main(args) -> int:
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

    ref_stubs.install()
    sampler = None
    if rank == 0:
        sys.path.insert(0, os.path.dirname(HERE))
        try:
            from universal_gemm_b200.utils.benchmarking import ClockSampler

            sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
            sampler.start()
        except Exception:  # noqa: BLE001
            sampler = None
    argv = [WORKER, "--method", "dtensor", "--m", str(args.m), "--n", str(args.n), "--k", str(args.k),
            "--a-partition", a_p, "--b-partition", b_p, "--c-partition", c_p,
            "--replication-factor", str(args.replication), "--warmup-iters", str(max(args.warmup, 3)),
            "--measure-iters", str(args.steps), "--result-file", result_file]
    saved = sys.argv
    sys.argv = argv
    try:
        runpy.run_path(WORKER, run_name="__main__")
    except SystemExit as exc:
        if exc.code not in (None, 0):
            return _unavailable(f"reference worker exited with {exc.code}")
    except Exception as exc:  # noqa: BLE001
        return _unavailable(f"reference worker raised {type(exc).__name__}: {str(exc)[:200]}")
    finally:
        sys.argv = saved
    clocks = sampler.stop() if sampler else None
    if rank != 0:
        return 0
    if not os.path.exists(result_file):
        return _unavailable("reference worker wrote no result file")
    with open(result_file, encoding="utf-8") as f:
        res = json.load(f)
    line = {
        "metric": "whole-box TFLOP/s (2*M*N*K / time per iteration, max over ranks)",
        "value": res["median_tflops"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": res["median_seconds"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 (hard-coded by the reference worker; cuBLAS without TF32)", "data": "synthetic (torch.randn)",
        "impl": "reference", "clocks": clocks,
        "config": {"model": "GPT-3-175B MLP up-projection GEMM" if (args.n, args.k) == (49152, 12288) else "GEMM",
                   "m": args.m, "n": args.n, "k": args.k, "global_batch": args.m, "seq_len": None,
                   "parallelism": f"{a_p},{b_p},{c_p} rep{args.replication} dtensor x{world}",
                   "method": "dtensor (reference's plain DTensor matmul: NCCL redistribute + cuBLAS)",
                   "timing": "host wall clock between NCCL barriers, max over ranks, median of iterations "
                             "(the reference's own timing)",
                   "max_tflops": res["max_tflops"]},
    }
    print(json.dumps(line), flush=True)
    return 0
