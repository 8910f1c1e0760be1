#!/usr/bin/env python3
"""How well does an asynchronous tile fetch overlap with local compute?  Rank 0 starts ``get_tile_async`` on a
large remote tile, runs small GEMMs meanwhile, and prints issue / compute / wait times (the experiment of the
reference's dtensor_async_test.py:85-127; here ``get()`` orders the stream instead of blocking the host)."""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192, help="rows of the remote tile")
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--small", type=int, default=1024, help="size of the local GEMMs run during the fetch")
    ap.add_argument("--gemms", type=int, default=20)
    args = ap.parse_args()
    world = ug.init()
    dev, size = world.device, world.size
    dtype = torch.bfloat16 if world.is_cuda else torch.float32
    big = ug.empty(world, (args.rows * size, args.cols), "row", dtype)
    big.local.normal_()
    ug.init_scratch(2 * args.rows * args.cols, dtype, world=world)
    x = torch.randn(args.small, args.small, device=dev, dtype=dtype)
    world.barrier()
    if world.rank == 0:
        sync = (lambda: torch.cuda.synchronize()) if world.is_cuda else (lambda: None)
        sync()
        t0 = time.perf_counter()
        fut = ug.get_tile_async(big, ((size - 1), 0))
        t1 = time.perf_counter()
        for _ in range(args.gemms):
            x = (x @ x) * 1e-3
        t2 = time.perf_counter()
        tile = fut.get()
        sync()
        t3 = time.perf_counter()
        mb = tile.numel() * tile.element_size() / 2 ** 20
        print(f"issue {1e3 * (t1 - t0):.3f} ms, host time of {args.gemms} GEMMs {1e3 * (t2 - t1):.3f} ms, "
              f"until tile ready {1e3 * (t3 - t0):.3f} ms for {mb:.0f} MiB")
    world.barrier()
    ug.free_get_tile_scratch()
    world.close()
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
