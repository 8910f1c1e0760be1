#!/usr/bin/env python3
"""Smoke test of asynchronous tile fetches: rank 0 fetches every tile of a small row-partitioned matrix and
checks shapes and values (what the reference's get_tile_async_test.py:59-72 checks, plus the values)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402


def main() -> None:
    world = ug.init()
    dev = world.device
    full = torch.arange(64 * 64, dtype=torch.float32, device=dev).reshape(64, 64)
    dm = ug.distribute_tensor(full, world, "row")
    ug.init_scratch(4 * ug.tile_shape(dm)[0] * ug.tile_shape(dm)[1], torch.float32, world=world)
    world.barrier()
    if world.rank == 0:
        grid = ug.grid_shape(dm)
        futures = {(i, j): ug.get_tile_async(dm, (i, j)) for i in range(grid[0]) for j in range(grid[1])}
        for coord, fut in futures.items():
            t = fut.get()
            if world.is_cuda:
                torch.cuda.synchronize()
            b = ug.tile_bounds(dm, coord)
            assert tuple(t.shape) == ug.tile_shape(dm, coord), (coord, t.shape)
            assert torch.equal(t, full[b.rows.as_slice(), b.cols.as_slice()])
            print(f"tile {coord}: shape {tuple(t.shape)} first value {float(t.flatten()[0]) if t.numel() else None}")
            ug.release_tile(t)
        print("get_tile_async smoke ok")
    world.barrier()
    ug.free_get_tile_scratch()
    world.close()
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
