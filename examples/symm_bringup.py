#!/usr/bin/env python3
"""Bring-up of the symmetric-memory layer without ``torch.distributed``: every process is started by hand
(or by any launcher) with RANK / WORLD_SIZE and a shared directory, exchanges CUDA IPC handles through files
with a poll timeout, allocates a symmetric buffer and checks that a peer's write is visible.

    UGEMM_RDZV_DIR=/tmp/rdzv RANK=0 WORLD_SIZE=2 python examples/symm_bringup.py &
    UGEMM_RDZV_DIR=/tmp/rdzv RANK=1 WORLD_SIZE=2 python examples/symm_bringup.py

Role of the reference's nvshmem_init_only.py / nvshmem_example.py / symm_mem_example.py (initialise, allocate
symmetric memory, move data one-sided); on a machine without GPUs it uses the shared-memory world."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402


def main() -> None:
    rank, size = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    comm = ug.FileComm(os.environ.get("UGEMM_RDZV_DIR", "/tmp/ugemm_rdzv"), rank, size, timeout_s=30.0)
    if torch.cuda.is_available():
        torch.cuda.set_device(rank % torch.cuda.device_count())
        world = ug.CudaIpcWorld(comm=comm)
    else:
        world = ug.ShmWorld(comm=comm)
    print(f"[Rank {rank}] world of {size} ranks on {world.device}")
    buf = ug.zeros(world, (size, 8), "row", torch.float32)
    ug.put_tile(buf, ((rank + 1) % size, 0), torch.full((1, 8), float(rank), device=world.device))
    if world.is_cuda:
        torch.cuda.synchronize()
    world.barrier()
    print(f"[Rank {rank}] my row now holds {buf.local[0].tolist()} (written by rank {(rank - 1) % size})")
    assert buf.local[0].tolist() == [float((rank - 1) % size)] * 8
    world.close()


if __name__ == "__main__":
    main()
