"""Worker for the file-rendezvous tests: CPU ranks without torch.distributed.

``python filecomm_worker.py DIR RANK SIZE MODE``; MODE ``ok`` runs a small distributed GEMM over a
shared-memory world bootstrapped through files; MODE ``absent`` makes the last rank exit before joining,
so the others must raise TimeoutError (exit code 3) instead of hanging."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402
from universal_gemm_b200.parallel.symm import FileComm, ShmWorld  # noqa: E402


def main() -> int:
    directory, rank, size, mode = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    if mode == "absent" and rank == size - 1:
        return 0                                    # this rank never joins
    comm = FileComm(directory, rank, size, timeout_s=2.0 if mode == "absent" else 60.0)
    try:
        world = ShmWorld(comm=comm)
    except TimeoutError as exc:
        print(f"rank {rank}: {exc}", flush=True)
        return 3
    g = torch.Generator().manual_seed(5)
    full_a, full_b = torch.randn(40, 24, generator=g), torch.randn(24, 32, generator=g)
    a = ug.distribute_tensor(full_a, world, "row")
    b = ug.distribute_tensor(full_b, world, "column")
    c = ug.zeros(world, (40, 32), "block" if size > 1 else "row", torch.float32)
    ug.matmul(a, b, c, method="stationary_b", beta=0)
    world.barrier()
    ok = torch.allclose(c.full_tensor(), full_a @ full_b, atol=1e-4)
    world.close()
    print(f"rank {rank}: {'ok' if ok else 'MISMATCH'}", flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
