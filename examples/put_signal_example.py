#!/usr/bin/env python3
"""One-sided put + signal between neighbouring ranks (launch with torchrun, any number of ranks >= 1).

Every rank writes ten floats into the next rank's window at an offset, then signals; the receiver waits on its
own signal slot (a bounded device-side wait on the GPU) and prints what arrived.  The put / signal /
wait_signal protocol of the reference's window experiments (torchcomms/put_01.py, put_02.py), expressed with
this package's symmetric memory."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import universal_gemm_b200 as ug  # noqa: E402


def main() -> None:
    world = ug.init()
    rank, size, dev = world.rank, world.size, world.device
    window = ug.zeros(world, (size, 32), "row", torch.float32)          # one 32-float row per rank
    pad = ug.SignalPad(world, slots=4)
    dst = (rank + 1) % size
    payload = torch.full((1, 10), float(rank + 1), device=dev)
    ug.put_tile(window, (dst, 0), payload, slice_=ug.Slice2D(ug.Slice1D(0, 1), ug.Slice1D(4, 14)))
    pad.signal(dst, slot=0)
    pad.wait(slot=0, value=1)
    if world.is_cuda:
        torch.cuda.synchronize()
        ug.check_status(dev)
    got = window.local[0, :16].tolist()
    print(f"[Rank {rank}] received from rank {(rank - 1) % size}: {got}")
    assert got[4:14] == [float((rank - 1) % size + 1)] * 10 and got[:4] == [0.0] * 4
    world.barrier()
    world.close()
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
