"""Partition helpers: row / column / 2-D block partitions with a replication factor.

Each helper returns a :class:`Partitioning` = (mesh of ranks, placements).  The
meshes match the reference's helpers (benchmark/util.py:63-126): replica groups
are contiguous chunks of ranks, a replicated layout is the mesh ``[r, P/r]`` (or
``[r, pr, pc]``) with ``Replicate()`` first, ``r == P`` collapses to a flat mesh
with a single ``Replicate()``, and the 2-D grid uses the two closest factors with
the larger one on rows.  Unlike the reference, a block partition of a single rank
is a valid 1 x 1 grid.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Any, Iterator

import numpy as np

from .tiles import Layout, Partial, Placement, Replicate, Shard

PARTITION_NAMES = ("row", "column", "block")


def normalize_partition(name: str) -> str:
    name = name.strip().lower()
    if name == "col":
        name = "column"
    if name not in PARTITION_NAMES:
        raise ValueError(f"unknown partition {name!r}; expected one of row, column (col), block")
    return name


def closest_factors(n: int) -> tuple[int, int]:
    """The factor pair ``(a, b)`` of ``n`` with ``a >= b`` and ``a - b`` minimal."""
    if n <= 0:
        raise ValueError("n must be positive")
    for i in range(math.isqrt(n), 0, -1):
        if n % i == 0:
            return (n // i, i)
    raise AssertionError("unreachable")


def get_rank_from_env() -> int:
    for var in ("PMI_RANK", "PMIX_RANK", "RANK"):
        if var in os.environ:
            return int(os.environ[var])
    raise RuntimeError("none of PMI_RANK, PMIX_RANK, RANK is set; launch with mpirun or torchrun")


def get_nprocs_from_env() -> int:
    for var in ("PMI_SIZE", "WORLD_SIZE"):
        if var in os.environ:
            return int(os.environ[var])
    raise RuntimeError("neither PMI_SIZE nor WORLD_SIZE is set; launch with mpirun or torchrun")


@dataclass(frozen=True)
class Partitioning:
    mesh: np.ndarray
    placements: tuple[Placement, ...]

    def __iter__(self) -> Iterator[Any]:
        # allows ``mesh, placements = partitioning``
        yield self.mesh
        yield list(self.placements)

    def layout(self, shape: tuple[int, int]) -> Layout:
        return Layout(shape, self.mesh, self.placements)

    def to_torch(self, device_type: str = "cuda"):
        """(DeviceMesh, [torch placements]) for use with torch DTensor APIs."""
        import torch
        from torch.distributed.device_mesh import DeviceMesh
        from torch.distributed.tensor import placement_types as pt

        conv = []
        for p in self.placements:
            if isinstance(p, Shard):
                conv.append(pt.Shard(p.dim))
            elif isinstance(p, Replicate):
                conv.append(pt.Replicate())
            else:
                conv.append(pt.Partial())
        return DeviceMesh(device_type, torch.from_numpy(self.mesh.copy())), conv


def _world(world_size: int | None) -> int:
    if world_size is not None:
        return int(world_size)
    import torch.distributed as dist

    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _check(world: int, rep: int) -> int:
    if rep <= 0 or world % rep != 0:
        raise RuntimeError(f"World size {world} not divisible by replication factor {rep}")
    return world // rep


def one_dimensional_partitioning(dimension: str = "row", replication_factor: int = 1,
                                 world_size: int | None = None) -> Partitioning:
    dimension = normalize_partition(dimension)
    if dimension == "block":
        raise RuntimeError("dimension block is not valid for one_dimensional_partitioning")
    shard = Shard(0 if dimension == "row" else 1)
    world = _world(world_size)
    per = _check(world, replication_factor)
    ranks = np.arange(world, dtype=np.int64)
    if replication_factor == 1:
        return Partitioning(ranks, (shard,))
    if replication_factor == world:
        return Partitioning(ranks, (Replicate(),))
    return Partitioning(ranks.reshape(replication_factor, per), (Replicate(), shard))


def row_partitioning(replication_factor: int = 1, world_size: int | None = None) -> Partitioning:
    return one_dimensional_partitioning("row", replication_factor, world_size)


def column_partitioning(replication_factor: int = 1, world_size: int | None = None) -> Partitioning:
    return one_dimensional_partitioning("column", replication_factor, world_size)


def two_dimensional_partitioning(process_grid: tuple[int, int] | None = None, replication_factor: int = 1,
                                 world_size: int | None = None) -> Partitioning:
    world = _world(world_size)
    per = _check(world, replication_factor)
    if process_grid is None:
        process_grid = closest_factors(per)
    if process_grid[0] * process_grid[1] != per:
        raise RuntimeError(f"process grid {process_grid} does not cover {per} ranks per replica")
    ranks = np.arange(world, dtype=np.int64)
    if replication_factor == 1:
        return Partitioning(ranks.reshape(process_grid), (Shard(0), Shard(1)))
    if replication_factor == world:
        return Partitioning(ranks, (Replicate(),))
    return Partitioning(ranks.reshape(replication_factor, *process_grid), (Replicate(), Shard(0), Shard(1)))


def get_partitioning(partition: str, replication_factor: int = 1, world_size: int | None = None) -> Partitioning:
    partition = normalize_partition(partition)
    if partition == "block":
        return two_dimensional_partitioning(replication_factor=replication_factor, world_size=world_size)
    return one_dimensional_partitioning(partition, replication_factor, world_size)


def materialized_placements(placements) -> tuple[bool, list]:
    """Replace every ``Partial`` by a shard on the matrix dimension that is not yet
    sharded (a reduce-scatter when redistributed).  Works on this package's
    placements and on torch's; the returned list uses the input's classes."""
    free = {0, 1}
    has_partial = False
    for p in placements:
        name = type(p).__name__
        if name in ("Partial", "_Partial"):
            has_partial = True
        elif name in ("Shard", "_StridedShard"):
            free.discard(int(p.dim))
    if not has_partial:
        return False, list(placements)
    if not free:
        raise ValueError("cannot materialize Partial: both matrix dimensions are already sharded")
    dim = min(free)
    shard_cls = None
    for p in placements:
        if type(p).__name__ in ("Shard", "_StridedShard"):
            shard_cls = type(p)
    out = []
    for p in placements:
        if type(p).__name__ in ("Partial", "_Partial"):
            if isinstance(p, Partial) or shard_cls is Shard:
                out.append(Shard(dim))
            else:
                from torch.distributed.tensor import placement_types as pt

                out.append(pt.Shard(dim))
        else:
            out.append(p)
    return True, out
