"""Partitioned matrices whose shards live in symmetric memory.

:class:`DistMatrix` couples a :class:`~.tiles.Layout` with one symmetric allocation
holding every rank's tile.  All tiles use the same padded geometry (maximal tile
shape, row pitch rounded up to 64 elements), so a peer's tile is at the same
offset in the peer's copy and every row starts on a 128-byte boundary - the
condition under which the kernels can use TMA and 16-byte vector accesses.

``DistMatrix.to_dtensor()`` wraps the local shard in a stock ``DTensor`` (for use
with the ``addmm`` hook); the registry maps such DTensors back to their
``DistMatrix``.  In the reference this role is played by a patched PyTorch whose
DTensors allocate from NVSHMEM (``DTensor.nvshmem_base()``, dtensor_utils.py:360,535).
"""
from __future__ import annotations

import weakref
from typing import Any

import torch

from . import tiles as T
from .partition import Partitioning, get_partitioning
from .symm import World

_LD_ALIGN = 64


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


# Local data pointer -> matrix, weakly: a matrix that nobody references any more drops out by itself.
_registry: "weakref.WeakValueDictionary[int, DistMatrix]" = weakref.WeakValueDictionary()


class DistMatrix:
    def __init__(self, world: World, shape: tuple[int, int], partitioning: Partitioning | T.Layout, dtype: torch.dtype):
        self.world = world
        self.layout = partitioning if isinstance(partitioning, T.Layout) else partitioning.layout(tuple(shape))
        if self.layout.shape != (int(shape[0]), int(shape[1])):
            raise ValueError("layout shape does not match the matrix shape")
        if sorted(self.layout.ranks()) != list(range(world.size)):
            raise ValueError("the mesh must contain every rank of the world exactly once")
        self.dtype = dtype
        self.itemsize = torch.empty(0, dtype=dtype).element_size()
        self.tile_rows, self.tile_cols = T.tile_shape(self.layout)
        self.ld = _round_up(max(self.tile_cols, 1), _LD_ALIGN)
        self.nbytes = max(self.tile_rows, 1) * self.ld * self.itemsize
        self.buffer = world.alloc(self.nbytes)
        self.coord = T.local_tile_coord(self.layout, world.rank)
        self._dtensor = None
        _registry[self.buffer.ptr(world.rank)] = self

    # ------------------------------------------------------------------ properties
    @property
    def shape(self) -> tuple[int, int]:
        return self.layout.shape

    @property
    def ndim(self) -> int:
        return 2

    @property
    def device(self) -> torch.device:
        return self.world.device

    @property
    def rank(self) -> int:
        return self.world.rank

    def local_shape(self, rank: int | None = None) -> tuple[int, int]:
        coord = self.coord if rank is None else T.local_tile_coord(self.layout, rank)
        return T.tile_shape(self.layout, coord)

    def _padded(self, rank: int) -> torch.Tensor | None:
        raw = self.buffer.tensor(rank)
        if raw is None:
            return None
        return raw[: self.nbytes].view(self.dtype).view(max(self.tile_rows, 1), self.ld)

    @property
    def local_padded(self) -> torch.Tensor:
        """This rank's tile storage: ``[tile_rows, ld]`` including padding."""
        t = self._padded(self.rank)
        assert t is not None
        return t

    @property
    def local(self) -> torch.Tensor:
        """This rank's tile, clipped to its true shape (a strided view, no copy)."""
        rows, cols = self.local_shape()
        return self.local_padded[:rows, :cols]

    def to_local(self) -> torch.Tensor:
        return self.local

    def peer_tile(self, rank: int) -> torch.Tensor | None:
        """Rank ``rank``'s tile as a tensor when this world can express peer memory as tensors."""
        t = self._padded(rank)
        if t is None:
            return None
        rows, cols = self.local_shape(rank)
        return t[:rows, :cols]

    def tile_ptr(self, rank: int) -> int:
        """Address (in this process) of element (0, 0) of ``rank``'s tile."""
        return self.buffer.ptr(rank)

    def is_remote(self, rank: int) -> bool:
        return rank != self.rank

    # ------------------------------------------------------------------ data movement (setup paths)
    def zero_(self) -> "DistMatrix":
        self.local_padded.zero_()
        return self

    def fill_from_full(self, full: torch.Tensor) -> "DistMatrix":
        """Copy this rank's shard out of a full matrix every rank holds (no communication)."""
        if tuple(full.shape) != self.shape:
            raise ValueError(f"expected a full tensor of shape {self.shape}, got {tuple(full.shape)}")
        b = T.tile_bounds(self.layout, self.coord)
        self.local.copy_(full[b.rows.as_slice(), b.cols.as_slice()].to(device=self.device, dtype=self.dtype))
        return self

    def full_tensor(self, replica: int = 0) -> torch.Tensor:
        """Assemble the full matrix from replica ``replica`` on every rank (collective)."""
        from . import runtime

        return runtime.gather_full(self, replica=replica)

    def to_dtensor(self):
        """A stock DTensor over the local shard (needs an initialised process group)."""
        if self._dtensor is None:
            from torch.distributed.device_mesh import DeviceMesh
            from torch.distributed.tensor import DTensor, placement_types as pt

            mesh = DeviceMesh(self.device.type, torch.from_numpy(self.layout.mesh.copy()))
            conv = []
            for p in self.layout.placements:
                conv.append(pt.Shard(p.dim) if isinstance(p, T.Shard) else
                            pt.Replicate() if isinstance(p, T.Replicate) else pt.Partial())
            dt = DTensor.from_local(self.local, mesh, conv, run_check=False, shape=torch.Size(self.shape),
                                    stride=(self.shape[1], 1))
            self._dtensor = dt
            dt._ug_matrix = self          # the DTensor keeps its matrix alive and names it directly
            _registry[dt._local_tensor.data_ptr()] = self
        return self._dtensor

    def free(self) -> None:
        """Release the symmetric allocation (collective: every rank frees the same matrix in the same order)."""
        from . import exec as _exec

        _exec.drop_programs_for(self.buffer.ptr(self.rank))
        _registry.pop(self.buffer.ptr(self.rank), None)
        if self._dtensor is not None:
            _registry.pop(self._dtensor._local_tensor.data_ptr(), None)
            self._dtensor._ug_matrix = None
            self._dtensor = None
        self.buffer.free()

    def __repr__(self) -> str:
        return (f"DistMatrix(shape={self.shape}, dtype={self.dtype}, grid={T.grid_shape(self.layout)}, "
                f"rep={T.replication_factor(self.layout)}, rank={self.rank}/{self.world.size}, ld={self.ld})")


def resolve(x: Any) -> DistMatrix:
    """Return the :class:`DistMatrix` behind ``x`` (itself, or a DTensor made by ``to_dtensor``)."""
    if isinstance(x, DistMatrix):
        return x
    hit = getattr(x, "_ug_matrix", None)
    if hit is None and hasattr(x, "_local_tensor"):     # e.g. a DTensor derived from the one to_dtensor() made
        hit = _registry.get(x._local_tensor.data_ptr())
    if hit is None:
        raise RuntimeError(
            "this DTensor is not backed by symmetric memory; create it with "
            "universal_gemm_b200.distribute_tensor(...) so that peers can address its shards")
    return hit


def empty(world: World, shape: tuple[int, int], partition: str | Partitioning, dtype: torch.dtype = torch.bfloat16,
          replication_factor: int = 1) -> DistMatrix:
    part = get_partitioning(partition, replication_factor, world.size) if isinstance(partition, str) else partition
    return DistMatrix(world, (int(shape[0]), int(shape[1])), part, dtype)


def zeros(world: World, shape: tuple[int, int], partition: str | Partitioning, dtype: torch.dtype = torch.float32,
          replication_factor: int = 1) -> DistMatrix:
    dm = empty(world, shape, partition, dtype, replication_factor).zero_()
    # Collective set-up call: nobody may write into a peer's shard before that peer has cleared it.
    if world.is_cuda:
        torch.cuda.synchronize(world.device)
    world.barrier()
    return dm


def distribute_tensor(full: torch.Tensor, world: World, partition: str | Partitioning, replication_factor: int = 1,
                      dtype: torch.dtype | None = None, src_rank: int | None = None) -> DistMatrix:
    """Scatter a full matrix into symmetric shards.

    With ``src_rank=None`` every rank is expected to hold the same ``full`` tensor and
    just cuts out its own shard.  With ``src_rank=r`` only rank r's data is used: it is
    broadcast over the world's process group first (what ``distribute_tensor`` of torch
    does from mesh rank 0, dtensor_example.py:106-108 in the reference).
    """
    dm = empty(world, tuple(full.shape), partition, dtype or full.dtype, replication_factor)
    if src_rank is not None and world.size > 1 and not world.emulated:
        import torch.distributed as dist

        buf = full.to(world.device).contiguous()
        dist.broadcast(buf, src=src_rank, group=getattr(world, "group", None))
        full = buf
    dm.local_padded.zero_()
    dm.fill_from_full(full)
    if world.is_cuda:
        torch.cuda.synchronize(world.device)
    world.barrier()
    return dm
