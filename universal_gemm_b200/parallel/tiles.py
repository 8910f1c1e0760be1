"""Tile geometry of partitioned matrices.

A distributed matrix is described by a :class:`Layout`: global shape, an n-d mesh
of ranks and one placement per mesh dimension (shard rows, shard columns,
replicate, partial).  One *tile* is one rank's shard; the tile grid has
``prod(mesh sizes sharding rows) x prod(mesh sizes sharding columns)`` tiles of
``ceil(dim / grid)`` rows / columns, the trailing ones clipped.

All functions accept a :class:`Layout`, any object with a ``layout`` attribute
(``DistMatrix``) or a ``torch.distributed.tensor.DTensor``; nothing here touches
a process group unless the caller leaves ``rank=None``.

Behaviour follows the reference's tile_bounds.py:71-136 and dtensor_utils.py:118-329
with one deliberate difference: a trailing tile that would start past the end of
the matrix (e.g. 9 rows over 8 ranks) is an *empty* tile here instead of an error.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Iterable, Sequence

import numpy as np


# ----------------------------------------------------------------------------- slices
@dataclass(frozen=True)
class Slice1D:
    """Half-open interval ``[start, stop)`` with ``0 <= start <= stop``."""

    start: int
    stop: int

    def __post_init__(self) -> None:
        if self.start < 0 or self.stop < self.start:
            raise ValueError(f"Slice1D needs 0 <= start <= stop, got [{self.start}, {self.stop})")

    @property
    def size(self) -> int:
        return self.stop - self.start

    def as_slice(self) -> slice:
        return slice(self.start, self.stop)

    def shifted(self, offset: int) -> "Slice1D":
        return Slice1D(self.start - offset, self.stop - offset)

    def __and__(self, other: "Slice1D") -> "Slice1D":
        return intersect_1d(self, other)


@dataclass(frozen=True)
class Slice2D:
    rows: Slice1D
    cols: Slice1D

    @property
    def row_slice(self) -> Slice1D:
        return self.rows

    @property
    def col_slice(self) -> Slice1D:
        return self.cols

    @property
    def shape(self) -> tuple[int, int]:
        return (self.rows.size, self.cols.size)

    @property
    def empty(self) -> bool:
        return self.rows.size == 0 or self.cols.size == 0

    def as_slices(self) -> tuple[slice, slice]:
        return (self.rows.as_slice(), self.cols.as_slice())

    def __and__(self, other: "Slice2D") -> "Slice2D":
        return intersect_2d(self, other)


def intersect_1d(a: Slice1D, b: Slice1D) -> Slice1D:
    lo = max(a.start, b.start)
    hi = max(min(a.stop, b.stop), lo)
    return Slice1D(lo, hi)


def intersect_2d(a: Slice2D, b: Slice2D) -> Slice2D:
    return Slice2D(intersect_1d(a.rows, b.rows), intersect_1d(a.cols, b.cols))


def subtract_offset(region: Slice2D, offset: tuple[int, int]) -> Slice2D:
    return Slice2D(region.rows.shifted(offset[0]), region.cols.shifted(offset[1]))


# ----------------------------------------------------------------------------- placements
@dataclass(frozen=True)
class Shard:
    dim: int

    def __post_init__(self) -> None:
        if self.dim not in (0, 1):
            raise ValueError(f"matrices can be sharded on dim 0 or 1, got {self.dim}")


@dataclass(frozen=True)
class Replicate:
    pass


@dataclass(frozen=True)
class Partial:
    pass


Placement = Shard | Replicate | Partial


def _coerce_placement(p: Any) -> Placement:
    if isinstance(p, (Shard, Replicate, Partial)):
        return p
    name = type(p).__name__
    if name in ("Shard", "_StridedShard"):
        return Shard(int(p.dim))
    if name == "Replicate":
        return Replicate()
    if name in ("Partial", "_Partial"):
        return Partial()
    raise ValueError(f"unsupported placement {p!r}")


# ----------------------------------------------------------------------------- layout
class Layout:
    """Shape + mesh + placements of one partitioned rank-2 matrix."""

    __slots__ = ("shape", "mesh", "placements", "_key")

    def __init__(self, shape: Sequence[int], mesh: Any, placements: Iterable[Any]):
        if len(shape) != 2:
            raise ValueError(f"expected a rank-2 shape, got {tuple(shape)}")
        self.shape = (int(shape[0]), int(shape[1]))
        arr = np.asarray(mesh, dtype=np.int64)
        if arr.ndim == 0:
            arr = arr.reshape(1)
        self.mesh = arr
        self.placements = tuple(_coerce_placement(p) for p in placements)
        if len(self.placements) != arr.ndim:
            raise ValueError(f"{arr.ndim}-d mesh needs {arr.ndim} placements, got {len(self.placements)}")
        self._key = (self.shape, arr.shape, tuple(int(v) for v in arr.reshape(-1)), self.placements)

    @classmethod
    def from_dtensor(cls, dt: Any) -> "Layout":
        if dt.ndim != 2:
            raise ValueError(f"expected a 2D DTensor, got ndim={dt.ndim}")
        return cls(tuple(dt.shape), dt.device_mesh.mesh.cpu().numpy(), dt.placements)

    def key(self) -> tuple:
        return self._key

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Layout) and self._key == other._key

    def __hash__(self) -> int:
        return hash(self._key)

    def __repr__(self) -> str:
        return f"Layout(shape={self.shape}, mesh={self.mesh.tolist()}, placements={self.placements})"

    # mesh dimensions by role
    def _dims(self, kind: str) -> list[int]:
        out = []
        for d, p in enumerate(self.placements):
            if kind == "rep" and isinstance(p, Replicate):
                out.append(d)
            elif kind == "row" and isinstance(p, Shard) and p.dim == 0:
                out.append(d)
            elif kind == "col" and isinstance(p, Shard) and p.dim == 1:
                out.append(d)
        return out

    def ranks(self) -> list[int]:
        return [int(v) for v in self.mesh.reshape(-1)]

    def coordinate_of(self, rank: int) -> tuple[int, ...] | None:
        hit = np.argwhere(self.mesh == rank)
        if hit.shape[0] == 0:
            return None
        return tuple(int(v) for v in hit[0])


def as_layout(x: Any) -> Layout:
    if isinstance(x, Layout):
        return x
    lay = getattr(x, "layout", None)
    if isinstance(lay, Layout):
        return lay
    if hasattr(x, "device_mesh") and hasattr(x, "placements"):
        return Layout.from_dtensor(x)
    raise TypeError(f"cannot interpret {type(x).__name__} as a partitioned matrix")


def _current_rank(rank: int | None) -> int:
    if rank is not None:
        return int(rank)
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _prod(sizes: Iterable[int]) -> int:
    out = 1
    for s in sizes:
        out *= int(s)
    return out


def _flatten(coords: Sequence[int], sizes: Sequence[int]) -> int:
    idx = 0
    for c, s in zip(coords, sizes):
        if not 0 <= c < s:
            raise ValueError(f"coordinate {c} out of range for size {s}")
        idx = idx * s + c
    return idx


def _unflatten(index: int, sizes: Sequence[int]) -> list[int]:
    out = []
    for s in reversed(sizes):
        out.append(index % s)
        index //= s
    return out[::-1]


# ----------------------------------------------------------------------------- geometry API
def grid_shape(x: Any) -> tuple[int, int]:
    """Tile grid ``(rows, cols)``; replication and partial placements do not add tiles."""
    lay = as_layout(x)
    return (_prod(lay.mesh.shape[d] for d in lay._dims("row")), _prod(lay.mesh.shape[d] for d in lay._dims("col")))


def matrix_numel(x: Any) -> int:
    lay = as_layout(x)
    return lay.shape[0] * lay.shape[1]


def replication_factor(x: Any) -> int:
    lay = as_layout(x)
    return _prod(lay.mesh.shape[d] for d in lay._dims("rep"))


def _max_tile(lay: Layout) -> tuple[int, int]:
    gr, gc = grid_shape(lay)
    return (-(-lay.shape[0] // gr), -(-lay.shape[1] // gc))


def _check_coord(lay: Layout, coord: tuple[int, int]) -> None:
    gr, gc = grid_shape(lay)
    if not (0 <= coord[0] < gr and 0 <= coord[1] < gc):
        raise ValueError(f"tile coord {tuple(coord)} out of range for grid {(gr, gc)}")


def tile_bounds(x: Any, coord: tuple[int, int]) -> Slice2D:
    """Global half-open bounds of tile ``coord`` (empty for tiles past the end)."""
    lay = as_layout(x)
    _check_coord(lay, coord)
    tr, tc = _max_tile(lay)
    m, n = lay.shape
    r0, c0 = min(coord[0] * tr, m), min(coord[1] * tc, n)
    return Slice2D(Slice1D(r0, min(r0 + tr, m)), Slice1D(c0, min(c0 + tc, n)))


def tile_shape(x: Any, coord: tuple[int, int] | None = None) -> tuple[int, int]:
    """Maximal tile shape, or the exact (clipped) shape of one tile."""
    lay = as_layout(x)
    if coord is None:
        return _max_tile(lay)
    return tile_bounds(lay, coord).shape


def tile_offset(x: Any, coord: tuple[int, int]) -> tuple[int, int]:
    b = tile_bounds(x, coord)
    return (b.rows.start, b.cols.start)


def overlapping_tiles(x: Any, region: Slice2D) -> list[tuple[int, int]]:
    """Coordinates (row-major) of the tiles that intersect a global region."""
    lay = as_layout(x)
    m, n = lay.shape
    r_lo, r_hi = max(0, region.rows.start), min(m, region.rows.stop)
    c_lo, c_hi = max(0, region.cols.start), min(n, region.cols.stop)
    if r_lo >= r_hi or c_lo >= c_hi:
        return []
    gr, gc = grid_shape(lay)
    tr, tc = _max_tile(lay)
    i0, i1 = min(gr - 1, r_lo // tr), min(gr - 1, (r_hi - 1) // tr)
    j0, j1 = min(gc - 1, c_lo // tc), min(gc - 1, (c_hi - 1) // tc)
    return [(i, j) for i in range(i0, i1 + 1) for j in range(j0, j1 + 1)]


def my_replica(x: Any, rank: int | None = None) -> int:
    """Index of the replica the rank belongs to (0 when the matrix is not replicated)."""
    lay = as_layout(x)
    rep = lay._dims("rep")
    if not rep:
        return 0
    coord = lay.coordinate_of(_current_rank(rank))
    if coord is None:
        raise RuntimeError("rank is not part of the matrix's device mesh")
    return _flatten([coord[d] for d in rep], [lay.mesh.shape[d] for d in rep])


def tile_rank(x: Any, coord: tuple[int, int], replica: int | None = None, rank: int | None = None) -> int:
    """Rank that stores tile ``coord`` of replica ``replica`` (default: the caller's replica)."""
    lay = as_layout(x)
    rep, rows, cols = lay._dims("rep"), lay._dims("row"), lay._dims("col")
    if replica is None:
        replica = my_replica(lay, rank)
    rep_sizes = [lay.mesh.shape[d] for d in rep]
    if not 0 <= replica < _prod(rep_sizes):
        raise ValueError(f"replica {replica} out of range for replication_factor {_prod(rep_sizes)}")
    full = [0] * lay.mesh.ndim
    for dims, index in ((rep, replica), (rows, coord[0]), (cols, coord[1])):
        if dims:
            for d, c in zip(dims, _unflatten(index, [lay.mesh.shape[d] for d in dims])):
                full[d] = c
    return int(lay.mesh[tuple(full)])


def owned_tiles(x: Any, rank: int | None = None, replica: int | None = None) -> list[tuple[int, int]]:
    """Tile coordinates stored by ``rank`` (in its own replica unless ``replica`` is given)."""
    lay = as_layout(x)
    r = _current_rank(rank)
    gr, gc = grid_shape(lay)
    return [(i, j) for i in range(gr) for j in range(gc) if tile_rank(lay, (i, j), replica=replica, rank=r) == r]


def local_tile_coord(x: Any, rank: int | None = None) -> tuple[int, int] | None:
    """The single tile a rank stores (every rank of the mesh stores exactly one)."""
    lay = as_layout(x)
    r = _current_rank(rank)
    coord = lay.coordinate_of(r)
    if coord is None:
        return None
    rows, cols = lay._dims("row"), lay._dims("col")
    i = _flatten([coord[d] for d in rows], [lay.mesh.shape[d] for d in rows]) if rows else 0
    j = _flatten([coord[d] for d in cols], [lay.mesh.shape[d] for d in cols]) if cols else 0
    return (i, j)
