"""Plan construction for the stationary distributed GEMM algorithms.

A plan is the list of tile-level multiply operations

    C.tile(c_idx)[c_slice] += A.tile(a_idx)[a_slice] @ B.tile(b_idx)[b_slice]

(slices in tile-local coordinates) that one rank executes.  Two algorithms:

* **Stationary-C**: the owner of a C tile computes it, pulling the A and B tiles
  it needs.  With replication factor r on C, replica q only covers a contiguous
  1/r chunk of K (rotated per tile), and the replicas are summed afterwards.
* **Stationary-B**: the owner of a B tile multiplies it with every A slice that
  meets it and adds the partial products into the owners of C.  With replication
  on B, replica q covers a 1/r chunk of M.

Both walk their free dimension (K resp. M) starting at a block that depends on
the tile coordinates, so that at any moment different ranks talk to different
peers.  The op lists (contents *and* order) equal the reference's
stationary_c_plan.py:182-283 and stationary_b_plan.py:153-255; the implementation
here is one generic walker instead of two copies.

:func:`group_ops` turns an op list into output *regions* with their K segments,
which is the unit the fused kernel executes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Sequence

from .tiles import (
    Layout,
    Slice1D,
    Slice2D,
    as_layout,
    grid_shape,
    intersect_1d,
    intersect_2d,
    matrix_numel,
    my_replica,
    overlapping_tiles,
    replication_factor,
    subtract_offset,
    tile_bounds,
    tile_offset,
    tile_rank,
    _current_rank,
)

STATIONARY_METHODS = ("auto", "stationary_c", "stationary_b", "min_traffic")


@dataclass(frozen=True)
class MultiplyOp:
    a_idx: tuple[int, int]
    b_idx: tuple[int, int]
    c_idx: tuple[int, int]
    a_slice: Slice2D
    b_slice: Slice2D
    c_slice: Slice2D


# ----------------------------------------------------------------------------- formatting
def _fmt(s: Slice2D) -> str:
    return f"[{s.rows.start}:{s.rows.stop}, {s.cols.start}:{s.cols.stop}]"


def format_op(op: MultiplyOp) -> str:
    return (f"C.tile{op.c_idx}{_fmt(op.c_slice)} += A.tile{op.a_idx}{_fmt(op.a_slice)} * "
            f"B.tile{op.b_idx}{_fmt(op.b_slice)}")


def _format_plan(title: str, ops: Sequence[MultiplyOp], rank: int | None) -> str:
    head = f"{title} (rank={rank})" if rank is not None else title
    lines = [f"{head}: {len(ops)} ops"]
    lines += [f"  {i:04d}: {format_op(op)}" for i, op in enumerate(ops)]
    return "\n".join(lines)


def format_plan(ops: Sequence[MultiplyOp], rank: int | None = None) -> str:
    return _format_plan("Stationary-C plan", ops, rank)


def format_stationary_b_op(op: MultiplyOp) -> str:
    return format_op(op)


def format_stationary_b_plan(ops: Sequence[MultiplyOp], rank: int | None = None) -> str:
    return _format_plan("Stationary-B plan", ops, rank)


# ----------------------------------------------------------------------------- helpers
def _check_shapes(a: Layout, b: Layout, c: Layout, who: str) -> None:
    if a.shape[1] != b.shape[0] or c.shape[0] != a.shape[0] or c.shape[1] != b.shape[1]:
        raise ValueError(f"{who}: shape mismatch: a={a.shape}, b={b.shape}, c={c.shape}")


def _block_starts(extent: int, *edges: Sequence[Slice1D]) -> list[int]:
    """Sorted starts of the blocks cut by all tile edges of two tilings of one dimension."""
    points = {0, extent}
    for group in edges:
        for s in group:
            points.add(s.start)
            points.add(s.stop)
    pts = sorted(points)
    return [pts[i] for i in range(len(pts) - 1) if pts[i] < pts[i + 1]]


def _replica_ranges(extent: int, rep: int, replica: int, turn: int, starts: list[int]) -> list[Slice1D]:
    """Replica ``replica``'s 1/rep chunk of ``[0, extent)``, rotated on the ring by the
    ``turn``-th block start; the result may wrap and split in two."""
    if extent <= 0:
        return []
    if rep <= 0 or not 0 <= replica < rep:
        raise ValueError(f"replica {replica} out of range for replication factor {rep}")
    chunk = -(-extent // rep)
    lo = chunk * replica
    length = max(min(extent, lo + chunk) - lo, 0)
    if length == 0:
        return []
    shift = (starts[turn % len(starts)] if starts else 0) % extent
    begin = (lo + shift) % extent
    end = begin + length
    if end <= extent:
        return [Slice1D(begin, end)]
    return [Slice1D(begin, extent), Slice1D(0, end - extent)]


def _rotate(items: list, by: int) -> list:
    if not items:
        return items
    k = by % len(items)
    return items[k:] + items[:k]


_plan_cache: dict[tuple, list[MultiplyOp]] = {}


def clear_plan_cache() -> None:
    _plan_cache.clear()


def clear_stationary_c_plan_cache() -> None:
    for k in [k for k in _plan_cache if k[0] == "c"]:
        del _plan_cache[k]


def clear_stationary_b_plan_cache() -> None:
    for k in [k for k in _plan_cache if k[0] == "b"]:
        del _plan_cache[k]


def _build(kind: str, a: Any, b: Any, c: Any, local_only: bool, rank: int | None) -> list[MultiplyOp]:
    la, lb, lc = as_layout(a), as_layout(b), as_layout(c)
    _check_shapes(la, lb, lc, f"build_stationary_{kind}_ops")
    me = _current_rank(rank)
    key = (kind, local_only, me, la.key(), lb.key(), lc.key())
    hit = _plan_cache.get(key)
    if hit is not None:
        return hit

    m_ext, k_ext = la.shape
    if kind == "c":
        anchor = lc
        extent = k_ext
        starts = _block_starts(k_ext,
                               [tile_bounds(la, (0, j)).cols for j in range(grid_shape(la)[1])],
                               [tile_bounds(lb, (i, 0)).rows for i in range(grid_shape(lb)[0])])
    else:
        anchor = lb
        extent = m_ext
        starts = _block_starts(m_ext,
                               [tile_bounds(la, (i, 0)).rows for i in range(grid_shape(la)[0])],
                               [tile_bounds(lc, (i, 0)).rows for i in range(grid_shape(lc)[0])])
    rep = replication_factor(anchor)
    replica = my_replica(anchor, me)

    ops: list[MultiplyOp] = []
    g_rows, g_cols = grid_shape(anchor)
    for p in range(g_rows):
        for q in range(g_cols):
            s_idx = (p, q)
            if local_only and tile_rank(anchor, s_idx, rank=me) != me:
                continue
            s_bounds = tile_bounds(anchor, s_idx)
            groups: dict[tuple[int, int], list[MultiplyOp]] = {}
            for rng in _replica_ranges(extent, rep, replica, p + q, starts):
                # Stationary-C walks K next to the C tile's rows; Stationary-B walks M next to
                # the B tile's rows (= K range).
                a_region = Slice2D(s_bounds.rows, rng) if kind == "c" else Slice2D(rng, s_bounds.rows)
                for a_idx in overlapping_tiles(la, a_region):
                    a_bounds = intersect_2d(tile_bounds(la, a_idx), a_region)
                    if kind == "c":
                        third, third_region = lb, Slice2D(a_bounds.cols, s_bounds.cols)
                    else:
                        third, third_region = lc, Slice2D(a_bounds.rows, s_bounds.cols)
                    for t_idx in overlapping_tiles(third, third_region):
                        t_bounds = tile_bounds(third, t_idx)
                        b_idx, b_bounds = (t_idx, t_bounds) if kind == "c" else (s_idx, s_bounds)
                        c_idx, c_bounds = (s_idx, s_bounds) if kind == "c" else (t_idx, t_bounds)
                        mb = intersect_1d(a_bounds.rows, c_bounds.rows)
                        kb = intersect_1d(a_bounds.cols, b_bounds.rows)
                        nb = intersect_1d(b_bounds.cols, c_bounds.cols)
                        if mb.size == 0 or kb.size == 0 or nb.size == 0:
                            continue
                        gkey = (kb.start, kb.stop) if kind == "c" else (mb.start, mb.stop)
                        groups.setdefault(gkey, []).append(MultiplyOp(
                            a_idx=a_idx, b_idx=b_idx, c_idx=c_idx,
                            a_slice=subtract_offset(Slice2D(mb, kb), tile_offset(la, a_idx)),
                            b_slice=subtract_offset(Slice2D(kb, nb), tile_offset(lb, b_idx)),
                            c_slice=subtract_offset(Slice2D(mb, nb), tile_offset(lc, c_idx)),
                        ))
            for members in groups.values():          # dicts keep first-seen order
                ops.extend(_rotate(members, p + q))
    _plan_cache[key] = ops
    return ops


def build_stationary_c_ops(a: Any, b: Any, c: Any, *, local_only: bool = True, rank: int | None = None) -> list[MultiplyOp]:
    """Op list of ``rank`` for Stationary-C (every op is anchored on a C tile it owns)."""
    return _build("c", a, b, c, local_only, rank)


def build_stationary_b_ops(a: Any, b: Any, c: Any, *, local_only: bool = True, rank: int | None = None) -> list[MultiplyOp]:
    """Op list of ``rank`` for Stationary-B (every op is anchored on a B tile it owns)."""
    return _build("b", a, b, c, local_only, rank)


def validate_op_shapes(op: MultiplyOp) -> None:
    if op.a_slice.shape[0] != op.c_slice.shape[0]:
        raise RuntimeError(f"Bad op (M mismatch): {op}")
    if op.a_slice.shape[1] != op.b_slice.shape[0]:
        raise RuntimeError(f"Bad op (K mismatch): {op}")
    if op.b_slice.shape[1] != op.c_slice.shape[1]:
        raise RuntimeError(f"Bad op (N mismatch): {op}")


def select_method(method: str, b: Any, c: Any, a: Any = None, *, in_bytes: int = 2, c_bytes: int = 4) -> str:
    """``auto`` picks Stationary-B when B has more elements than C (K > M), else Stationary-C
    (rule of the reference's dtensor_mm_handler.py:109-114).  ``min_traffic`` (not in the reference; needs ``a``)
    picks the method whose busiest rank moves fewer bytes over the links, see :func:`plan_traffic`; the reference's
    rule decides ties."""
    if method not in STATIONARY_METHODS:
        raise ValueError("stationary_method must be one of: auto, stationary_c, stationary_b, min_traffic")
    by_size = "stationary_b" if matrix_numel(b) > matrix_numel(c) else "stationary_c"
    if method == "auto":
        return by_size
    if method != "min_traffic":
        return method
    if a is None:
        raise ValueError("min_traffic needs the layout of A as well")
    cost = {m: max(plan_traffic(m, a, b, c, in_bytes=in_bytes, c_bytes=c_bytes)) for m in ("stationary_b", "stationary_c")}
    if cost["stationary_b"] == cost["stationary_c"]:
        return by_size
    return min(cost, key=cost.get)


def plan_traffic(method: str, a: Any, b: Any, c: Any, *, in_bytes: int = 2, c_bytes: int = 4) -> tuple[int, int]:
    """Bytes the busiest rank pulls in (operand slices of tiles it does not own) and pushes out (partial C for tiles
    it does not own) in one execution of ``method``: the link-side cost of a plan.  With a replicated C every replica
    pushes into replica 0 (the fused replica reduction)."""
    kind = "b" if method == "stationary_b" else "c"
    la, lb, lc = (as_layout(x) for x in (a, b, c))
    push_to_origin = replication_factor(lc) > 1
    worst_in = worst_out = 0
    for rank in lc.ranks():
        ops = _build(kind, la, lb, lc, True, rank)
        seen_a: set = set()
        seen_b: set = set()
        bytes_in = bytes_out = 0
        for op in ops:
            if tile_rank(la, op.a_idx, rank=rank) != rank and (op.a_idx, op.a_slice) not in seen_a:
                seen_a.add((op.a_idx, op.a_slice))
                bytes_in += op.a_slice.shape[0] * op.a_slice.shape[1] * in_bytes
            if tile_rank(lb, op.b_idx, rank=rank) != rank and (op.b_idx, op.b_slice) not in seen_b:
                seen_b.add((op.b_idx, op.b_slice))
                bytes_in += op.b_slice.shape[0] * op.b_slice.shape[1] * in_bytes
        for region in group_ops(ops):
            owner = tile_rank(lc, region.c_idx, replica=0 if push_to_origin else None, rank=rank)
            if owner != rank:
                bytes_out += region.c_slice.shape[0] * region.c_slice.shape[1] * c_bytes
        worst_in, worst_out = max(worst_in, bytes_in), max(worst_out, bytes_out)
    return worst_in, worst_out


# ----------------------------------------------------------------------------- regions
@dataclass
class Region:
    """One output rectangle of a plan and the ops (K segments) that add into it."""

    c_idx: tuple[int, int]
    c_slice: Slice2D
    ops: list[MultiplyOp]


def group_ops(ops: Sequence[MultiplyOp]) -> list[Region]:
    """Group a plan by output rectangle, keeping first-seen order of regions and the plan's
    op order inside each region.  The rectangles of one plan are pairwise disjoint or
    identical (they are cut by the row tiling of A and the column tiling of B), so a
    region can be accumulated over all its segments before C is touched once."""
    table: dict[tuple, Region] = {}
    for op in ops:
        validate_op_shapes(op)
        key = (op.c_idx, op.c_slice)
        reg = table.get(key)
        if reg is None:
            table[key] = reg = Region(op.c_idx, op.c_slice, [])
        reg.ops.append(op)
    regions = list(table.values())
    _assert_disjoint(regions)
    return regions


def _assert_disjoint(regions: Sequence[Region]) -> None:
    by_tile: dict[tuple[int, int], list[Slice2D]] = {}
    for r in regions:
        by_tile.setdefault(r.c_idx, []).append(r.c_slice)
    for slices in by_tile.values():
        if len(slices) > 64:      # quadratic check only on small plans; large ones share the construction
            continue
        for i in range(len(slices)):
            for j in range(i + 1, len(slices)):
                if not intersect_2d(slices[i], slices[j]).empty:
                    raise RuntimeError(f"plan regions overlap: {slices[i]} and {slices[j]}")
