"""One-sided tile operations on :class:`~.matrix.DistMatrix` (or DTensors made from one):
fetch a (possibly remote) tile, view a local tile, add a block into a (possibly
remote) tile, reduce replicas into the origin replica, gather a full matrix.

On a GPU the data moves with this package's kernels over peer pointers
(``ug_pull_2d`` / ``ug_accumulate_2d``); nothing blocks the host: futures carry CUDA
events and ``get()`` / ``wait()`` make the *current stream* wait.  On CPU worlds the
same calls act on shared-memory tensors.

API parity with the reference's dtensor_utils.py:30-115 and :332-629.  Differences,
all deliberate: ``get_tile`` can fetch just a sub-region (the reference always moves
the maximal tile), scratch tiles have tracked lifetimes (``release_tile`` is real),
and bf16 accumulation is supported next to fp32.
"""
from __future__ import annotations

import contextlib
import fcntl
from typing import Any

import torch

from . import tiles as T
from .matrix import DistMatrix, resolve
from .symm import ShmWorld, SymmHeap, World
from .tiles import Slice1D, Slice2D

_default_world: World | None = None
_heap: SymmHeap | None = None
_side_streams: dict[int, torch.cuda.Stream] = {}


def set_default_world(world: World | None) -> None:
    global _default_world
    _default_world = world


def default_world() -> World:
    if _default_world is None:
        raise RuntimeError("no default world: call universal_gemm_b200.init(...) or set_default_world(...)")
    return _default_world


# ----------------------------------------------------------------------------- scratch
def init_scratch(num_elements: int, dtype: torch.dtype, world: World | None = None) -> None:
    """Allocate (collectively) the symmetric scratch heap used for fetched tiles."""
    global _heap
    world = world or default_world()
    if _heap is None or _heap.dtype != dtype or _heap.world is not world or _heap.capacity < num_elements:
        if _heap is not None:
            _heap.close()
        _heap = SymmHeap(world, int(num_elements), dtype)
    _heap.reset()


def free_get_tile_scratch(dt: Any | None = None) -> None:
    """Free the scratch heap (collective)."""
    global _heap
    if _heap is None:
        return
    if dt is not None and resolve(dt).dtype != _heap.dtype:
        return
    _heap.close()
    _heap = None


def clear_peer_tensor_cache() -> None:
    """Kept for API compatibility: peer mappings belong to the symmetric buffers here."""
    return


def _scratch(dm: DistMatrix, shape: tuple[int, int]) -> torch.Tensor:
    if _heap is not None and _heap.dtype == dm.dtype and _heap.world is dm.world:
        return _heap.alloc(shape)
    return torch.empty(shape, dtype=dm.dtype, device=dm.device)


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _side_streams.get(idx)
    if s is None:
        s = _side_streams[idx] = torch.cuda.Stream(device=device)
    return s


# ----------------------------------------------------------------------------- futures
class TileFuture:
    def __init__(self, view: torch.Tensor, event: "torch.cuda.Event | None" = None):
        self._view = view
        self._event = event

    def get(self) -> torch.Tensor:
        if self._event is not None:
            torch.cuda.current_stream(self._view.device).wait_event(self._event)
            self._event = None
        return self._view


class AccumulateFuture:
    def __init__(self, event: "torch.cuda.Event | None" = None):
        self._event = event

    def wait(self) -> None:
        if self._event is not None:
            self._event.synchronize()
            self._event = None


class ReduceReplicasFuture:
    def __init__(self, futures: list[AccumulateFuture]):
        self._futures = futures

    def wait(self) -> None:
        for f in self._futures:
            f.wait()


# ----------------------------------------------------------------------------- tiles
def _check_coord(dm: DistMatrix, coord: tuple[int, int]) -> None:
    gr, gc = T.grid_shape(dm.layout)
    if not (0 <= coord[0] < gr and 0 <= coord[1] < gc):
        raise ValueError(f"tile coord {tuple(coord)} out of range for grid {(gr, gc)}")


def tile(dt: Any, coord: tuple[int, int], replica: int | None = None) -> torch.Tensor:
    """Local view of a tile this rank owns; raises when the tile is remote."""
    dm = resolve(dt)
    _check_coord(dm, coord)
    owner = T.tile_rank(dm.layout, coord, replica=replica, rank=dm.rank)
    if owner != dm.rank:
        raise RuntimeError(f"tile {coord} is owned by rank {owner}, current rank is {dm.rank}")
    rows, cols = T.tile_shape(dm.layout, coord)
    return dm.local_padded[:rows, :cols]


def release_tile(t: torch.Tensor) -> None:
    """End the life of a scratch tile so that the heap may reuse its memory."""
    if _heap is not None:
        base = getattr(t, "_scratch_owner", t)
        _heap.release(base)


def _fetch(dm: DistMatrix, coord: tuple[int, int], replica: int | None, region: Slice2D | None,
           side_stream: bool) -> TileFuture:
    _check_coord(dm, coord)
    rows, cols = T.tile_shape(dm.layout, coord)
    if region is None:
        region = Slice2D(Slice1D(0, rows), Slice1D(0, cols))
    if region.rows.stop > rows or region.cols.stop > cols:
        raise ValueError(f"region {region} out of bounds for tile shape {(rows, cols)}")
    owner = T.tile_rank(dm.layout, coord, replica=replica, rank=dm.rank)
    if owner == dm.rank:
        return TileFuture(dm.local_padded[region.rows.as_slice(), region.cols.as_slice()])
    r, c = region.shape
    out = _scratch(dm, (r, c))
    peer = dm.peer_tile(owner)
    if not dm.world.is_cuda:
        out.copy_(peer[region.rows.as_slice(), region.cols.as_slice()])
        return TileFuture(out)
    from ..ops.device import DeviceState

    state = DeviceState.get(dm.device)
    src = dm.tile_ptr(owner) + (region.rows.start * dm.ld + region.cols.start) * dm.itemsize
    args = (out.data_ptr(), out.stride(0) * dm.itemsize, src, dm.ld * dm.itemsize, r, c * dm.itemsize, dm.itemsize)
    if not side_stream:
        state.pull_2d(*args)
        return TileFuture(out)
    cur = torch.cuda.current_stream(dm.device)
    side = _side_stream(dm.device)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        state.pull_2d(*args)
        ev = torch.cuda.Event()
        ev.record(side)
    return TileFuture(out, ev)


def get_tile(dt: Any, coord: tuple[int, int], replica: int | None = None, region: Slice2D | None = None) -> torch.Tensor:
    """Copy a (possibly remote) tile - or only ``region`` of it - into local memory.

    Stream-ordered on the GPU: the returned tensor is valid for work queued on the
    current stream; the host is not blocked."""
    return _fetch(resolve(dt), coord, replica, region, side_stream=False).get()


def get_tile_async(dt: Any, coord: tuple[int, int], replica: int | None = None,
                   region: Slice2D | None = None) -> TileFuture:
    """Start fetching a tile on a side stream; ``.get()`` orders the current stream after it."""
    return _fetch(resolve(dt), coord, replica, region, side_stream=True)


@contextlib.contextmanager
def _owner_lock(world: World, owner: int):
    if isinstance(world, ShmWorld):
        with open(world.lock_path(owner), "a+") as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                yield
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)
    else:
        yield


def accumulate_tile(dt: Any, coord: tuple[int, int], view: torch.Tensor, *, slice_: Slice2D | None = None,
                    replica: int | None = None) -> AccumulateFuture:
    """``dt.tile(coord)[slice_] += view``, one-sided: the owner does not take part."""
    dm = resolve(dt)
    if view.ndim != 2:
        raise ValueError(f"accumulate_tile expects a rank-2 view, got ndim={view.ndim}")
    if view.dtype != dm.dtype:
        raise RuntimeError(f"accumulate_tile dtype mismatch: view={view.dtype}, dt={dm.dtype}")
    _check_coord(dm, coord)
    rows, cols = T.tile_shape(dm.layout, coord)
    if slice_ is None:
        slice_ = Slice2D(Slice1D(0, rows), Slice1D(0, cols))
    if slice_.rows.stop > rows or slice_.cols.stop > cols:
        raise ValueError(f"slice {slice_} out of bounds for tile shape {(rows, cols)}")
    if tuple(view.shape) != slice_.shape:
        raise ValueError(f"view shape {tuple(view.shape)} does not match slice shape {slice_.shape}")
    owner = T.tile_rank(dm.layout, coord, replica=replica, rank=dm.rank)
    if not dm.world.is_cuda:
        target = dm.peer_tile(owner)
        with _owner_lock(dm.world, owner):
            target[slice_.rows.as_slice(), slice_.cols.as_slice()] += view
        return AccumulateFuture()
    if view.stride(1) != 1:
        view = view.contiguous()
    from ..ops.device import DeviceState, torch_dtype_code

    state = DeviceState.get(dm.device)
    dst = dm.tile_ptr(owner) + (slice_.rows.start * dm.ld + slice_.cols.start) * dm.itemsize
    state.accumulate_2d(dst, dm.ld, view.data_ptr(), view.stride(0), view.shape[0], view.shape[1],
                        torch_dtype_code(dm.dtype))
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(dm.device))
    return AccumulateFuture(ev)


def reduce_replicas_async(dt: Any, *, origin_replica: int = 0) -> ReduceReplicasFuture:
    """Every non-origin replica adds its tiles into the origin replica (collective by
    convention; the result is valid in the origin replica only)."""
    dm = resolve(dt)
    rep = T.replication_factor(dm.layout)
    if rep <= 1:
        return ReduceReplicasFuture([])
    if not 0 <= origin_replica < rep:
        raise ValueError(f"origin_replica {origin_replica} out of range for replication_factor {rep}")
    futures = []
    mine = T.my_replica(dm.layout, dm.rank)
    if mine != origin_replica:
        for coord in T.owned_tiles(dm.layout, dm.rank, replica=mine):
            futures.append(accumulate_tile(dm, coord, tile(dm, coord, replica=mine), replica=origin_replica))
    return ReduceReplicasFuture(futures)


def reduce_replicas(dt: Any, *, origin_replica: int = 0) -> None:
    reduce_replicas_async(dt, origin_replica=origin_replica).wait()


def gather_full(dm: DistMatrix, replica: int = 0) -> torch.Tensor:
    """Full matrix assembled from ``replica``'s tiles, on every rank (collective: peers must
    have finished writing; callers synchronise before)."""
    dm = resolve(dm)
    out = torch.empty(dm.shape, dtype=dm.dtype, device=dm.device)
    gr, gc = T.grid_shape(dm.layout)
    for i in range(gr):
        for j in range(gc):
            b = T.tile_bounds(dm.layout, (i, j))
            if b.empty:
                continue
            owner = T.tile_rank(dm.layout, (i, j), replica=replica, rank=dm.rank)
            dst = out[b.rows.as_slice(), b.cols.as_slice()]
            peer = dm.peer_tile(owner)
            if peer is not None:
                dst.copy_(peer)
            else:
                from ..ops.device import DeviceState

                r, c = b.shape
                DeviceState.get(dm.device).pull_2d(dst.data_ptr(), out.stride(0) * dm.itemsize, dm.tile_ptr(owner),
                                                   dm.ld * dm.itemsize, r, c * dm.itemsize, dm.itemsize)
    return out


# ----------------------------------------------------------------------------- put + signal
def put_tile(dt: Any, coord: tuple[int, int], view: torch.Tensor, *, slice_: Slice2D | None = None,
             replica: int | None = None) -> None:
    """``dt.tile(coord)[slice_] = view``, one-sided (the counterpart of ``get_tile``; stream-ordered on the GPU)."""
    dm = resolve(dt)
    _check_coord(dm, coord)
    rows, cols = T.tile_shape(dm.layout, coord)
    if slice_ is None:
        slice_ = Slice2D(Slice1D(0, rows), Slice1D(0, cols))
    if slice_.rows.stop > rows or slice_.cols.stop > cols or tuple(view.shape) != slice_.shape:
        raise ValueError(f"view {tuple(view.shape)} / slice {slice_} do not fit tile shape {(rows, cols)}")
    if view.dtype != dm.dtype:
        raise RuntimeError(f"put_tile dtype mismatch: view={view.dtype}, dt={dm.dtype}")
    owner = T.tile_rank(dm.layout, coord, replica=replica, rank=dm.rank)
    if not dm.world.is_cuda:
        dm.peer_tile(owner)[slice_.rows.as_slice(), slice_.cols.as_slice()] = view
        return
    if view.stride(1) != 1:
        view = view.contiguous()
    from ..ops.device import DeviceState

    dst = dm.tile_ptr(owner) + (slice_.rows.start * dm.ld + slice_.cols.start) * dm.itemsize
    DeviceState.get(dm.device).pull_2d(dst, dm.ld * dm.itemsize, view.data_ptr(), view.stride(0) * dm.itemsize,
                                       view.shape[0], view.shape[1] * dm.itemsize, dm.itemsize)


class SignalPad:
    """``slots`` uint32 counters per rank in symmetric memory for put + signal protocols
    (the window ``signal`` / ``wait_signal`` pair of the reference's torchcomms experiments,
    torchcomms/put_02.py:43-55).  ``signal(peer, slot)`` is ordered after everything queued before it on the
    current stream; ``wait(slot, value)`` blocks the *stream*, not the host, and is bounded on the device."""

    def __init__(self, world: World, slots: int = 64, timeout_s: float = 10.0):
        self.world = world
        self.slots = int(slots)
        self.timeout_ns = int(timeout_s * 1e9)
        self.buffer = world.alloc(self.slots * 4)
        self.buffer.local.zero_()
        if world.is_cuda:
            torch.cuda.synchronize(world.device)
        world.barrier()

    def _counters(self, rank: int) -> torch.Tensor:
        return self.buffer.tensor(rank)[: self.slots * 4].view(torch.int32)

    def signal(self, peer: int, slot: int, value: int = 1) -> None:
        if not 0 <= slot < self.slots:
            raise ValueError(f"slot {slot} out of range")
        if not self.world.is_cuda:
            with _owner_lock(self.world, peer):
                self._counters(peer)[slot] += value
            return
        import ctypes

        from ..ops import native
        from ..ops.device import DeviceState

        st = DeviceState.get(self.world.device)
        native.check(native.lib().ug_signal_add(self.buffer.ptr(peer) + 4 * slot, value, ctypes.c_void_p(st.stream())),
                     "ug_signal_add")
        st.launches += 1

    def wait(self, slot: int, value: int) -> None:
        if not self.world.is_cuda:
            import time

            deadline = time.monotonic() + self.timeout_ns * 1e-9
            while int(self._counters(self.world.rank)[slot]) < value:
                if time.monotonic() > deadline:
                    raise TimeoutError(f"signal slot {slot} did not reach {value}")
                time.sleep(0.0005)
            return
        import ctypes

        from ..ops import native
        from ..ops.device import DeviceState

        st = DeviceState.get(self.world.device)
        native.check(native.lib().ug_signal_wait(self.buffer.ptr(self.world.rank) + 4 * slot, value, st.status_ptr,
                                                 self.timeout_ns, ctypes.c_void_p(st.stream())), "ug_signal_wait")
        st.launches += 1


# ----------------------------------------------------------------------------- redistribute
def redistribute(dt: Any, partition, replication_factor: int = 1, dtype: torch.dtype | None = None,
                 out: DistMatrix | None = None) -> DistMatrix:
    """Return a copy of the matrix in another partition (collective).

    One-sided: every rank pulls the pieces of the source tiles that overlap its new tile straight from their
    owners (``ug_pull_2d`` over peer pointers on the GPU), then converts the dtype locally if asked
    (``ug_convert_2d``).  This is the data movement the plain DTensor path performs with NCCL collectives
    (``redistribute`` in the reference's benchmark/matmul_bench_worker.py:96-105).  ``out``: an existing matrix in
    the target partition to fill instead of allocating one (allocation is a collective host operation)."""
    from .matrix import empty

    src = resolve(dt)
    world = src.world
    if out is None:
        out = empty(world, src.shape, partition, src.dtype if dtype is None else dtype, replication_factor)
    elif out.shape != src.shape or out.world is not world:
        raise ValueError("`out` must be a matrix of the same shape in the same world")
    staging = out if out.dtype == src.dtype else None
    mine = T.tile_bounds(out.layout, out.coord)
    tmp = None
    if staging is None:
        tmp = torch.zeros(out.local.shape, dtype=src.dtype, device=src.device)
    world.device_barrier()                       # the source is complete on every rank
    if not mine.empty:
        for coord in T.overlapping_tiles(src.layout, mine):
            sb = T.tile_bounds(src.layout, coord)
            inter = T.intersect_2d(sb, mine)
            if inter.empty:
                continue
            owner = T.tile_rank(src.layout, coord, rank=src.rank)
            local_src = T.subtract_offset(inter, (sb.rows.start, sb.cols.start))
            local_dst = T.subtract_offset(inter, (mine.rows.start, mine.cols.start))
            dst_t = (out.local if tmp is None else tmp)[local_dst.rows.as_slice(), local_dst.cols.as_slice()]
            if not world.is_cuda:
                dst_t.copy_(src.peer_tile(owner)[local_src.rows.as_slice(), local_src.cols.as_slice()])
                continue
            from ..ops.device import DeviceState

            r, c = inter.shape
            sptr = src.tile_ptr(owner) + (local_src.rows.start * src.ld + local_src.cols.start) * src.itemsize
            DeviceState.get(src.device).pull_2d(dst_t.data_ptr(), dst_t.stride(0) * src.itemsize, sptr,
                                                src.ld * src.itemsize, r, c * src.itemsize, src.itemsize)
    if tmp is not None:
        if world.is_cuda:
            from ..ops.device import DeviceState, torch_dtype_code

            rows, cols = tmp.shape
            if rows and cols:
                DeviceState.get(src.device).convert_2d(out.local.data_ptr(), out.ld, torch_dtype_code(out.dtype),
                                                       tmp.data_ptr(), tmp.stride(0), torch_dtype_code(src.dtype), rows, cols)
        else:
            out.local.copy_(tmp)
    world.device_barrier()                       # peers are done reading the source
    return out
