"""Execution of Stationary-B / Stationary-C plans.

Two executors:

* **fused** (GPU, bf16 operands, or fp32 operands as three bf16 products): the plan is grouped into output regions, lowered
  once into the device tables of the persistent tcgen05 kernel (cached per matrix
  triple) and every call is ``signal barrier -> fused kernel -> signal barrier`` on
  the current stream.  Remote operand slices are pulled by the kernel's fetch
  warps, partial C tiles of Stationary-B (and of replicated runs) are pushed into
  the owner with ``red.add`` from the epilogue.  No host synchronisation.
* **tilewise** (any device / dtype): one ``get_tile`` + matmul + ``accumulate_tile``
  per op, the structure of the reference's executors
  (stationary_c_plan.py:295-355, stationary_b_plan.py:267-337).  It is the CPU
  path (and the path of dtype combinations the kernel does not take).

Signatures follow the reference's ``execute_stationary_{b,c}`` family
(stationary_c_plan.py:526-581, stationary_b_plan.py:567-623); arguments that tuned
its host loop (``max_outstanding_prefetch`` ...) are accepted and ignored by the
fused executor.
"""
from __future__ import annotations

import time
from typing import Any, Sequence

import torch

from ..utils import profile, trace
from . import plan as P
from . import runtime as R
from . import tiles as T
from .matrix import DistMatrix, resolve
from .plan import MultiplyOp

_program_cache: dict[tuple, Any] = {}


def clear_program_cache() -> None:
    _program_cache.clear()


def drop_programs_for(local_ptr: int) -> None:
    """Forget lowered programs that reference the symmetric buffer at ``local_ptr`` (called when a matrix is
    freed: a later allocation may get the same local address but different peer mappings)."""
    for key in [k for k in _program_cache if local_ptr in k[1:4]]:
        del _program_cache[key]


# ----------------------------------------------------------------------------- lowering
def _owner(dm: DistMatrix, idx: tuple[int, int], replica: int | None = None) -> int:
    return T.tile_rank(dm.layout, idx, replica=replica, rank=dm.rank)


def lower_plan(kind: str, a: DistMatrix, b: DistMatrix, c: DistMatrix, ops: Sequence[MultiplyOp], *,
               fuse_replica_reduce: bool = True, range_check: bool = True, beta: int = 1):
    """Lower an op list into a :class:`~universal_gemm_b200.ops.fused.FusedProgram`.

    ``beta=1`` is ``C += A @ B``.  ``beta=0`` is ``C = A @ B``: when every element of C has a single
    writer in the whole plan the epilogue stores (locally or into the peer) and C is neither read nor
    zeroed; otherwise the program keeps adding atomically and reports that C must be zeroed first.
    Returns ``(program, needs_zero)``."""
    from ..ops import native
    from ..ops.device import DeviceState, torch_dtype_code
    from ..ops.fused import FusedProgramBuilder, OperandSlice, TaskSpec

    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("the fused executor needs A and B of one dtype, bfloat16 or float32")
    split_f32 = a.dtype == torch.float32      # fp32 operands: three bf16 products per op (hi x hi + hi x lo + lo x hi)
    state = DeviceState.get(c.device)
    me = c.rank
    rep_c = T.replication_factor(c.layout)
    push_to_origin = fuse_replica_reduce and rep_c > 1
    # One writer per C element: Stationary-C without replicated C (the owner computes the whole K range),
    # Stationary-B whose B is not split along K (each B tile owner covers all of K for its rows / columns).
    # With a separate replica reduction (replicated C, nothing pushed to replica 0 by the epilogue) every replica
    # fills only its share of its own copy and the reduction then adds whole tiles, so all copies must start at zero.
    single_writer = ((kind == "c" and rep_c == 1) or (kind == "b" and T.grid_shape(b.layout)[0] == 1)) \
        and not (rep_c > 1 and not fuse_replica_reduce)
    needs_zero = beta == 0 and not single_writer
    # Skinny problems (few output tiles per rank, long K): every rank cuts K into parts that add into C atomically,
    # so that all SMs stream the operands.  Decided from the global shape alone, hence the same on every rank: all
    # of them then treat C as a multi-writer matrix (zeroed before the entry barrier when beta = 0).
    tiles_per_rank = -(-c.shape[0] // 256) * -(-c.shape[1] // 256) / max(c.world.size, 1)
    split_k = (c.dtype == torch.float32 and 4 * tiles_per_rank <= state.num_sms and a.shape[1] >= 32 * 64)
    if split_k:
        single_writer = False
        needs_zero = beta == 0

    buffers = (a.buffer, b.buffer, c.buffer)

    def check(ptr: int, nbytes: int, what: str) -> None:
        if not any(buf.contains(ptr, nbytes) for buf in buffers):
            raise RuntimeError(f"{what}: [{ptr:#x}, +{nbytes}) is outside the matrices' symmetric allocations")

    builder = FusedProgramBuilder(c.device, num_sms=state.num_sms,
                                  timeout_ns=getattr(c.world, "timeout_ns", 4_000_000_000),
                                  range_check=check if range_check else None, split_k=split_k)
    for region in P.group_ops(ops):
        c_owner = _owner(c, region.c_idx, replica=0 if push_to_origin else None)
        sl = region.c_slice
        c_ptr = c.tile_ptr(c_owner) + (sl.rows.start * c.ld + sl.cols.start) * c.itemsize
        m, n = sl.shape
        if range_check:
            check(c_ptr, ((m - 1) * c.ld + n) * c.itemsize, "C region")
        if kind == "c" and not push_to_origin:
            if c_owner != me:
                raise RuntimeError(f"Stationary-C expects local c_idx={region.c_idx}, owner={c_owner}, rank={me}")
            mode = native.C_ATOMIC if split_k else native.C_ADD
        else:
            mode = native.C_ATOMIC
        if beta == 0 and single_writer:
            mode = native.C_STORE
        segs = []
        for op in region.ops:
            ao, bo = _owner(a, op.a_idx), _owner(b, op.b_idx)
            if kind == "b" and bo != me:
                raise RuntimeError(f"Stationary-B expects local b_idx={op.b_idx}, owner={bo}, rank={me}")
            sa = OperandSlice(base=a.tile_ptr(ao), ld=a.ld, row0=op.a_slice.rows.start, col0=op.a_slice.cols.start,
                              rows=op.a_slice.shape[0], cols=op.a_slice.shape[1], remote=ao != me,
                              elem_bytes=a.itemsize)
            sb = OperandSlice(base=b.tile_ptr(bo), ld=b.ld, row0=op.b_slice.rows.start, col0=op.b_slice.cols.start,
                              rows=op.b_slice.shape[0], cols=op.b_slice.shape[1], remote=bo != me,
                              elem_bytes=b.itemsize)
            if split_f32:
                from dataclasses import replace

                a_hi, a_lo, b_hi, b_lo = replace(sa, split=1), replace(sa, split=2), replace(sb, split=1), replace(sb, split=2)
                segs += [(a_lo, b_hi), (a_hi, b_lo), (a_hi, b_hi)]      # small terms first
            else:
                segs.append((sa, sb))
        builder.add_task(TaskSpec(c_ptr=c_ptr, ldc=c.ld, m=m, n=n, c_mode=mode, c_dtype=torch_dtype_code(c.dtype),
                                  segments=segs, c_remote=c_owner != me))
    if split_k:
        builder.merge_row_tasks()      # skinny problems: tasks of a few rows each that share their B slices become one
    return builder.build(state.status_ptr), needs_zero


def _program(kind: str, a: DistMatrix, b: DistMatrix, c: DistMatrix, ops: Sequence[MultiplyOp], fuse: bool,
             beta: int = 1):
    key = (kind, a.buffer.ptr(a.rank), b.buffer.ptr(b.rank), c.buffer.ptr(c.rank), c.rank, fuse, beta)
    hit = _program_cache.get(key)
    if hit is not None and (hit[0] is ops or hit[0] == ops) and hit[1] == (a.layout, b.layout, c.layout):
        return hit[2]
    prog = lower_plan(kind, a, b, c, ops, fuse_replica_reduce=fuse, beta=beta)
    _program_cache[key] = (ops, (a.layout, b.layout, c.layout), prog)
    trace.register(f"stationary_{kind} rank{c.rank} {a.shape[0]}x{b.shape[1]}x{a.shape[1]} beta{beta}", prog[0])
    return prog


def cached_programs() -> list:
    """``(label, FusedProgram)`` of every lowered plan in the cache (for timeline tracing of programs that exist already)."""
    out = []
    for key, (_ops, _layouts, prog) in _program_cache.items():
        out.append((f"stationary_{key[0]} rank{key[4]} beta{key[6]}", prog[0]))
    return out


def _can_fuse(a: DistMatrix, b: DistMatrix, c: DistMatrix) -> bool:
    if not c.world.is_cuda:
        return False
    if a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16:
        return c.dtype in (torch.float32, torch.bfloat16)
    # fp32 operands (the reference's benchmark dtype, benchmark/matmul_bench_worker.py:163-165) run through the
    # same kernel as three bf16 products with fp32 accumulation; C stays fp32
    return a.dtype == torch.float32 and b.dtype == torch.float32 and c.dtype == torch.float32


# ----------------------------------------------------------------------------- fused executor
def _run_fused(kind: str, a: DistMatrix, b: DistMatrix, c: DistMatrix, ops: Sequence[MultiplyOp], *,
               fuse_replica_reduce: bool = True, barriers: bool = True, beta: int = 1,
               checksum: torch.Tensor | None = None) -> None:
    from ..ops.device import DeviceState

    world = c.world
    state = DeviceState.get(c.device)
    prog, needs_zero = _program(kind, a, b, c, ops, fuse_replica_reduce, beta)
    if needs_zero:        # several ranks add into C: clear it before the entry barrier lets anyone push
        pad = c.local_padded
        state.zero_2d(pad.data_ptr(), c.ld * c.itemsize, pad.shape[0], c.ld * c.itemsize)
    prof = profile.enabled
    if prof:
        e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        e0.record()
    # Entry barrier: every rank's operands (and zeroed C) are in place before any peer touches
    # them; it also clears this plan's chunk counters.
    if barriers or prog.num_clear:
        if barriers:
            world.device_barrier(prog.clear_ptr, prog.num_clear)
        else:
            state.zero_2d(prog.clear_ptr, prog.num_clear * 4, 1, prog.num_clear * 4)
    if prof:
        e1.record()
    if checksum is not None:
        if checksum.dtype != torch.float64 or checksum.numel() < 1 or checksum.device != c.device:
            raise ValueError("checksum must be a float64 tensor on the device of C")
        prog.params.checksum = checksum.data_ptr()
    try:
        prog.launch(state.stream())
    finally:
        prog.params.checksum = 0
    state.launches += 1
    if prof:
        e2.record()
    # Exit barrier: all pushes into this rank's C have landed and peers are done reading A / B.
    if barriers:
        world.device_barrier()
    if prof:
        e3.record()
        profile.record_events("comm_sync", e0, e1)
        profile.record_events("compute", e1, e2)
        profile.record_events("comm_sync", e2, e3)


# ----------------------------------------------------------------------------- tilewise executor
def _acc_dtype(dtype: torch.dtype) -> torch.dtype:
    return torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype


def _run_tilewise(kind: str, a: DistMatrix, b: DistMatrix, c: DistMatrix, ops: Sequence[MultiplyOp]) -> None:
    """Region by region: fetch the needed slices, multiply with the library matmul, add into C.
    Operand slices (not whole tiles) are fetched."""
    me = c.rank
    clock = time.perf_counter
    for region in P.group_ops(ops):
        acc = None
        for op in region.ops:
            t0 = clock()
            a_view = R.get_tile(a, op.a_idx, region=op.a_slice)
            b_view = R.get_tile(b, op.b_idx, region=op.b_slice)
            t1 = clock()
            prod = torch.matmul(a_view.to(_acc_dtype(a.dtype)), b_view.to(_acc_dtype(b.dtype)))
            acc = prod if acc is None else acc.add_(prod)
            t2 = clock()
            profile.add_comm_sync(t1 - t0)
            profile.add_compute(t2 - t1)
            R.release_tile(a_view)
            R.release_tile(b_view)
        owner = _owner(c, region.c_idx)
        t0 = clock()
        if owner == me and kind == "c":
            c_view = R.tile(c, region.c_idx)[region.c_slice.rows.as_slice(), region.c_slice.cols.as_slice()]
            c_view.add_(acc.to(c.dtype))
            profile.add_compute(clock() - t0)
            continue
        R.accumulate_tile(c, region.c_idx, acc.to(c.dtype), slice_=region.c_slice)
        profile.add_comm_issue(clock() - t0)


# ----------------------------------------------------------------------------- entry points
def _execute(kind: str, a: Any, b: Any, c: Any, ops: Sequence[MultiplyOp] | None, *, local_only: bool,
             executor: str | None, fuse_replica_reduce: bool, barriers: bool, beta: int = 1,
             checksum: torch.Tensor | None = None) -> list[MultiplyOp]:
    if beta not in (0, 1):
        raise ValueError("beta must be 0 (C = A @ B) or 1 (C += A @ B)")
    a, b, c = resolve(a), resolve(b), resolve(c)
    world = c.world
    rep_c = T.replication_factor(c.layout)
    if ops is None:
        build = P.build_stationary_c_ops if kind == "c" else P.build_stationary_b_ops
        ops = build(a.layout, b.layout, c.layout, local_only=local_only, rank=c.rank)
    if executor is None:
        executor = "fused" if _can_fuse(a, b, c) else "tilewise"
    if executor == "fused":
        if not _can_fuse(a, b, c):
            raise RuntimeError("the fused executor needs a CUDA world and bfloat16 (or float32) A / B")
        if rep_c > 1 and not fuse_replica_reduce and T.my_replica(c.layout, c.rank) != 0:
            c.local_padded.zero_()
        _run_fused(kind, a, b, c, ops, fuse_replica_reduce=fuse_replica_reduce, barriers=barriers, beta=beta,
                   checksum=checksum)
        if rep_c > 1 and not fuse_replica_reduce:
            R.reduce_replicas(c)
            world.device_barrier()
        return list(ops)
    if executor != "tilewise":
        raise ValueError(f"unknown executor {executor!r}")
    if checksum is not None:
        raise ValueError("checksum= is computed by the fused kernel's epilogue; the tilewise executor has none")
    if beta == 0:
        c.local_padded.zero_()
    if rep_c > 1 and T.my_replica(c.layout, c.rank) != 0:
        # Partial results are reduced into replica 0; stale values of other replicas must not be re-added.
        c.local_padded.zero_()
    if barriers:
        world.device_barrier()
    _run_tilewise(kind, a, b, c, ops)
    if barriers:
        world.device_barrier()
    if rep_c > 1:
        R.reduce_replicas(c)
        if barriers:
            world.device_barrier()
    return list(ops)


def execute_stationary_c(a: Any, b: Any, c: Any, *, local_only: bool = True, release_remote_tiles: bool = True,
                         use_async: bool | None = None, max_outstanding_prefetch: int = 1,
                         executor: str | None = None, fuse_replica_reduce: bool = True,
                         barriers: bool = True, beta: int = 1, checksum: torch.Tensor | None = None) -> list[MultiplyOp]:
    """``C += A @ B`` with the owner of every C tile computing it.  Returns the op list.

    ``checksum`` (fused executor): a float64 device tensor to whose first element this rank's kernel adds the sum of
    all values it writes or adds into C in this call (its share of ``sum(A @ B)``); it is never reset."""
    return _execute("c", a, b, c, None, local_only=local_only, executor=executor,
                    fuse_replica_reduce=fuse_replica_reduce, barriers=barriers, beta=beta, checksum=checksum)


def execute_stationary_b(a: Any, b: Any, c: Any, *, local_only: bool = True, release_remote_tiles: bool = True,
                         use_async: bool | None = None, max_outstanding_prefetch: int = 1,
                         max_outstanding_accumulates: int = 4, num_compute_streams: int = 2,
                         executor: str | None = None, fuse_replica_reduce: bool = True,
                         barriers: bool = True, beta: int = 1, checksum: torch.Tensor | None = None) -> list[MultiplyOp]:
    """``C += A @ B`` with the owner of every B tile multiplying it and pushing partial C tiles.
    ``checksum``: see :func:`execute_stationary_c`."""
    return _execute("b", a, b, c, None, local_only=local_only, executor=executor,
                    fuse_replica_reduce=fuse_replica_reduce, barriers=barriers, beta=beta, checksum=checksum)


def execute_stationary_c_ops(a: Any, b: Any, c: Any, ops: Sequence[MultiplyOp], *, release_remote_tiles: bool = True,
                             barriers: bool = True) -> None:
    """Execute a given Stationary-C op list op by op (tilewise executor)."""
    _execute("c", a, b, c, ops, local_only=True, executor="tilewise", fuse_replica_reduce=False, barriers=barriers)


def execute_stationary_c_ops_async(a: Any, b: Any, c: Any, ops: Sequence[MultiplyOp], *,
                                   release_remote_tiles: bool = True, max_outstanding_prefetch: int = 1,
                                   barriers: bool = True) -> None:
    """Execute a given Stationary-C op list with the fused kernel when possible."""
    _execute("c", a, b, c, ops, local_only=True, executor=None, fuse_replica_reduce=True, barriers=barriers)


def execute_stationary_b_ops(a: Any, b: Any, c: Any, ops: Sequence[MultiplyOp], *, release_remote_tiles: bool = True,
                             barriers: bool = True) -> None:
    _execute("b", a, b, c, ops, local_only=True, executor="tilewise", fuse_replica_reduce=False, barriers=barriers)


def execute_stationary_b_ops_async(a: Any, b: Any, c: Any, ops: Sequence[MultiplyOp], *,
                                   release_remote_tiles: bool = True, max_outstanding_prefetch: int = 1,
                                   max_outstanding_accumulates: int = 4, num_compute_streams: int = 2,
                                   barriers: bool = True) -> None:
    _execute("b", a, b, c, ops, local_only=True, executor=None, fuse_replica_reduce=True, barriers=barriers)


def row_partitioned_matmul(a: Any, b: Any, c: Any, **kwargs) -> list[MultiplyOp]:
    """``C += A @ B`` for three row-partitioned matrices as a ring: every rank walks the B row tiles starting at
    its own index and multiplies them with the matching K slice of its local A rows.  This is the Stationary-C
    plan of the row / row / row triple (the reference keeps a hand-written version of it,
    dtensor_mm_handler.py:19-79); layouts are checked, execution is the fused kernel."""
    la, lb, lc = (resolve(x).layout for x in (a, b, c))
    for lay in (la, lb, lc):
        if T.grid_shape(lay)[1] != 1 or T.replication_factor(lay) != 1:
            raise ValueError("row_partitioned_matmul expects row-partitioned, unreplicated matrices")
    return execute_stationary_c(a, b, c, **kwargs)


def matmul(a: Any, b: Any, c: Any, *, method: str = "auto", **kwargs) -> list[MultiplyOp]:
    """``C += A @ B`` with ``method`` in {auto, stationary_c, stationary_b, min_traffic}."""
    ra, rb, rc = resolve(a), resolve(b), resolve(c)
    chosen = P.select_method(method, rb.layout, rc.layout, ra.layout, in_bytes=ra.itemsize, c_bytes=rc.itemsize)
    if chosen == "stationary_b":
        return execute_stationary_b(a, b, c, **kwargs)
    return execute_stationary_c(a, b, c, **kwargs)
