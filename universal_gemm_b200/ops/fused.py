"""Host side of the fused stationary GEMM: lower a list of region tasks into the
device tables of ``ug_fused_gemm`` (tensor maps, tasks, K segments, staged-copy
pieces and their completion counters) and launch them.

A *task* is one output region ``C[0:m, 0:n] (+)= sum_s A_s @ B_s``; every ``A_s``/``B_s``
is a 2-D slice of some rank's tile.  Slices that live in this GPU's memory and
satisfy the TMA alignment rules are read in place; remote slices (peer memory)
and misaligned ones are *staged*: fetch warps inside the same kernel copy them
into a local, aligned staging buffer and the TMA producer waits on per-chunk
counters.  The order of the staged pieces follows the order in which the
persistent CTAs will need them.

The executors this replaces in the reference are host loops:
stationary_c_plan.py:358-523 and stationary_b_plan.py:340-564.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field, replace
from typing import Callable, Sequence

import numpy as np
import torch

from . import native
from .native import BN, BK

_PIECE_BYTES = 32 * 1024
# Tile variants.  kb_us: microseconds per 64-deep K block of one tile; epi_us: epilogue of a full fp32 tile stored
# into local memory; both measured with the in-kernel timeline on an 8192^3 GEMM under the power cap.  "hidden": the
# accumulators are double buffered, so the epilogue runs behind the next tile's main loop.
_VARIANTS = {
    128: dict(rows=128, cols=256, pair=False, kb_us=0.483, epi_us=3.6, hidden=True),
    256: dict(rows=256, cols=256, pair=False, kb_us=0.696, epi_us=7.1, hidden=False),
    "pair": dict(rows=256, cols=256, pair=True, kb_us=0.394, epi_us=4.0, hidden=True),
    "pair512": dict(rows=256, cols=512, pair=True, kb_us=0.695, epi_us=6.7, hidden=False),
}
_AUTO_VARIANTS = (128, 256, "pair")      # "pair512" measured level with 256 and quantises worse: on request only
_REMOTE_EPILOGUE_FACTOR = 1.3            # epilogue into a peer's C against local stores (10.6-11.1 vs 9.2 us on 2 GPUs)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass(frozen=True)
class OperandSlice:
    """``rows x cols`` slice starting at ``(row0, col0)`` of a row-major tile.

    ``base`` is the address, in this process, of element (0, 0) of the tile's
    storage and ``ld`` its row pitch in elements.  ``remote`` marks memory of
    another GPU (it is then never handed to TMA).
    """

    base: int
    ld: int
    row0: int
    col0: int
    rows: int
    cols: int
    remote: bool = False
    elem_bytes: int = 2
    # fp32 operands run as three bf16 products (a = hi + lo with hi = bf16(a), lo = bf16(a - hi);
    # A @ B ~ Ahi Bhi + Ahi Blo + Alo Bhi): split = 1 names the high part of an fp32 slice, 2 the low part.
    # Such a slice has elem_bytes = 4 and is always staged; the fetch warps convert while they copy.
    split: int = 0

    def tma_ok(self) -> bool:
        return self.split == 0 and (not self.remote) and self.base % 16 == 0 \
            and (self.ld * self.elem_bytes) % 16 == 0 and (self.col0 * self.elem_bytes) % 16 == 0

    def vector_ok(self) -> bool:
        return self.base % 16 == 0 and (self.ld * self.elem_bytes) % 16 == 0 \
            and (self.col0 * self.elem_bytes) % 16 == 0

    def address(self, r: int = 0, c: int = 0) -> int:
        return self.base + ((self.row0 + r) * self.ld + self.col0 + c) * self.elem_bytes

    # the three operations below exist on StackedSlice too
    def row_parts(self) -> list[tuple["OperandSlice", int]]:
        """(contiguous source, first row of it in this slice) pairs."""
        return [(self, 0)]

    def with_cols(self, first: int, count: int) -> "OperandSlice":
        return replace(self, col0=self.col0 + first, cols=count)

    def with_split(self, split: int) -> "OperandSlice":
        return replace(self, split=split)

    def remote_bytes(self) -> int:
        return self.rows * self.cols * self.elem_bytes if self.remote else 0


@dataclass(frozen=True)
class StackedSlice:
    """Row slices of several tiles (same columns, same dtype) stacked into one A operand.  It exists only in the
    staging buffer: the fetch warps copy every part, local ones too, to its place in the stack.  Used to merge the
    tasks of a skinny problem whose A is partitioned by rows (M = 64 on 8 ranks gives tiles of 8 rows; one task per
    tile would run a full 128-row tensor tile, and stream all of B, for 8 rows of output)."""

    parts: tuple[OperandSlice, ...]

    @property
    def rows(self) -> int:
        return sum(p.rows for p in self.parts)

    @property
    def cols(self) -> int:
        return self.parts[0].cols

    @property
    def elem_bytes(self) -> int:
        return self.parts[0].elem_bytes

    @property
    def split(self) -> int:
        return self.parts[0].split

    @property
    def remote(self) -> bool:
        return any(p.remote for p in self.parts)

    def tma_ok(self) -> bool:
        return False

    def row_parts(self) -> list[tuple[OperandSlice, int]]:
        out, off = [], 0
        for p in self.parts:
            out.append((p, off))
            off += p.rows
        return out

    def with_cols(self, first: int, count: int) -> "StackedSlice":
        return StackedSlice(tuple(p.with_cols(first, count) for p in self.parts))

    def with_split(self, split: int) -> "StackedSlice":
        return StackedSlice(tuple(p.with_split(split) for p in self.parts))

    def remote_bytes(self) -> int:
        return sum(p.remote_bytes() for p in self.parts)


@dataclass
class TaskSpec:
    c_ptr: int
    ldc: int
    m: int
    n: int
    c_mode: int
    c_dtype: int
    segments: list[tuple[OperandSlice, OperandSlice]] = field(default_factory=list)
    c_remote: bool = False      # C lives in a peer's memory (the epilogue pushes over NVLink)
    tile_n: int = BN            # columns per output tile (128 for tasks moved into the last, partial wave)
    # Output rows that live in several places (a task merged from tasks of different C tiles): (address of the first
    # row's first column, row pitch in elements, rows) per part, in row order; c_ptr / ldc are then unused.
    c_rows: tuple[tuple[int, int, int], ...] | None = None


@dataclass
class _Staged:
    kind: str            # "a" (chunks of BM rows) or "b" (chunks of BN columns)
    src: OperandSlice
    offset: int          # byte offset into the staging buffer
    ld: int              # elements
    flag_base: int
    num_chunks: int
    map_index: int = -1
    pieces_of: "_Staged | None" = None   # low part of a split fp32 slice: the high part's pieces fill this buffer too
    low: "_Staged | None" = None         # high part of a split fp32 slice: where the low part goes


class FusedProgram:
    """Device-resident tables of one lowered plan, ready to launch."""

    def __init__(self, *, device: torch.device, tables: torch.Tensor, staging: torch.Tensor | None,
                 params: native.FusedParams, grid: int, clear_ptr: int, num_clear: int, stats: dict):
        self.device = device
        self._tables = tables
        self._staging = staging
        self.params = params
        self.grid = grid
        self.clear_ptr = clear_ptr
        self.num_clear = num_clear
        self.stats = stats
        self._trace: torch.Tensor | None = None

    # ------------------------------------------------------------------ optional per-tile timeline
    def enable_trace(self, slots: int | None = None) -> None:
        """Make later launches record a timeline: one record of ``native.TRACE_FIELDS`` uint64 words per (CTA, tile iteration) plus a
        summary record per CTA (layout: ``UG_TR_*`` in ugemm_b200.h).  Each launch overwrites the previous one."""
        workers = max(self.grid // 2 if self.params.cta_pair else self.grid, 1)
        if slots is None:     # with dynamic claiming a fast worker runs more tiles than the average
            slots = (int(self.params.total_tiles) + workers - 1) // workers * 5 // 4 + 2
        slots = max(int(slots), 1)
        self._trace = torch.zeros(self.grid, slots + 1, native.TRACE_FIELDS, dtype=torch.int64, device=self.device)
        self.params.trace = self._trace.data_ptr()
        self.params.trace_slots = slots

    def disable_trace(self) -> None:
        self._trace = None
        self.params.trace = 0
        self.params.trace_slots = 0

    def read_trace(self):
        """The timeline of the last launch as a numpy array ``[grid, slots + 1, native.TRACE_FIELDS]`` (synchronises the device);
        ``None`` when tracing is off."""
        if self._trace is None:
            return None
        torch.cuda.synchronize(self.device)
        return self._trace.cpu().numpy()

    @property
    def num_pieces(self) -> int:
        return int(self.params.num_pieces)

    def set_status_ptr(self, ptr: int) -> None:
        self.params.status = ptr

    def reset_flags(self, stream: int) -> None:
        """Zero the chunk counters and the piece cursor (needed before every launch
        when the program stages anything and no barrier kernel clears them)."""
        if self.num_clear > 0:
            native.check(native.lib().ug_zero_2d(self.clear_ptr, self.num_clear * 4, 1, self.num_clear * 4,
                                                 ctypes.c_void_p(stream)), "ug_zero_2d(flags)")

    def launch(self, stream: int) -> None:
        fn = native.lib().ug_fused_gemm_pair if self.params.cta_pair else native.lib().ug_fused_gemm
        native.check(fn(ctypes.byref(self.params), self.grid, ctypes.c_void_p(stream)), "ug_fused_gemm")


class FusedProgramBuilder:
    def __init__(self, device: torch.device, *, num_sms: int | None = None, timeout_ns: int = 4_000_000_000,
                 range_check: Callable[[int, int, str], None] | None = None, tile_m: int | None = None,
                 split_k: bool = False):
        self.device = torch.device(device)
        self.split_k = bool(split_k)
        if num_sms is None:
            num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.num_sms = int(num_sms)
        self.timeout_ns = int(timeout_ns)
        self.range_check = range_check
        if tile_m is None and os.environ.get("UGEMM_TILE_M"):
            env = os.environ["UGEMM_TILE_M"]
            tile_m = env if env.startswith("pair") else int(env)
        if tile_m not in (None, 128, 256, "pair", "pair512"):
            raise ValueError('tile_m must be 128, 256, "pair" or "pair512"')
        self.tile_m = tile_m
        self.tasks: list[TaskSpec] = []

    def merge_row_tasks(self, max_rows: int = 256) -> int:
        """Merge tasks that multiply different rows of A with the same B slices (and write equally wide regions of an
        fp32 C) into one task whose A is the stack of their row slices and whose output rows go to their several
        places.  Only tasks of fewer than 128 rows are merged, up to ``max_rows`` rows per merged task: this is for
        skinny problems, where every such task would otherwise occupy a whole tensor tile and stream B again.
        Returns the number of tasks saved."""
        groups: dict[tuple, list[TaskSpec]] = {}
        order: list[tuple] = []
        for t in self.tasks:
            key = None
            if t.m < 128 and t.c_dtype == native.DT_F32 and t.c_rows is None and (t.ldc * 4) % 16 == 0 and \
                    t.c_ptr % 4 == 0 and all(isinstance(a, OperandSlice) for a, _ in t.segments):
                key = (t.n, t.c_mode, t.tile_n, (t.c_ptr % 16, (t.ldc * 4) % 16),
                       tuple((b, a.col0, a.cols, a.elem_bytes, a.split) for a, b in t.segments))
            else:
                key = ("single", id(t))
            if key not in groups:
                groups[key] = []
                order.append(key)
            groups[key].append(t)
        merged: list[TaskSpec] = []
        for key in order:
            bucket = groups[key]
            while bucket:
                take, rows = [], 0
                while bucket and (not take or rows + bucket[0].m <= max_rows):
                    rows += bucket[0].m
                    take.append(bucket.pop(0))
                if len(take) == 1:
                    merged.append(take[0])
                    continue
                segs = [(StackedSlice(tuple(t.segments[i][0] for t in take)), take[0].segments[i][1])
                        for i in range(len(take[0].segments))]
                merged.append(TaskSpec(c_ptr=take[0].c_ptr, ldc=take[0].ldc, m=rows, n=take[0].n, c_mode=take[0].c_mode,
                                       c_dtype=take[0].c_dtype, segments=segs, c_remote=any(t.c_remote for t in take),
                                       tile_n=take[0].tile_n, c_rows=tuple((t.c_ptr, t.ldc, t.m) for t in take)))
        saved = len(self.tasks) - len(merged)
        self.tasks = merged
        return saved

    def add_task(self, task: TaskSpec) -> None:
        if task.m <= 0 or task.n <= 0 or not task.segments:
            return
        for a, b in task.segments:
            if a.rows != task.m or b.cols != task.n or a.cols != b.rows or a.cols <= 0:
                raise ValueError(f"inconsistent segment shapes: A {a.rows}x{a.cols}, B {b.rows}x{b.cols}, "
                                 f"C {task.m}x{task.n}")
        self.tasks.append(task)

    # ------------------------------------------------------------------ tile shape
    def choose_tile_m(self):
        """Pick the tile variant (128, 256 or "pair") from a time model of the persistent grid.

        Per tile: main loop = K blocks x the variant's measured time per K block; epilogue = the variant's measured
        epilogue time, scaled by the bytes of C it moves (bf16 halves them, read-modify-write doubles them) and by a
        factor when C is a peer's memory.  Variants with double-buffered accumulators pay max(main, epilogue) per
        tile, the others main + epilogue.  Tiles are dealt round-robin to the workers (CTAs, or CTA pairs) as the
        kernel does; the variant with the smallest busiest worker wins."""
        if self.tile_m is not None:
            return self.tile_m
        best = None
        for variant in _AUTO_VARIANTS:
            total = self.model_us(variant)
            if total is not None and (best is None or total < best[0]):
                best = (total, variant)
        return best[1] if best else 128

    def model_us(self, variant) -> float | None:
        """Modelled kernel time in microseconds of the tasks added so far under tile variant ``variant`` (the busiest
        worker of the model described in :meth:`choose_tile_m`); ``None`` when the variant cannot run here."""
        v = _VARIANTS[variant]
        workers = self.num_sms // 2 if v["pair"] else self.num_sms
        if workers < 1:
            return None
        per_worker = [0.0] * workers
        tile = 0
        tasks = self.tasks
        if self.split_k and os.environ.get("UGEMM_SPLIT_K", "1") != "0":
            tasks = self._split_k([t if v["cols"] == BN else self._with_tile_n(t, v["cols"]) for t in tasks],
                                  v["rows"], workers)
        for t in tasks:
            kblocks = sum((a.cols + BK - 1) // BK for a, _ in t.segments)
            tiles = ((t.m + v["rows"] - 1) // v["rows"]) * ((t.n + v["cols"] - 1) // v["cols"])
            main = kblocks * v["kb_us"]
            epi = v["epi_us"] * (0.75 if t.c_dtype == native.DT_BF16 else 1.0) \
                * (1.5 if t.c_mode == native.C_ADD else 1.0) * (_REMOTE_EPILOGUE_FACTOR if t.c_remote else 1.0)
            cost = max(main, epi) if v["hidden"] else main + epi
            full, rest = divmod(tiles, workers)
            if full:
                for w in range(workers):
                    per_worker[w] += full * cost
            for _ in range(rest):
                per_worker[tile % workers] += cost
                tile += 1
        return max(per_worker)

    # ------------------------------------------------------------------ lowering
    def build(self, status_ptr: int) -> FusedProgram:
        dev = self.device
        variant = self.choose_tile_m()
        pair = variant in ("pair", "pair512")   # two CTAs share a 256-row tile; each loads 128 rows of A
        wide = variant == "pair512"             # ... of 512 columns (two UMMAs per K step, accumulators fill TMEM)
        BM = 256 if pair else variant
        a_box_rows = 128 if pair else BM
        workers = (self.num_sms // 2) if pair else self.num_sms
        tasks = self.tasks
        if wide:
            tasks = [replace(t, tile_n=2 * BN) if t.tile_n == BN else t for t in tasks]
        if os.environ.get("UGEMM_TAIL_SPLIT", "1") != "0":
            tasks = self._split_tail(tasks, BM, workers, 2 * BN if wide else BN)
        if self.split_k and os.environ.get("UGEMM_SPLIT_K", "1") != "0":
            tasks = self._split_k(tasks, BM, workers)
        map_keys: dict[tuple, int] = {}
        map_specs: list[tuple] = []

        def add_map(base_or_offset, staged: bool, inner: int, outer: int, stride_bytes: int, box: tuple[int, int]) -> int:
            key = (base_or_offset, staged, inner, outer, stride_bytes, box)
            idx = map_keys.get(key)
            if idx is None:
                idx = len(map_specs)
                map_keys[key] = idx
                map_specs.append(key)
            return idx

        staged: dict[tuple, _Staged] = {}
        staging_bytes = 0
        num_flags = 0

        def stage(kind: str, src: OperandSlice) -> _Staged:
            nonlocal staging_bytes, num_flags
            key = (kind, src)
            st = staged.get(key)
            if st is not None:
                return st
            if src.split == 2:                 # the low part lives beside its high part and shares its counters
                stage(kind, src.with_split(1))
                return staged[key]
            ld = _round_up(src.cols, 64)
            nbytes = _round_up(src.rows * ld * 2, 1024)        # staged data is always bf16
            chunks = (src.rows + BM - 1) // BM if kind == "a" else (src.cols + BN - 1) // BN
            st = _Staged(kind=kind, src=src, offset=staging_bytes, ld=ld, flag_base=num_flags, num_chunks=chunks)
            staging_bytes += nbytes
            num_flags += chunks
            staged[key] = st
            if src.split == 1:
                low = _Staged(kind=kind, src=src.with_split(2), offset=staging_bytes, ld=ld,
                              flag_base=st.flag_base, num_chunks=chunks, pieces_of=st)
                staging_bytes += nbytes
                st.low = low
                staged[(kind, low.src)] = low
            return st

        # Pass 1: decide direct vs staged per operand and lay out tasks / segments.
        seg_rows = []
        task_rows = []
        row_table: list[int] = []      # per-row C addresses of tasks whose output rows live in several places
        tile_begin = 0
        seg_sources: list[tuple[_Staged | None, _Staged | None]] = []
        for task in tasks:
            m_tiles = (task.m + BM - 1) // BM
            n_tiles = (task.n + task.tile_n - 1) // task.tile_n
            seg_begin = len(seg_rows)
            kblocks = 0
            for a, b in task.segments:
                row = dict(a_flag=-1, b_flag=-1, k_len=a.cols)
                if a.tma_ok():
                    row["a_map"] = add_map(a.base, False, a.col0 + a.cols, a.row0 + a.rows, a.ld * a.elem_bytes, (BK, a_box_rows))
                    row["a_row0"], row["a_col0"] = a.row0, a.col0
                    sa = None
                else:
                    sa = stage("a", a)
                    sa.map_index = add_map(sa.offset, True, a.cols, a.rows, sa.ld * 2, (BK, a_box_rows))
                    row["a_map"], row["a_row0"], row["a_col0"], row["a_flag"] = sa.map_index, 0, 0, sa.flag_base
                if b.tma_ok():
                    row["b_map"] = add_map(b.base, False, b.col0 + b.cols, b.row0 + b.rows, b.ld * b.elem_bytes, (64, BK))
                    row["b_row0"], row["b_col0"] = b.row0, b.col0
                    sb = None
                else:
                    sb = stage("b", b)
                    sb.map_index = add_map(sb.offset, True, b.cols, b.rows, sb.ld * 2, (64, BK))
                    row["b_map"], row["b_row0"], row["b_col0"], row["b_flag"] = sb.map_index, 0, 0, sb.flag_base
                seg_rows.append(row)
                seg_sources.append((sa, sb))
                kblocks += (a.cols + BK - 1) // BK
            c_elem = 4 if task.c_dtype == native.DT_F32 else 2
            c_vec = int(task.c_ptr % 16 == 0 and (task.ldc * c_elem) % 16 == 0)
            if task.c_ptr % c_elem == 0 and (task.ldc * c_elem) % 16 == 0:
                c_vec |= 2          # rows share one alignment phase: vector stores from the next 16-byte boundary on
            row_tab_at = -1
            if task.c_rows is not None:
                # rows in several places: the kernel reads each row's address from a table (bit 2 of c_vec); all
                # rows must share one 16-byte phase, which the vector stores of the epilogue rely on
                if task.c_dtype != native.DT_F32 or sum(r for _, _, r in task.c_rows) != task.m:
                    raise ValueError("a task with several output parts needs fp32 C and parts that add up to m")
                addrs = [ptr + i * ld * c_elem for ptr, ld, rows in task.c_rows for i in range(rows)]
                if len({x % 16 for x in addrs}) != 1 or addrs[0] % c_elem:
                    raise ValueError("the output rows of a merged task differ in alignment")
                c_vec = 2 | 4
                row_tab_at = len(row_table)
                row_table.extend(addrs)
            if task.tile_n != BN:
                c_vec |= task.tile_n << 16
            band = 2048 // BM
            group_m = m_tiles if m_tiles <= band else band
            task_rows.append(dict(c_ptr=task.c_ptr, ldc=task.ldc, m=task.m, n=task.n, seg_begin=seg_begin,
                                  seg_count=len(task.segments), tile_begin=tile_begin, m_tiles=m_tiles,
                                  n_tiles=n_tiles, kblocks=kblocks, c_mode=task.c_mode, c_dtype=task.c_dtype,
                                  c_vec=c_vec, group_m=group_m))
            task_rows[-1]["tile_n"] = task.tile_n
            task_rows[-1]["row_tab_at"] = row_tab_at
            tile_begin += m_tiles * n_tiles
        total_tiles = tile_begin
        if len(map_specs) > 4096:
            raise ValueError(f"plan needs {len(map_specs)} tensor maps (limit 4096)")

        if pair:
            sms = self.num_sms // 2 * 2
            grid = sms if (staged or 2 * total_tiles >= sms) else max(2 * total_tiles, 2)
            wave_tiles = grid // 2
        else:
            grid = self.num_sms if (staged or total_tiles >= self.num_sms) else max(total_tiles, 1)
            wave_tiles = grid

        # Pass 2: pieces of the staged copies, ordered by first use.
        staging = None
        staging_base = 0
        if staging_bytes:
            staging = torch.zeros(staging_bytes + 1024, dtype=torch.uint8, device=dev)
            staging_base = _round_up(staging.data_ptr(), 1024)
        pieces_by_chunk: dict[tuple[int, int], list[dict]] = {}
        flag_need = np.zeros(max(num_flags, 1), dtype=np.int32)
        for st in staged.values():
            if st.pieces_of is not None:
                continue
            src = st.src
            eb = src.elem_bytes
            dist_kib = 0
            if src.split:
                # convert while copying: mode 2 (16-byte loads) / 3 (4-byte loads); the distance to the low part's
                # buffer travels in the upper bits of the mode word, in KiB
                dist_kib = (st.low.offset - st.offset) >> 10
                if (st.low.offset - st.offset) % 1024 or dist_kib >= 1 << 22:
                    raise ValueError("staging area too large for split fp32 operands")
            for c in range(st.num_chunks):
                plist = []
                if st.kind == "a":
                    r0, r1 = c * BM, min(src.rows, (c + 1) * BM)
                    c0, c1 = 0, src.cols
                else:
                    r0, r1 = 0, src.rows
                    c0, c1 = c * BN, min(src.cols, (c + 1) * BN)
                row_bytes = (c1 - c0) * 2                      # payload per row of the (bf16) destination
                rpp = max(1, _PIECE_BYTES // max(row_bytes, 1))
                for part, first in src.row_parts():            # one contiguous source at a time
                    p0, p1 = max(r0, first), min(r1, first + part.rows)
                    if part.split:
                        mode = (2 if part.vector_ok() else 3) | (dist_kib << 8)
                    else:
                        mode = 0 if part.vector_ok() else 1
                    for r in range(p0, p1, rpp):
                        rows = min(rpp, p1 - r)
                        plist.append(dict(src=part.address(r - first, c0),
                                          dst=staging_base + st.offset + (r * st.ld + c0) * 2,
                                          src_ld=part.ld * eb, dst_ld=st.ld * 2, rows=rows, row_bytes=row_bytes,
                                          flag=st.flag_base + c, mode=mode))
                        if self.range_check is not None:
                            src_row = (c1 - c0) * eb
                            span = (rows - 1) * part.ld * eb + (_round_up(src_row, 16) if mode & 0xff in (0, 2) else src_row)
                            self.range_check(part.address(r - first, c0), span, "staged source")
                pieces_by_chunk[(id(st), c)] = plist
                flag_need[st.flag_base + c] = len(plist)

        ordered: list[dict] = []
        if staged:
            emitted: set[tuple[int, int]] = set()
            # Tile order of the persistent grid: CTA b runs tiles b, b + grid, ...  All CTAs walk
            # their K segments in order, so within a wave chunks are needed segment by segment.
            coords = self._tile_coords(task_rows)
            for wave_start in range(0, total_tiles, wave_tiles):
                wave = coords[wave_start:wave_start + wave_tiles]
                max_segs = max(task_rows[t]["seg_count"] for t, _, _ in wave)
                for s in range(max_segs):
                    for t, mt, nt in wave:
                        tr = task_rows[t]
                        if s >= tr["seg_count"]:
                            continue
                        sa, sb = seg_sources[tr["seg_begin"] + s]
                        b_first = nt * tr["tile_n"] // BN            # a 512-column tile spans two staged chunks
                        b_last = min(((nt + 1) * tr["tile_n"] - 1) // BN, (sb.num_chunks - 1) if sb else 0)
                        wanted = [(sa, mt)] + [(sb, ci) for ci in range(b_first, b_last + 1)]
                        for st, ci in wanted:
                            if st is None:
                                continue
                            key = (id(st.pieces_of or st), ci)
                            if key not in emitted:
                                emitted.add(key)
                                ordered.extend(pieces_by_chunk[key])
            for key, plist in pieces_by_chunk.items():   # chunks no tile asked for (cannot happen; keep counters sane)
                if key not in emitted:
                    ordered.extend(plist)

        # Pass 3: pack tables into one device buffer.
        seg_arr = np.zeros(max(len(seg_rows), 1), dtype=native.SEGMENT_DTYPE)
        for i, row in enumerate(seg_rows):
            for k, v in row.items():
                seg_arr[i][k] = v
        task_arr = np.zeros(max(len(task_rows), 1), dtype=native.TASK_DTYPE)
        for i, row in enumerate(task_rows):
            for k, v in row.items():
                if k not in ("tile_n", "row_tab_at"):
                    task_arr[i][k] = v
        piece_arr = np.zeros(max(len(ordered), 1), dtype=native.PIECE_DTYPE)
        for i, row in enumerate(ordered):
            for k, v in row.items():
                piece_arr[i][k] = v
        maps_blob = bytearray()
        for (base_or_off, is_staged, inner, outer, stride_bytes, box) in map_specs:
            base = staging_base + base_or_off if is_staged else base_or_off
            maps_blob += native.encode_tensor_map(base, native.DT_BF16, inner, outer, stride_bytes, box[0], box[1], 3)
        if not maps_blob:
            maps_blob = bytearray(128)

        def pad(b: bytes, align: int = 256) -> bytes:
            return b + bytes((-len(b)) % align)

        row_tab_arr = np.asarray(row_table or [0], dtype=np.uint64)
        lengths = [len(pad(bytes(x))) for x in (maps_blob, task_arr.tobytes(), seg_arr.tobytes(), piece_arr.tobytes(),
                                                flag_need.tobytes(), bytes(4 * (num_flags + 1)), bytes(8),
                                                row_tab_arr.tobytes())]
        offsets = np.cumsum([0] + lengths)
        tables = torch.empty(int(offsets[-1]) + 256, dtype=torch.uint8, device=dev)
        base = _round_up(tables.data_ptr(), 256)
        shift = base - tables.data_ptr()
        for i, row in enumerate(task_rows):          # tasks with a row table point at their part of it
            if row["row_tab_at"] >= 0:
                task_arr[i]["c_ptr"] = base + int(offsets[7]) + 8 * row["row_tab_at"]
                task_arr[i]["ldc"] = 0
        sections = [pad(bytes(maps_blob)), pad(task_arr.tobytes()), pad(seg_arr.tobytes()), pad(piece_arr.tobytes()),
                    pad(flag_need.tobytes()), pad(bytes(4 * (num_flags + 1))), pad(bytes(8)), pad(row_tab_arr.tobytes())]
        blob = np.frombuffer(b"".join(sections), dtype=np.uint8).copy()
        tables[shift:shift + len(blob)].copy_(torch.from_numpy(blob))

        params = native.FusedParams()
        params.maps = base + int(offsets[0])
        params.tasks = base + int(offsets[1])
        params.segs = base + int(offsets[2])
        params.pieces = base + int(offsets[3])
        params.flag_need = base + int(offsets[4])
        params.flags = base + int(offsets[5])
        params.piece_counter = params.flags + 4 * num_flags
        params.status = status_ptr
        params.num_maps = len(map_specs)
        params.num_tasks = len(task_rows)
        params.num_pieces = len(ordered)
        params.num_flags = num_flags
        params.total_tiles = total_tiles
        params.tile_m = BM
        params.cta_pair = 2 if wide else (1 if pair else 0)
        params.num_segs = len(seg_rows)
        # Dynamic tile claiming (two uint32 counters, re-armed by the kernel itself).  Default: on for the CTA-pair
        # variants, where it measured +6-9 % on the headline GEMM (workers finish 90 us apart instead of 450 us); off
        # for the one-CTA variants, where it measured level: under the power cap the SMs that finish early leave their
        # share of the power budget to the others.  UGEMM_DYNAMIC_TILES=0 / 1 overrides.
        dyn_env = os.environ.get("UGEMM_DYNAMIC_TILES", "")
        dynamic = pair if dyn_env == "" else dyn_env != "0"
        params.sched = base + int(offsets[6]) if dynamic else 0
        params.epi_poll_ns = int(os.environ.get("UGEMM_EPI_POLL_NS", "0"))
        # Loads in flight per fetch-warp lane.  Sixteen reach the link rate (450-530 GB/s) but slow the main loops that
        # run beside them by 25-40 % (the tiles' TMA loads and the fetch warps' loads share the SM's outstanding-request
        # capacity, and loads over NVLink hold it three times as long); eight still copy at 435 GB/s and cost 10 %.
        # A plan that needs its remote bytes no faster than 300 GB/s over its modelled kernel time takes eight.
        remote_total = sum(st.src.remote_bytes() for st in staged.values() if st.pieces_of is None)
        modelled_us = self.model_us(variant) or 0.0
        need_gbs = remote_total / (modelled_us * 1e3) if modelled_us > 0 else float("inf")
        params.fetch_depth = int(os.environ.get("UGEMM_FETCH_DEPTH", "0")) or (8 if need_gbs < 300.0 else 16)
        params.timeout_ns = self.timeout_ns
        stats = dict(tasks=len(task_rows), segments=len(seg_rows), tiles=total_tiles, maps=len(map_specs),
                     pieces=len(ordered), staged_bytes=staging_bytes, tile_m=variant if pair else BM,
                     indirect_rows=len(row_table), fetch_depth=int(params.fetch_depth),
                     push_bytes=sum(t.m * t.n * (4 if t.c_dtype == native.DT_F32 else 2) for t in tasks if t.c_remote),
                     model_us=round(self.model_us(variant) or 0.0, 1),
                     remote_bytes=sum(st.src.remote_bytes() for st in staged.values() if st.pieces_of is None),
                     grid=grid)
        return FusedProgram(device=dev, tables=tables, staging=staging, params=params, grid=grid,
                            clear_ptr=params.flags if staged else 0, num_clear=(num_flags + 1) if staged else 0,
                            stats=stats)

    @staticmethod
    def _split_tail(tasks: list[TaskSpec], bm: int, workers: int, tn: int = BN) -> list[TaskSpec]:
        """Halve the tile width of the tiles that would form the last, partly filled wave.

        With T tiles (``tn`` columns wide) on W workers the last wave holds T mod W tiles; if they are at most W / 2
        and consist of whole trailing tile columns of the last task(s), those columns become a task of their own with
        tiles of ``tn / 2`` columns: twice as many tiles of half the cost, so the last wave costs half a tile time
        instead of a full one."""
        BN = tn                                                        # noqa: N806 (tile width of this variant)
        counts = [((t.m + bm - 1) // bm) * ((t.n + BN - 1) // BN) for t in tasks]
        total = sum(counts)
        tail = total % workers if workers > 0 else 0
        if total <= workers or tail == 0 or 2 * tail > workers:
            return list(tasks)
        out = list(tasks)
        remaining = tail
        idx = len(out) - 1
        while remaining > 0 and idx >= 0:
            t = out[idx]
            m_tiles = (t.m + bm - 1) // bm
            n_tiles = (t.n + BN - 1) // BN
            if m_tiles > 2048 // bm:          # several raster bands: the last tiles are not whole columns
                return list(tasks)
            if m_tiles * n_tiles <= remaining:
                out[idx] = FusedProgramBuilder._columns(t, 0, t.n, BN // 2)
                remaining -= m_tiles * n_tiles
                idx -= 1
                continue
            if remaining % m_tiles:
                return list(tasks)
            cut = (n_tiles - remaining // m_tiles) * BN
            out[idx:idx + 1] = [FusedProgramBuilder._columns(t, 0, cut, BN),
                                FusedProgramBuilder._columns(t, cut, t.n, BN // 2)]
            remaining = 0
        return out

    @staticmethod
    def _with_tile_n(t: TaskSpec, tile_n: int) -> TaskSpec:
        return replace(t, tile_n=tile_n) if t.tile_n == BN else t

    @staticmethod
    def _split_k(tasks: list[TaskSpec], bm: int, workers: int) -> list[TaskSpec]:
        """Cut the K range of atomically accumulating tasks into several tasks when the plan has far fewer output
        tiles than workers (skinny GEMMs: M = 64 against N = K = 16383 gives a rank 8 tiles, each streaming all of
        B's rows through one SM).  Every part adds its partial product into C with ``red.add``, so the whole GPU
        streams B; the parts are whole K blocks, which keeps every slice's TMA alignment."""
        counts = [((t.m + bm - 1) // bm) * ((t.n + t.tile_n - 1) // t.tile_n) for t in tasks]
        total = sum(counts)
        if total == 0 or total > workers:
            return list(tasks)
        target = workers // total
        if target < 2:
            return list(tasks)
        out: list[TaskSpec] = []
        for t in tasks:
            kblocks = sum((a.cols + BK - 1) // BK for a, _ in t.segments)
            parts = min(target, kblocks // 4)
            if t.c_mode != native.C_ATOMIC or parts < 2:
                out.append(t)
                continue
            per = (kblocks + parts - 1) // parts            # K blocks per part
            cur: list[tuple[OperandSlice, OperandSlice]] = []
            room = per
            for a, b in t.segments:
                done = 0
                while done < a.cols:
                    take = min(a.cols - done, room * BK)
                    cur.append((a.with_cols(done, take), replace(b, row0=b.row0 + done, rows=take)))
                    done += take
                    room -= (take + BK - 1) // BK
                    if room <= 0:
                        out.append(replace(t, segments=cur))
                        cur, room = [], per
            if cur:
                out.append(replace(t, segments=cur))
        return out

    @staticmethod
    def _columns(t: TaskSpec, c0: int, c1: int, tile_n: int) -> TaskSpec:
        """The sub-task of ``t`` that covers output columns ``[c0, c1)``."""
        elem = 4 if t.c_dtype == native.DT_F32 else 2
        segs = [(a, replace(b, col0=b.col0 + c0, cols=c1 - c0)) for a, b in t.segments]
        c_rows = None if t.c_rows is None else tuple((ptr + c0 * elem, ld, rows) for ptr, ld, rows in t.c_rows)
        return TaskSpec(c_ptr=t.c_ptr + c0 * elem, ldc=t.ldc, m=t.m, n=c1 - c0, c_mode=t.c_mode, c_dtype=t.c_dtype,
                        segments=segs, c_remote=t.c_remote, tile_n=tile_n, c_rows=c_rows)

    @staticmethod
    def _tile_coords(task_rows: Sequence[dict]) -> list[tuple[int, int, int]]:
        """Linear tile index -> (task, m tile, n tile); mirrors ``locate`` in fused_gemm.cu."""
        out: list[tuple[int, int, int]] = []
        for t, tr in enumerate(task_rows):
            m_tiles, n_tiles, gm = tr["m_tiles"], tr["n_tiles"], tr["group_m"]
            for first_m in range(0, m_tiles, gm):
                band_m = min(gm, m_tiles - first_m)
                for nt in range(n_tiles):
                    for i in range(band_m):
                        out.append((t, first_m + i, nt))
        return out


def tile_coords_for_test(task_rows: Sequence[dict]) -> list[tuple[int, int, int]]:
    return FusedProgramBuilder._tile_coords(task_rows)
