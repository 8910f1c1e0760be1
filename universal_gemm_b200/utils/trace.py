"""Device-side timeline of the fused GEMM kernels.

With tracing on, every persistent CTA writes ``globaltimer`` stamps per output tile: when its TMA producer
reached the tile, how long it waited for staged (remote) operand chunks, when the tensor-core loop of the
tile could start, when its accumulator was complete and when the epilogue had pushed it out, plus a summary
record per CTA (start, end, when its fetch warps ran dry, pieces copied).  The reference's profiler
(dtensor_profile.py:1-60) accumulates three host-side counters; this is the in-kernel counterpart that the
fused design needs, because a whole plan is one launch.

    UGEMM_TRACE=1 python bench.py --trace-dir out/         # or: trace.enable() before the first matmul
    summary = trace.collect()[0]["summary"]

Record layout: ``UG_TR_*`` in ops/csrc/ugemm_b200.h.  Everything below the ``register`` hook is plain numpy
and runs without a GPU.
"""
from __future__ import annotations

import json
import os
import weakref
from typing import Any

import numpy as np

TILE, PROD_BEGIN, PROD_FLAGWAIT, PROD_END, MMA_BEGIN, MMA_ISSUED, EPI_BEGIN, EPI_END, MMA_CLK, EPI_CLK = range(10)
S_START, S_FETCH_END, S_END, S_PIECES, S_CLK_START, S_CLK_END = range(6)

enabled: bool = os.environ.get("UGEMM_TRACE", "0") not in ("", "0")

_programs: list[tuple[str, Any]] = []          # (label, weakref to FusedProgram)


def enable() -> None:
    """Trace programs lowered from now on (already cached programs: call ``program.enable_trace()``)."""
    global enabled
    enabled = True


def disable() -> None:
    global enabled
    enabled = False


def register(label: str, program: Any) -> None:
    """Called by the executor for every newly lowered program."""
    if not enabled:
        return
    program.enable_trace()
    _programs.append((label, weakref.ref(program)))


def reset() -> None:
    _programs.clear()


def attach_cached() -> int:
    """Turn tracing on for the programs the executor has lowered already; returns how many."""
    from ..parallel import exec as X

    known = {id(ref()) for _, ref in _programs}
    n = 0
    for label, prog in X.cached_programs():
        prog.enable_trace()
        if id(prog) not in known:
            _programs.append((label, weakref.ref(prog)))
        n += 1
    return n


def detach_all() -> None:
    for _, ref in _programs:
        prog = ref()
        if prog is not None:
            prog.disable_trace()
    _programs.clear()


# ----------------------------------------------------------------------------- analysis (numpy only)
def summarize(arr: np.ndarray, *, pair: bool = False) -> dict:
    """Figures of one launch from its ``[grid, slots + 1, fields]`` timeline (times in microseconds from the first
    CTA's start)."""
    arr = np.asarray(arr, dtype=np.int64)
    grid, slots = arr.shape[0], arr.shape[1] - 1
    tiles, summ = arr[:, :slots, :], arr[:, slots, :]
    starts = summ[:, S_START]
    live = starts > 0
    if not live.any():
        return {"grid": int(grid), "recorded_tiles": 0}
    t0 = int(starts[live].min())
    t_end = int(summ[live, S_END].max())
    us = lambda ns: float(ns) / 1e3                                            # noqa: E731
    rec = tiles[:, :, TILE] > 0
    out: dict = {"grid": int(grid), "pair": bool(pair), "slots": int(slots),
                 "recorded_tiles": int(rec[::2].sum() if pair else rec.sum()),
                 "kernel_us": us(t_end - t0),
                 "cta_start_spread_us": us(int(starts[live].max()) - t0)}
    clk = (summ[:, S_CLK_END] - summ[:, S_CLK_START])[live]
    dur = (summ[:, S_END] - summ[:, S_START])[live]
    if (clk > 0).any() and (dur > 0).all():
        out["sm_clock_ghz"] = float(np.median(clk[clk > 0] / dur[clk > 0]))      # SM cycles per nanosecond
    has_mma = rec & (tiles[:, :, MMA_BEGIN] > 0) & (tiles[:, :, EPI_BEGIN] > 0)
    if has_mma.any():
        main = (tiles[:, :, EPI_BEGIN] - tiles[:, :, MMA_BEGIN])[has_mma]
        out["first_mma_us"] = us(int(tiles[:, :, MMA_BEGIN][has_mma].min()) - t0)
        out["main_us_mean"] = us(main.mean())
        out["main_us_p95"] = us(np.percentile(main, 95))
        out["main_us_max"] = us(main.max())
        by_iter = []
        for i in range(slots):
            sel = has_mma[:, i]
            if sel.any():
                by_iter.append(round(us((tiles[:, i, EPI_BEGIN] - tiles[:, i, MMA_BEGIN])[sel].mean()), 2))
        out["main_us_by_iteration"] = by_iter
        if arr.shape[2] > EPI_CLK:
            # SM clock during each main loop: cycles between the two stamps over nanoseconds between them
            cyc = tiles[:, :, EPI_CLK] - tiles[:, :, MMA_CLK]
            ns = tiles[:, :, EPI_BEGIN] - tiles[:, :, MMA_BEGIN]
            okc = has_mma & (tiles[:, :, MMA_CLK] > 0) & (cyc > 0) & (ns > 0)
            by_iter = []
            for i in range(slots):
                sel = okc[:, i]
                if sel.any():
                    by_iter.append(round(float((cyc[:, i][sel] / ns[:, i][sel]).mean()), 3))
            out["sm_clock_ghz_by_iteration"] = by_iter
    has_epi = rec & (tiles[:, :, EPI_BEGIN] > 0) & (tiles[:, :, EPI_END] > 0)
    if has_epi.any():
        epi = (tiles[:, :, EPI_END] - tiles[:, :, EPI_BEGIN])[has_epi]
        out["epilogue_us_mean"] = us(epi.mean())
        out["epilogue_us_max"] = us(epi.max())
        last_end = np.where(has_epi, tiles[:, :, EPI_END], 0).max(axis=1)
        done = last_end > 0
        out["cta_finish_spread_us"] = us(int(last_end[done].max()) - int(last_end[done].min()))
        out["last_epilogue_end_us"] = us(int(last_end[done].max()) - t0)
    wait = np.where(rec, tiles[:, :, PROD_FLAGWAIT], 0).sum(axis=1)
    out["flagwait_us_mean_per_cta"] = us(wait[live].mean())
    out["flagwait_us_max_per_cta"] = us(wait[live].max())
    if rec.any():
        by_iter = []
        for i in range(slots):
            sel = rec[:, i]
            if sel.any():
                by_iter.append(round(us(tiles[:, i, PROD_FLAGWAIT][sel].mean()), 2))
        out["flagwait_us_by_iteration"] = by_iter
    fetch_end = summ[:, S_FETCH_END]
    if (fetch_end > 0).any():
        out["fetch_end_us"] = us(int(fetch_end.max()) - t0)
        out["pieces_copied"] = int(summ[:, S_PIECES].sum())
        out["pieces_per_cta_min_max"] = [int(summ[live, S_PIECES].min()), int(summ[live, S_PIECES].max())]
    # share of the kernel during which a CTA's tensor loop had an accumulator in flight
    if has_mma.any():
        busy = np.where(has_mma, tiles[:, :, EPI_BEGIN] - tiles[:, :, MMA_BEGIN], 0).sum(axis=1)
        rows = has_mma.any(axis=1)
        # with two accumulator buffers consecutive main loops overlap slightly (issue runs ahead); clip at 1
        out["main_loop_share_of_kernel"] = float(min(1.0, busy[rows].mean() / max(t_end - t0, 1)))
    return out


def to_chrome_trace(arr: np.ndarray, *, pid: int = 0, label: str = "fused") -> list[dict]:
    """Events for chrome://tracing / Perfetto: one track per CTA with flag waits, main loops and epilogues."""
    arr = np.asarray(arr, dtype=np.int64)
    slots = arr.shape[1] - 1
    starts = arr[:, slots, S_START]
    if not (starts > 0).any():
        return []
    t0 = int(starts[starts > 0].min())
    ev: list[dict] = []

    def span(name: str, cta: int, b: int, e: int, args: dict) -> None:
        if b > 0 and e >= b:
            ev.append({"name": name, "cat": label, "ph": "X", "pid": pid, "tid": cta, "ts": (b - t0) / 1e3,
                       "dur": (e - b) / 1e3, "args": args})

    for cta in range(arr.shape[0]):
        for i in range(slots):
            r = arr[cta, i]
            if r[TILE] <= 0:
                continue
            args = {"tile": int(r[TILE]) - 1, "iteration": i}
            span("load", cta, int(r[PROD_BEGIN]), int(r[PROD_END]), {**args, "flagwait_us": float(r[PROD_FLAGWAIT]) / 1e3})
            span("main", cta, int(r[MMA_BEGIN]), int(r[EPI_BEGIN]), args)
            span("epilogue", cta, int(r[EPI_BEGIN]), int(r[EPI_END]), args)
        s = arr[cta, slots]
        if s[S_FETCH_END] > 0:
            span("fetch", cta, int(s[S_START]), int(s[S_FETCH_END]), {"pieces": int(s[S_PIECES])})
    return ev


def device_breakdown(summary: dict) -> dict:
    """Split one launch's kernel time the way the host profiler names things (``utils.profile``; reference
    dtensor_profile.py:1-37), but from the device's own stamps, in seconds, averaged over the CTAs:
    ``comm_sync`` = producers waiting for staged (remote) chunks, ``compute`` = main loops,
    ``epilogue`` = exposed part of the epilogues, ``other`` = start-up, tail and idle."""
    if not summary.get("recorded_tiles"):
        return {"comm_sync": 0.0, "compute": 0.0, "epilogue": 0.0, "other": 0.0}
    kernel = summary["kernel_us"] * 1e-6
    wait = summary.get("flagwait_us_mean_per_cta", 0.0) * 1e-6
    main = max(summary.get("main_loop_share_of_kernel", 0.0) * kernel - wait, 0.0)
    workers = summary["grid"] // 2 if summary.get("pair") else summary["grid"]
    tiles_per_worker = summary["recorded_tiles"] / max(workers, 1)
    # the epilogue is exposed when the accumulators are single buffered, i.e. when main loops do not fill the kernel
    epi_total = summary.get("epilogue_us_mean", 0.0) * 1e-6 * tiles_per_worker
    epi = min(epi_total, max(kernel - main - wait, 0.0))
    return {"comm_sync": wait, "compute": main, "epilogue": epi, "other": max(kernel - wait - main - epi, 0.0)}


def add_to_profile() -> int:
    """Add the device-side breakdown of every traced program's last launch to the ``utils.profile`` counters
    (``comm_sync`` and ``compute``; epilogue and idle time count as compute there).  Returns the number of launches."""
    from . import profile

    n = 0
    for item in collect():
        b = device_breakdown(item["summary"])
        profile.add_comm_sync(b["comm_sync"])
        profile.add_compute(b["compute"] + b["epilogue"] + b["other"])
        n += 1
    return n


# ----------------------------------------------------------------------------- collection
def collect() -> list[dict]:
    """Timelines of the last launch of every traced program that is still alive."""
    out = []
    for label, ref in _programs:
        prog = ref()
        if prog is None:
            continue
        arr = prog.read_trace()
        if arr is None:
            continue
        pair = bool(prog.params.cta_pair)
        out.append({"label": label, "stats": dict(prog.stats), "summary": summarize(arr, pair=pair), "raw": arr})
    return out


def dump(directory: str, *, rank: int = 0, chrome: bool = True) -> list[str]:
    """Write ``trace_rank<r>_<i>.json`` (summary) and, with ``chrome``, ``..._events.json`` per traced program."""
    os.makedirs(directory, exist_ok=True)
    paths = []
    for i, item in enumerate(collect()):
        base = os.path.join(directory, f"trace_rank{rank}_{i}")
        with open(base + ".json", "w", encoding="utf-8") as f:
            json.dump({"label": item["label"], "stats": item["stats"], "summary": item["summary"]}, f, indent=1,
                      default=str)
        paths.append(base + ".json")
        if chrome:
            with open(base + "_events.json", "w", encoding="utf-8") as f:
                json.dump({"traceEvents": to_chrome_trace(item["raw"], pid=rank, label=item["label"])}, f)
            paths.append(base + "_events.json")
    return paths
