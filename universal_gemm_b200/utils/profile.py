"""Coarse profiler: four accumulating counters (seconds) and a printed breakdown.

Same counter names, update functions and report as the reference's
dtensor_profile.py:1-60.  The GPU executors feed it from CUDA events instead of
host wall-clock: ``record_events`` queues (start, end) event pairs without
blocking, and ``print_stats`` / ``snapshot`` fold the finished pairs in.
"""
from __future__ import annotations

comm_issue: float = 0.0
comm_sync: float = 0.0
compute: float = 0.0
total_runtime: float = 0.0
enabled: bool = False

_pending: list[tuple[str, object, object]] = []


def add_comm_issue(duration_s: float) -> None:
    global comm_issue
    comm_issue += float(duration_s)


def add_comm_sync(duration_s: float) -> None:
    global comm_sync
    comm_sync += float(duration_s)


def add_compute(duration_s: float) -> None:
    global compute
    compute += float(duration_s)


def add_total_runtime(duration_s: float) -> None:
    global total_runtime
    total_runtime += float(duration_s)


def set_total_runtime(duration_s: float) -> None:
    global total_runtime
    total_runtime = float(duration_s)


def reset_stats() -> None:
    global comm_issue, comm_sync, compute, total_runtime
    comm_issue = comm_sync = compute = total_runtime = 0.0
    _pending.clear()


def enable(flag: bool = True) -> None:
    global enabled
    enabled = bool(flag)


def record_events(kind: str, start, end) -> None:
    """Queue a CUDA event pair; ``kind`` is one of comm_issue / comm_sync / compute."""
    _pending.append((kind, start, end))


def _drain() -> None:
    if not _pending:
        return
    adders = {"comm_issue": add_comm_issue, "comm_sync": add_comm_sync, "compute": add_compute}
    for kind, start, end in _pending:
        end.synchronize()
        adders[kind](start.elapsed_time(end) / 1000.0)
    _pending.clear()


def snapshot() -> dict[str, float]:
    _drain()
    return {"comm_issue": comm_issue, "comm_sync": comm_sync, "compute": compute, "total_runtime": total_runtime}


def print_stats(runtime_total_s: float | None = None) -> None:
    _drain()
    total = comm_issue + comm_sync + compute
    print(f"comm_issue: {comm_issue}, comm_sync: {comm_sync}, compute: {compute}")
    if total > 0:
        print(f"comm_issue: {100 * (comm_issue / total)}%, comm_sync: {100 * (comm_sync / total)}%, "
              f"compute: {100 * (compute / total)}")
    benchmark_total = total_runtime if runtime_total_s is None else float(runtime_total_s)
    if benchmark_total > 0:
        residual = benchmark_total - total
        print(f"total_runtime: {benchmark_total}, accounted: {total}, unaccounted: {residual}")
        print(f"accounted: {100 * (total / benchmark_total)}%, unaccounted: {100 * (residual / benchmark_total)}%")
