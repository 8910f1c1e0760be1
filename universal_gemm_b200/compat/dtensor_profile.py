"""Reference module name ``dtensor_profile``: the same counters and report."""
from ..utils.profile import (  # noqa: F401
    add_comm_issue, add_comm_sync, add_compute, add_total_runtime, print_stats, reset_stats, set_total_runtime,
)
from ..utils import profile as _p


def __getattr__(name):          # live counter values: comm_issue, comm_sync, compute, total_runtime
    if name in ("comm_issue", "comm_sync", "compute", "total_runtime"):
        return getattr(_p, name)
    raise AttributeError(name)
