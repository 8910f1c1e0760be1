"""``torch.addmm(c, a, b, out=c)`` on DTensors -> stationary distributed GEMM.

``enable(method)`` installs a handler for ``aten.addmm.out`` in DTensor's custom-op
table (the hook point the reference uses, dtensor_mm_handler.py:117-136);
``disable()`` removes it.  The DTensors must come from
``DistMatrix.to_dtensor()`` so that their shards are addressable by peers.
Unlike the reference's handler, this one returns ``out``.
"""
from __future__ import annotations

from typing import Literal

import torch

from ..utils import profile
from . import exec as X
from . import plan as P
from .matrix import resolve

StationaryMethod = Literal["auto", "stationary_c", "stationary_b"]
_stationary_method: str = "auto"
_installed = False


def print_stats(runtime_total_s: float | None = None) -> None:
    profile.print_stats(runtime_total_s=runtime_total_s)


def current_method() -> str:
    return _stationary_method


def _addmm_out_handler(op_call, args, kwargs):
    e, a, b = args[0], args[1], args[2]
    c = kwargs.get("out")
    if c is not e:
        raise RuntimeError("NotImplemented: aten.addmm.out handler requires input and output to alias")
    for name in ("beta", "alpha"):
        if kwargs.get(name, 1) != 1:
            raise RuntimeError(f"aten.addmm.out handler supports {name}=1 only")
    if not all(hasattr(t, "device_mesh") for t in (a, b, c)):
        raise RuntimeError("aten.addmm.out handler expects a, b, and out to be DTensors")
    if not (a.ndim == 2 and b.ndim == 2 and c.ndim == 2):
        raise RuntimeError("aten.addmm.out handler expects a, b, and out to be rank-2 DTensors")
    if a.shape[1] != b.shape[0] or c.shape[0] != a.shape[0] or c.shape[1] != b.shape[1]:
        raise RuntimeError(f"aten.addmm.out handler shape mismatch: a.shape={tuple(a.shape)}, "
                           f"b.shape={tuple(b.shape)}, c.shape={tuple(c.shape)}")
    X.matmul(resolve(a), resolve(b), resolve(c), method=_stationary_method)
    return c


def _table():
    from torch.distributed.tensor import DTensor

    return DTensor._op_dispatcher._custom_op_handlers


def enable(stationary_method: str = "auto") -> None:
    global _stationary_method, _installed
    if stationary_method not in P.STATIONARY_METHODS:
        raise ValueError("stationary_method must be one of: auto, stationary_c, stationary_b")
    _stationary_method = stationary_method
    _table()[torch.ops.aten.addmm.out] = _addmm_out_handler
    _installed = True


def disable() -> None:
    global _stationary_method, _installed
    _stationary_method = "auto"
    if _installed:
        _table().pop(torch.ops.aten.addmm.out, None)
    _installed = False
