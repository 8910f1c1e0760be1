"""Modules named like the reference's flat modules, for scripts written against it.

``import universal_gemm_b200.compat.dtensor_utils as dt`` gives the same function names as the reference's
``dtensor_utils`` facade (geometry, scratch, tiles, planners, executors); likewise ``dtensor_mm_handler``,
``dtensor_profile``, ``tile_bounds``, ``stationary_c_plan``, ``stationary_b_plan``, ``dtensor_scratch`` and
``accumulate_kernels``.  ``install()`` additionally registers them in ``sys.modules`` under the bare
reference names so that ``import dtensor_utils`` resolves to this package.
"""
from __future__ import annotations

import importlib
import sys

NAMES = ("tile_bounds", "dtensor_scratch", "dtensor_profile", "accumulate_kernels", "stationary_c_plan",
         "stationary_b_plan", "dtensor_utils", "dtensor_mm_handler")


def install() -> None:
    for name in NAMES:
        sys.modules.setdefault(name, importlib.import_module(f"{__name__}.{name}"))
