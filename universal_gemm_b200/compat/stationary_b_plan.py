"""Reference module name ``stationary_b_plan``."""
from ..parallel.exec import execute_stationary_b, execute_stationary_b_ops, execute_stationary_b_ops_async  # noqa: F401
from ..parallel.plan import (  # noqa: F401
    MultiplyOp, build_stationary_b_ops, clear_stationary_b_plan_cache, format_stationary_b_op,
    format_stationary_b_plan, validate_op_shapes as _validate_op_shapes,
)
