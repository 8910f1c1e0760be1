"""Reference module name ``stationary_c_plan``."""
from ..parallel.exec import execute_stationary_c, execute_stationary_c_ops, execute_stationary_c_ops_async  # noqa: F401
from ..parallel.plan import (  # noqa: F401
    MultiplyOp, build_stationary_c_ops, clear_stationary_c_plan_cache, format_op, format_plan,
    validate_op_shapes as _validate_op_shapes,
)
