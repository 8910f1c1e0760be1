"""Reference module name ``dtensor_utils``: the facade with geometry, scratch, tile and executor functions."""
from ..parallel.tiles import (  # noqa: F401
    Slice1D, Slice2D, grid_shape, intersect_1d, intersect_2d, matrix_numel, my_replica, overlapping_tiles,
    replication_factor, subtract_offset, tile_bounds, tile_offset, tile_rank, tile_shape,
)
from ..parallel.runtime import (  # noqa: F401
    accumulate_tile, clear_peer_tensor_cache, free_get_tile_scratch, get_tile, get_tile_async, init_scratch,
    reduce_replicas, reduce_replicas_async, release_tile, tile,
)
from ..parallel.plan import (  # noqa: F401
    MultiplyOp, build_stationary_b_ops, build_stationary_c_ops, format_op, format_plan, format_stationary_b_op,
    format_stationary_b_plan,
)
from ..parallel.exec import (  # noqa: F401
    execute_stationary_b, execute_stationary_b_ops, execute_stationary_b_ops_async, execute_stationary_c,
    execute_stationary_c_ops, execute_stationary_c_ops_async,
)
