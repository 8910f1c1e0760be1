"""Reference module name ``tile_bounds`` -> :mod:`universal_gemm_b200.parallel.tiles`."""
from ..parallel.tiles import Slice1D, Slice2D, grid_shape as _grid_shape, overlapping_tiles, tile_bounds  # noqa: F401
