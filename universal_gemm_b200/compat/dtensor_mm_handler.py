"""Reference module name ``dtensor_mm_handler``."""
from ..parallel.handler import StationaryMethod, disable, enable, print_stats  # noqa: F401
