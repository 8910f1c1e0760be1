"""Hand-written sm_100a kernels and their host-side lowering."""
from . import native  # noqa: F401
from .build import build as build_native, library_path  # noqa: F401
