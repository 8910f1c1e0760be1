"""Reference module name ``dtensor_scratch``: the symmetric bump heap."""
import torch

from ..parallel import runtime as _rt
from ..parallel.symm import SymmHeap


class NvshmemHeap(SymmHeap):
    """``NvshmemHeap(capacity_elements, dtype)`` on the default world (symmetric memory over CUDA IPC / shm)."""

    def __init__(self, capacity_elements: int, dtype: torch.dtype) -> None:
        super().__init__(_rt.default_world(), capacity_elements, dtype)
