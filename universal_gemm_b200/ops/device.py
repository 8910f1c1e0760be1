"""Per-device state shared by all launches: the status word the kernels report
errors into, and helpers that wrap the small tile kernels.

A kernel never traps: a wait that runs out stores an error code in the status
word and returns.  ``DeviceState.check`` reads the word back (synchronising the
stream) and raises ``KernelStatusError`` so the CUDA context stays usable.
"""
from __future__ import annotations

import ctypes

import torch

from . import native


class KernelStatusError(RuntimeError):
    def __init__(self, code: int):
        self.code = code
        super().__init__(f"kernel reported status {code}: {native.STATUS_NAMES.get(code, 'unknown error')}")


def require_cuda_extension(device: torch.device) -> None:
    """Fail loudly when the native library is missing on a machine with a GPU."""
    if torch.device(device).type != "cuda":
        raise RuntimeError("the sm_100a kernels need a CUDA device")
    native.lib()


class DeviceState:
    _instances: dict[int, "DeviceState"] = {}

    def __init__(self, device: torch.device):
        self.device = torch.device(device)
        require_cuda_extension(self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        props = torch.cuda.get_device_properties(self.device)
        self.num_sms = props.multi_processor_count
        self.launches = 0          # kernels of this library launched through this object

    @classmethod
    def get(cls, device: torch.device | int | None = None) -> "DeviceState":
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        device = torch.device(device)
        index = device.index if device.index is not None else torch.cuda.current_device()
        inst = cls._instances.get(index)
        if inst is None:
            inst = cls(torch.device("cuda", index))
            cls._instances[index] = inst
        return inst

    @property
    def status_ptr(self) -> int:
        return self.status.data_ptr()

    def stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def read_status(self) -> int:
        return int(self.status[0].item())

    def clear_status(self) -> None:
        self.status.zero_()

    def check(self) -> None:
        code = self.read_status()
        if code != native.OK:
            self.clear_status()
            raise KernelStatusError(code)

    # ---------------------------------------------------------------- tile kernels
    def zero_2d(self, ptr: int, ld_bytes: int, rows: int, row_bytes: int) -> None:
        native.check(native.lib().ug_zero_2d(ptr, ld_bytes, rows, row_bytes, ctypes.c_void_p(self.stream())),
                     "ug_zero_2d")
        self.launches += 1

    def pull_2d(self, dst: int, dst_ld_bytes: int, src: int, src_ld_bytes: int, rows: int, row_bytes: int,
                elem_bytes: int) -> None:
        native.check(native.lib().ug_pull_2d(dst, dst_ld_bytes, src, src_ld_bytes, rows, row_bytes, elem_bytes,
                                             ctypes.c_void_p(self.stream())), "ug_pull_2d")
        self.launches += 1

    def accumulate_2d(self, dst: int, dst_ld: int, src: int, src_ld: int, rows: int, cols: int, dtype: int) -> None:
        native.check(native.lib().ug_accumulate_2d(dst, dst_ld, src, src_ld, rows, cols, dtype,
                                                   ctypes.c_void_p(self.stream())), "ug_accumulate_2d")
        self.launches += 1

    def convert_2d(self, dst: int, dst_ld: int, dst_dtype: int, src: int, src_ld: int, src_dtype: int, rows: int,
                   cols: int) -> None:
        native.check(native.lib().ug_convert_2d(dst, dst_ld, dst_dtype, src, src_ld, src_dtype, rows, cols,
                                                ctypes.c_void_p(self.stream())), "ug_convert_2d")
        self.launches += 1


def torch_dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return native.DT_F32
    if dtype == torch.bfloat16:
        return native.DT_BF16
    raise TypeError(f"unsupported dtype {dtype}; the kernels handle float32 and bfloat16")
