"""Reference module name ``accumulate_kernels``: strided ``dst += src`` with atomic adds.

The reference launches a Triton kernel (accumulate_kernels.py:12-60); here it is the sm_100a
``ug_accumulate_2d`` kernel (vector ``red.global.add``), fp32 and bf16.
"""
import torch


def is_available() -> bool:
    return torch.cuda.is_available()


def launch_atomic_add(dst: torch.Tensor, src: torch.Tensor) -> None:
    from ..ops.device import DeviceState, torch_dtype_code

    if dst.shape != src.shape or dst.dim() != 2 or dst.dtype != src.dtype:
        raise ValueError("launch_atomic_add expects two rank-2 tensors of equal shape and dtype")
    if dst.stride(1) != 1:
        raise ValueError("the destination must have unit column stride")
    if src.stride(1) != 1:
        src = src.contiguous()
    DeviceState.get(dst.device).accumulate_2d(dst.data_ptr(), dst.stride(0), src.data_ptr(), src.stride(0),
                                              src.shape[0], src.shape[1], torch_dtype_code(dst.dtype))
