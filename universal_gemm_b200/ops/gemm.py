"""Single-GPU entry points of the fused GEMM kernel on plain torch tensors.

``gemm`` runs ``C (+)= A @ B`` (bf16 inputs, or fp32 inputs as three bf16 products; fp32 accumulation in TMEM) through the
same persistent tcgen05 kernel the distributed executors use, with one task and
one K segment.  ``segmented_gemm`` exposes K segments and staging for tests.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import native
from .device import DeviceState, torch_dtype_code
from .fused import FusedProgram, FusedProgramBuilder, OperandSlice, TaskSpec


def _slice_of(t: torch.Tensor, *, remote: bool = False) -> OperandSlice:
    if t.dim() != 2 or t.dtype not in (torch.bfloat16, torch.float32) or t.stride(1) != 1:
        raise ValueError("operands must be 2-D bfloat16 or float32 tensors with unit column stride")
    return OperandSlice(base=t.data_ptr(), ld=t.stride(0), row0=0, col0=0, rows=t.shape[0], cols=t.shape[1],
                        remote=remote, elem_bytes=t.element_size())


def _segments(a: OperandSlice, b: OperandSlice) -> list[tuple[OperandSlice, OperandSlice]]:
    """bf16 operands: one product.  fp32 operands: three bf16 products of their high / low parts."""
    if a.elem_bytes != b.elem_bytes:
        raise ValueError("A and B must have the same dtype")
    if a.elem_bytes == 2:
        return [(a, b)]
    from dataclasses import replace

    return [(replace(a, split=2), replace(b, split=1)), (replace(a, split=1), replace(b, split=2)),
            (replace(a, split=1), replace(b, split=1))]


def build_gemm_program(a_parts: Sequence[torch.Tensor], b_parts: Sequence[torch.Tensor], c: torch.Tensor,
                       *, mode: int = native.C_ADD, stage_a: bool = False, stage_b: bool = False,
                       timeout_ns: int = 4_000_000_000, tile_m: int | None = None) -> FusedProgram:
    """``C (+)= sum_i a_parts[i] @ b_parts[i]``; ``stage_*`` forces the in-kernel staged
    copy path for that operand (as if it lived in a peer's memory)."""
    if c.dim() != 2 or c.stride(1) != 1:
        raise ValueError("C must be 2-D with unit column stride")
    state = DeviceState.get(c.device)
    builder = FusedProgramBuilder(c.device, num_sms=state.num_sms, timeout_ns=timeout_ns, tile_m=tile_m)
    segs = [sg for a, b in zip(a_parts, b_parts)
            for sg in _segments(_slice_of(a, remote=stage_a), _slice_of(b, remote=stage_b))]
    builder.add_task(TaskSpec(c_ptr=c.data_ptr(), ldc=c.stride(0), m=c.shape[0], n=c.shape[1], c_mode=mode,
                              c_dtype=torch_dtype_code(c.dtype), segments=segs))
    return builder.build(state.status_ptr)


def run_program(prog: FusedProgram, device: torch.device) -> None:
    state = DeviceState.get(device)
    stream = state.stream()
    if prog.num_clear:
        prog.reset_flags(stream)
        state.launches += 1
    prog.launch(stream)
    state.launches += 1


def gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, *, mode: int = native.C_ADD,
         tile_m: int | None = None) -> torch.Tensor:
    """``C (+)= A @ B`` on one GPU with the tcgen05 kernel.  A: [M, K] bf16, B: [K, N] bf16."""
    prog = build_gemm_program([a], [b], c, mode=mode, tile_m=tile_m)
    run_program(prog, c.device)
    return c
