"""ctypes bindings of ``libugemm_b200.so`` and numpy mirrors of its table structs.

The structs follow ``csrc/ugemm_b200.h`` field by field; ``check_layouts`` asserts the
sizes so that a drift between the header and this file fails at import of the ops.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p, c_char_p, POINTER

import numpy as np

from . import build as _build

BM, BN, BK = 128, 256, 64

OK = 0
ERR_TIMEOUT_MBAR = 1
ERR_TIMEOUT_FLAG = 2
ERR_TIMEOUT_PEER = 3
ERR_BAD_TABLE = 4

STATUS_NAMES = {
    OK: "ok",
    ERR_TIMEOUT_MBAR: "an mbarrier wait inside the fused kernel timed out",
    ERR_TIMEOUT_FLAG: "a staged-chunk wait inside the fused kernel timed out",
    ERR_TIMEOUT_PEER: "a cross-rank signal wait timed out (a peer never arrived)",
    ERR_BAD_TABLE: "a work-table entry failed an in-kernel bounds check",
}

# C output modes of a task.
C_ADD = 0        # C += acc with plain loads / stores (this rank is the only writer)
C_ATOMIC = 1     # red.add (C may be a peer's memory, or several ranks add into it)
C_STORE = 2      # C = acc

DT_F32 = 0
DT_BF16 = 1

SEGMENT_DTYPE = np.dtype(
    [
        ("a_map", "<i4"), ("b_map", "<i4"),
        ("a_row0", "<i4"), ("a_col0", "<i4"),
        ("b_row0", "<i4"), ("b_col0", "<i4"),
        ("k_len", "<i4"),
        ("a_flag", "<i4"), ("b_flag", "<i4"),
        ("pad", "<i4", (7,)),
    ],
    align=False,
)

TASK_DTYPE = np.dtype(
    [
        ("c_ptr", "<u8"), ("ldc", "<i8"),
        ("m", "<i4"), ("n", "<i4"),
        ("seg_begin", "<i4"), ("seg_count", "<i4"),
        ("tile_begin", "<i4"),
        ("m_tiles", "<i4"), ("n_tiles", "<i4"),
        ("kblocks", "<i4"),
        ("c_mode", "<i4"), ("c_dtype", "<i4"), ("c_vec", "<i4"),
        ("group_m", "<i4"),
    ],
    align=False,
)

PIECE_DTYPE = np.dtype(
    [
        ("src", "<u8"), ("dst", "<u8"),
        ("src_ld", "<i8"), ("dst_ld", "<i8"),
        ("rows", "<i4"), ("row_bytes", "<i4"),
        ("flag", "<i4"), ("mode", "<i4"),
    ],
    align=False,
)


class FusedParams(ctypes.Structure):
    _fields_ = [
        ("maps", c_uint64), ("tasks", c_uint64), ("segs", c_uint64), ("pieces", c_uint64),
        ("flags", c_uint64), ("flag_need", c_uint64), ("piece_counter", c_uint64), ("status", c_uint64),
        ("num_maps", c_int32), ("num_tasks", c_int32), ("num_pieces", c_int32), ("num_flags", c_int32),
        ("total_tiles", c_int32), ("tile_m", c_int32),
        ("timeout_ns", c_uint64),
        ("num_segs", c_int32), ("cta_pair", c_int32),
        ("trace", c_uint64), ("trace_slots", c_int32), ("epi_poll_ns", c_int32),
        ("sched", c_uint64),
        ("fetch_depth", c_int32), ("reserved0", c_int32),
        ("checksum", c_uint64),
    ]


TRACE_FIELDS = 16     # uint64 words per timeline record (UG_TR_FIELDS)


def check_layouts() -> None:
    assert SEGMENT_DTYPE.itemsize == 64, SEGMENT_DTYPE.itemsize
    assert TASK_DTYPE.itemsize == 64, TASK_DTYPE.itemsize
    assert PIECE_DTYPE.itemsize == 48, PIECE_DTYPE.itemsize
    assert ctypes.sizeof(FusedParams) == 144, ctypes.sizeof(FusedParams)


check_layouts()

_configured = False


def lib() -> ctypes.CDLL:
    """Load the library (building when stale) and declare the signatures once."""
    global _configured
    L = _build.load()
    if _configured:
        return L
    L.ug_version.restype = c_int
    L.ug_last_error.restype = c_char_p
    L.ug_malloc.argtypes = [c_uint64, POINTER(c_uint64)]
    L.ug_free.argtypes = [c_uint64]
    L.ug_ipc_get_handle.argtypes = [c_uint64, c_void_p]
    L.ug_ipc_open.argtypes = [c_void_p, POINTER(c_uint64)]
    L.ug_ipc_close.argtypes = [c_uint64]
    L.ug_encode_tensor_map.argtypes = [c_void_p, c_uint64, c_int, c_uint64, c_uint64, c_uint64, c_uint32,
                                       c_uint32, c_int]
    L.ug_fused_gemm.argtypes = [POINTER(FusedParams), c_int, c_void_p]
    L.ug_fused_gemm_smem_bytes.restype = c_int
    L.ug_fused_gemm_pair.argtypes = [POINTER(FusedParams), c_int, c_void_p]
    L.ug_fused_gemm_pair.restype = c_int
    L.ug_fused_gemm_pair_max_pairs.restype = c_int
    L.ug_signal_barrier.argtypes = [c_uint64, c_int, c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int,
                                    c_void_p]
    L.ug_zero_2d.argtypes = [c_uint64, c_int64, c_int32, c_int64, c_void_p]
    L.ug_signal_add.argtypes = [c_uint64, c_uint32, c_void_p]
    L.ug_signal_wait.argtypes = [c_uint64, c_uint32, c_uint64, c_uint64, c_void_p]
    L.ug_pull_2d.argtypes = [c_uint64, c_int64, c_uint64, c_int64, c_int32, c_int64, c_int32, c_void_p]
    L.ug_accumulate_2d.argtypes = [c_uint64, c_int64, c_uint64, c_int64, c_int32, c_int32, c_int32, c_void_p]
    L.ug_convert_2d.argtypes = [c_uint64, c_int64, c_int32, c_uint64, c_int64, c_int32, c_int32, c_int32,
                                c_void_p]
    for name in ("ug_malloc", "ug_free", "ug_ipc_get_handle", "ug_ipc_open", "ug_ipc_close",
                 "ug_encode_tensor_map", "ug_fused_gemm", "ug_signal_barrier", "ug_signal_add", "ug_signal_wait", "ug_zero_2d", "ug_pull_2d",
                 "ug_accumulate_2d", "ug_convert_2d"):
        getattr(L, name).restype = c_int
    _configured = True
    return L


class CudaCallError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        detail = lib().ug_last_error()
        detail = detail.decode() if detail else ""
        raise CudaCallError(f"{what} failed with CUDA error {code}. {detail}")


def encode_tensor_map(base: int, dtype: int, inner: int, outer: int, row_stride_bytes: int, box_inner: int,
                      box_outer: int, swizzle: int = 3) -> bytes:
    """Encode one 2-D tiled TMA descriptor and return its 128 bytes.

    The host-side checks repeat what the hardware requires and the driver does not
    all verify: 16-byte aligned base and row pitch, and an inner box that is a
    multiple of 16 bytes.
    """
    elem = 4 if dtype == DT_F32 else 2
    if base % 16:
        raise ValueError(f"TMA base address {base:#x} is not 16-byte aligned")
    if row_stride_bytes % 16:
        raise ValueError(f"TMA row pitch {row_stride_bytes} is not a multiple of 16 bytes")
    if (box_inner * elem) % 16:
        raise ValueError("TMA inner box extent must be a multiple of 16 bytes")
    if inner <= 0 or outer <= 0:
        raise ValueError(f"TMA extents must be positive, got {(inner, outer)}")
    buf = (ctypes.c_uint8 * 128)()
    code = lib().ug_encode_tensor_map(ctypes.cast(buf, c_void_p), base, dtype, inner, outer, row_stride_bytes,
                                      box_inner, box_outer, swizzle)
    check(code, "ug_encode_tensor_map")
    return bytes(buf)
