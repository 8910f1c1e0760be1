"""Build and load ``libugemm_b200.so`` (hand-written sm_100a kernels + host runtime).

The library is compiled in-tree with ``nvcc -gencode arch=compute_100a,code=sm_100a``
and loaded through ctypes, so that it is visible as a file of this package and
needs no Python headers.  ``nvcc`` cross-compiles without a GPU; loading works
without a GPU as well (the CUDA runtime is linked statically and only touches
the driver on first use).

A stamp file next to the library records a hash of the sources and flags; the
library is rebuilt only when that hash changes.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from pathlib import Path

_OPS_DIR = Path(__file__).resolve().parent
_CSRC = _OPS_DIR / "csrc"
_LIB_PATH = _OPS_DIR / "libugemm_b200.so"
_STAMP_PATH = _OPS_DIR / "libugemm_b200.so.stamp"

SOURCES = ("fused_gemm.cu", "fused_gemm_pair.cu", "tile_ops.cu", "barrier.cu", "runtime.cu", "no_alloc.cu")
HEADERS = ("ugemm_b200.h", "ptx_sm100.cuh", "fused_common.cuh", "no_alloc.h")

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
)

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


def _existing(names: tuple[str, ...]) -> list[Path]:
    return [(_CSRC / n) for n in names if (_CSRC / n).exists()]


def _source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in _existing(SOURCES) + _existing(HEADERS):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    default = "/usr/local/cuda/bin/nvcc"
    return default if os.path.exists(default) else None


def needs_build() -> bool:
    if not _LIB_PATH.exists() or not _STAMP_PATH.exists():
        return True
    return _STAMP_PATH.read_text().strip() != _source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``.cu`` source for sm_100a into one shared library."""
    with _lock:
        if not force and not needs_build():
            return _LIB_PATH
        nvcc = find_nvcc()
        if nvcc is None:
            raise RuntimeError("nvcc not found: cannot build libugemm_b200.so")
        tmp = _LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, *NVCC_FLAGS]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", str(tmp), *[str(p) for p in _existing(SOURCES)]]
        proc = subprocess.run(cmd, cwd=str(_CSRC), capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            print(proc.stderr)
        os.replace(tmp, _LIB_PATH)
        _STAMP_PATH.write_text(_source_hash() + "\n")
        return _LIB_PATH


def library_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Return the loaded library, building it first when it is missing or stale."""
    global _lib
    if _lib is not None:
        return _lib
    if needs_build():
        build()
    with _lock:
        if _lib is None:
            _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib
