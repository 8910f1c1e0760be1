"""Import stubs that let the reference's benchmark worker be imported on a stock PyTorch image.

The reference imports ``nvshmem.core`` (nvshmem4py) and ``cuda.core.experimental`` at module
level; neither is installed here.  Its plain-DTensor method (``--method dtensor``) never calls
into them, so empty stand-ins are enough to run that method's stock code path unmodified.
Calling any NVSHMEM entry point raises, which keeps the stationary methods honest: they are
reported as unavailable instead of being emulated by this repository's own engine.
"""
from __future__ import annotations

import sys
import types


class _Unavailable:
    def __init__(self, name: str):
        self._name = name

    def __call__(self, *a, **k):
        raise RuntimeError(f"{self._name} is not available on this image (nvshmem4py / cuda.core are not installed)")

    def __getattr__(self, item):
        if item.startswith("__"):
            raise AttributeError(item)
        return _Unavailable(f"{self._name}.{item}")


def install() -> None:
    if "nvshmem.core" not in sys.modules:
        nv = types.ModuleType("nvshmem")
        core = types.ModuleType("nvshmem.core")
        nv_types = types.ModuleType("nvshmem.core.nvshmem_types")
        nv_types.NvshmemStream = object
        core.nvshmem_types = nv_types

        def _core_getattr(name: str):
            if name.startswith("__"):
                raise AttributeError(name)
            return _Unavailable(f"nvshmem.core.{name}")

        core.__getattr__ = _core_getattr  # type: ignore[attr-defined]
        nv.core = core
        sys.modules.update({"nvshmem": nv, "nvshmem.core": core, "nvshmem.core.nvshmem_types": nv_types})
    try:
        import cuda.core.experimental  # noqa: F401
    except Exception:
        import cuda  # the cuda-python namespace exists; only cuda.core is missing

        ccore = types.ModuleType("cuda.core")
        exp = types.ModuleType("cuda.core.experimental")
        exp.Device = _Unavailable("cuda.core.experimental.Device")
        st = types.ModuleType("cuda.core.experimental._stream")
        st.Stream = object
        mem = types.ModuleType("cuda.core.experimental._memory")
        mem.Buffer = _Unavailable("cuda.core.experimental._memory.Buffer")
        ccore.experimental = exp
        cuda.core = ccore
        sys.modules.update({"cuda.core": ccore, "cuda.core.experimental": exp,
                            "cuda.core.experimental._stream": st, "cuda.core.experimental._memory": mem})
