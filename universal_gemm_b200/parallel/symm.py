"""Symmetric memory: allocations of equal size on every rank that every rank of the
node can address directly (one-sided loads, stores and atomics).

Three interchangeable *worlds* provide it:

* :class:`CudaIpcWorld` - one process per GPU; ``cudaMalloc`` + legacy CUDA IPC
  handles exchanged through ``torch.distributed``.  Peer pointers are plain device
  addresses the kernels dereference over NVLink.  No multicast object is created.
* :class:`ShmWorld` - CPU ranks (``gloo``); allocations are files under ``/dev/shm``
  mapped by every rank.  Used for the CPU configuration and the multi-process tests.
* :class:`EmulatedCluster` - all ranks inside one process (CPU or one GPU), executed
  one after the other.  The k-th allocation of every rank resolves to the k-th
  allocation of the cluster, so code written for real worlds runs unchanged.

This replaces the NVSHMEM symmetric heap and ``get_peer_tensor`` mappings of the
reference (dtensor_scratch.py:9-53, dtensor_utils.py:30-115,546-552).
"""
from __future__ import annotations

import ctypes
import os
import uuid
import weakref
from typing import Sequence

import torch

_ALIGN = 1024


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


GUARD_BYTE = 0xA5


class GuardViolation(RuntimeError):
    """Something wrote outside a symmetric allocation (into one of its guard regions)."""


class SymmBuffer:
    """One collective allocation as seen from one rank.

    With ``guard`` > 0 the raw allocation is ``guard + nbytes + guard`` bytes: the payload sits between two regions
    filled with ``GUARD_BYTE`` that nothing may touch; ``check_guards`` looks at this rank's copy."""

    def __init__(self, world: "World", nbytes: int, ptrs: Sequence[int], tensors: Sequence[torch.Tensor | None],
                 closer=None, guard: int = 0):
        self.world = world
        self.guard = int(guard)
        self.nbytes = int(nbytes) - 2 * self.guard
        self._ptrs = [int(p) + self.guard for p in ptrs]
        self._raw_local = tensors[world.rank] if self.guard else None
        self._tensors = [t[self.guard:self.guard + self.nbytes] if (t is not None and self.guard) else t for t in tensors]
        self._closer = closer
        self.closed = False
        if self.guard and self._raw_local is not None:
            self._raw_local[:self.guard].fill_(GUARD_BYTE)
            self._raw_local[self.guard + self.nbytes:].fill_(GUARD_BYTE)

    def check_guards(self) -> None:
        """Raise :class:`GuardViolation` if a byte of this rank's guard regions has changed."""
        if not self.guard or self._raw_local is None or self.closed:
            return
        if self._raw_local.is_cuda:
            torch.cuda.synchronize(self._raw_local.device)
        for name, region, base in (("below", self._raw_local[:self.guard], -self.guard),
                                   ("above", self._raw_local[self.guard + self.nbytes:], self.nbytes)):
            bad = (region != GUARD_BYTE).nonzero()
            if bad.numel():
                first = int(bad[0])
                raise GuardViolation(f"rank {self.world.rank}: {int(bad.numel())} guard byte(s) {name} a symmetric "
                                     f"allocation of {self.nbytes} bytes were overwritten, first at payload offset "
                                     f"{base + first}")

    @property
    def local(self) -> torch.Tensor:
        t = self._tensors[self.world.rank]
        assert t is not None
        return t

    def ptr(self, rank: int) -> int:
        """Address of ``rank``'s copy, valid in this process (and on this GPU)."""
        return self._ptrs[rank]

    def tensor(self, rank: int) -> torch.Tensor | None:
        """uint8 tensor over ``rank``'s copy when this world can express it (CPU, emulation, self)."""
        return self._tensors[rank]

    def contains(self, ptr: int, nbytes: int) -> bool:
        return any(base <= ptr and ptr + nbytes <= base + self.nbytes for base in self._ptrs)

    def free(self) -> None:
        if not self.closed and self._closer is not None:
            self._closer()
        self.closed = True


class World:
    rank: int
    size: int
    device: torch.device
    emulated = False

    # Bytes of guard region on each side of every allocation (a multiple of 256 keeps the payload's alignment);
    # 0 = none.  Set per world (``world.guard_bytes = 4096`` before the first allocation, same on every rank) or for
    # all worlds with UGEMM_GUARD_BYTES.  The reference has no sanitizer hook; this is the stand-in for one.
    guard_bytes: int = _round_up(int(os.environ.get("UGEMM_GUARD_BYTES", "0")), 256)

    def alloc(self, nbytes: int) -> SymmBuffer:
        """Collective allocation of ``nbytes`` per rank (plus guard regions when enabled)."""
        guard = _round_up(int(self.guard_bytes), 256) if self.guard_bytes else 0
        buf = self._alloc_raw(_round_up(max(int(nbytes), 1), _ALIGN) + 2 * guard, guard)
        if guard:
            live = self.__dict__.setdefault("_guarded", [])
            live.append(weakref.ref(buf))
        return buf

    def _alloc_raw(self, nbytes: int, guard: int) -> SymmBuffer:
        raise NotImplementedError

    def check_guards(self) -> int:
        """Check the guard regions of every live allocation of this rank; returns how many were checked."""
        n = 0
        for ref in self.__dict__.get("_guarded", []):
            buf = ref()
            if buf is not None and not buf.closed:
                buf.check_guards()
                n += 1
        return n

    def barrier(self) -> None:
        """Host-level barrier across the ranks (collective)."""
        raise NotImplementedError

    def device_barrier(self, clear_ptr: int = 0, num_clear: int = 0) -> int:
        """Stream-ordered barrier across the ranks; returns the number of kernels launched."""
        raise NotImplementedError

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    def close(self) -> None:
        pass


# ----------------------------------------------------------------------------- control-plane communicators
class DistComm:
    """Control plane over a ``torch.distributed`` process group (bootstrap, handle exchange, host barriers)."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self._dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def all_gather(self, obj):
        out: list = [None] * self.size
        self._dist.all_gather_object(out, obj, group=self.group)
        return out

    def barrier(self) -> None:
        self._dist.barrier(group=self.group)


class FileComm:
    """Control plane over a shared directory: no process group needed.

    Every collective writes one small file per rank and polls for the others; a rank that never shows up
    makes the others raise ``TimeoutError`` after ``timeout_s`` instead of hanging.  This is the bootstrap
    the reference does with a unique-id file and a 30 s poll (nvshmem_init_only.py:16-44), extended to all
    handle exchanges and host barriers."""

    def __init__(self, directory: str, rank: int, size: int, timeout_s: float = 30.0, poll_s: float = 0.005):
        self.dir = directory
        self.rank = int(rank)
        self.size = int(size)
        self.timeout_s = float(timeout_s)
        self.poll_s = poll_s
        self.group = None
        self._round = 0
        os.makedirs(directory, exist_ok=True)

    def all_gather(self, obj):
        import pickle
        import time

        k = self._round
        self._round += 1
        mine = os.path.join(self.dir, f"r{k}_{self.rank}.pkl")
        with open(mine + ".tmp", "wb") as f:
            pickle.dump(obj, f)
        os.replace(mine + ".tmp", mine)
        deadline = time.monotonic() + self.timeout_s
        out = []
        for r in range(self.size):
            path = os.path.join(self.dir, f"r{k}_{r}.pkl")
            while not os.path.exists(path):
                if time.monotonic() > deadline:
                    raise TimeoutError(f"rank {r} did not reach collective #{k} within {self.timeout_s:.1f} s")
                time.sleep(self.poll_s)
            with open(path, "rb") as f:
                out.append(pickle.load(f))
        if k >= 2:      # everyone has passed round k-2 once they wrote round k-1... keep the directory small
            try:
                os.unlink(os.path.join(self.dir, f"r{k - 2}_{self.rank}.pkl"))
            except OSError:
                pass
        return out

    def barrier(self) -> None:
        self.all_gather(None)


# ----------------------------------------------------------------------------- CUDA IPC
class _CudaWrapper:
    """Exposes a raw device allocation through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


class CudaIpcWorld(World):
    """One process per GPU of one node; symmetric allocations over CUDA IPC."""

    def __init__(self, group=None, device: torch.device | None = None, timeout_s: float = 10.0, comm=None):
        from ..ops import native
        from ..ops.device import DeviceState

        self.comm = comm if comm is not None else DistComm(group)
        self.group = self.comm.group
        self.rank = self.comm.rank
        self.size = self.comm.size
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self._native = native
        self.state = DeviceState.get(self.device)
        self.timeout_ns = int(timeout_s * 1e9)
        self._buffers: list[SymmBuffer] = []
        # signal slots for the device barrier
        self._signal = self.alloc(_ALIGN)
        self._signal.local.zero_()
        self._slots = torch.tensor([self._signal.ptr(r) for r in range(self.size)], dtype=torch.int64,
                                   device=self.device)
        self._seq = torch.zeros(1, dtype=torch.int32, device=self.device)     # barrier round, advanced on the device
        torch.cuda.synchronize(self.device)
        self.barrier()

    def _alloc_raw(self, nbytes: int, guard: int) -> SymmBuffer:
        native = self._native
        L = native.lib()
        nbytes = _round_up(max(int(nbytes), 1), _ALIGN)
        with torch.cuda.device(self.device):
            ptr = ctypes.c_uint64(0)
            native.check(L.ug_malloc(nbytes, ctypes.byref(ptr)), "ug_malloc")
            handle = (ctypes.c_uint8 * 64)()
            native.check(L.ug_ipc_get_handle(ptr.value, ctypes.cast(handle, ctypes.c_void_p)), "ug_ipc_get_handle")
            mine = (bytes(handle), nbytes)
            gathered = self.comm.all_gather(mine)
            ptrs, opened = [], []
            for r, (h, nb) in enumerate(gathered):
                if nb != nbytes:
                    raise RuntimeError(f"symmetric allocation size differs between ranks: {nb} vs {nbytes}")
                if r == self.rank:
                    ptrs.append(ptr.value)
                    continue
                peer = ctypes.c_uint64(0)
                hb = (ctypes.c_uint8 * 64).from_buffer_copy(h)
                native.check(L.ug_ipc_open(ctypes.cast(hb, ctypes.c_void_p), ctypes.byref(peer)), "ug_ipc_open")
                ptrs.append(peer.value)
                opened.append(peer.value)
            local = torch.as_tensor(_CudaWrapper(ptr.value, nbytes), device=self.device)
        tensors: list[torch.Tensor | None] = [None] * self.size
        tensors[self.rank] = local

        def closer(own=ptr.value, opened=tuple(opened)):
            # Collective: every rank unmaps its peers' memory before any owner frees it (freeing exported
            # memory that an importer still has open is undefined).
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                for p in opened:
                    L.ug_ipc_close(p)
                self.comm.barrier()
                L.ug_free(own)

        buf = SymmBuffer(self, nbytes, ptrs, tensors, closer, guard)
        self._buffers.append(buf)
        return buf

    def barrier(self) -> None:
        self.comm.barrier()

    def device_barrier(self, clear_ptr: int = 0, num_clear: int = 0) -> int:
        L = self._native.lib()
        self._native.check(
            L.ug_signal_barrier(self._slots.data_ptr(), self.size, self.rank, self._seq.data_ptr(),
                                self.state.status_ptr, self.timeout_ns, clear_ptr, num_clear,
                                ctypes.c_void_p(self.state.stream())), "ug_signal_barrier")
        self.state.launches += 1
        return 1

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self.barrier()
        for buf in self._buffers:       # same order on every rank: free() is collective
            buf.free()
        self._buffers.clear()
        self.barrier()


class SymmMemWorld(CudaIpcWorld):
    """One process per GPU; symmetric allocations from ``torch.distributed._symmetric_memory`` (``empty`` +
    ``rendezvous``, CUDA or NVSHMEM backend) instead of raw CUDA IPC.  The kernels see the same thing either way: a
    table of peer pointers.  The role of the reference's ``symm_mem_example.py:23-30`` bring-up.

    torch binds such allocations to an NVLink multicast object where the hardware offers one
    (``multicast_ptr`` below is then non-zero); a rank that dies while bound can disturb its peers, so the
    CUDA-IPC world stays the default and this one is opt-in (``ug.init(world="symm_mem")``)."""

    def __init__(self, group=None, device: torch.device | None = None, timeout_s: float = 10.0, backend: str | None = None):
        import torch.distributed._symmetric_memory as symm_mem

        self._symm_mem = symm_mem
        if backend is not None:
            symm_mem.set_backend(backend)
        self._handles: list = []
        super().__init__(group=group, device=device, timeout_s=timeout_s)

    def _alloc_raw(self, nbytes: int, guard: int) -> SymmBuffer:
        import torch.distributed as dist

        nbytes = _round_up(max(int(nbytes), 1), _ALIGN)
        with torch.cuda.device(self.device):
            local = self._symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            group = self.group if self.group is not None else dist.group.WORLD
            handle = self._symm_mem.rendezvous(local, group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        if len(ptrs) != self.size or ptrs[self.rank] != local.data_ptr():
            raise RuntimeError("symmetric-memory rendezvous returned an unexpected pointer table")
        tensors: list[torch.Tensor | None] = [None] * self.size
        tensors[self.rank] = local
        self._handles.append(handle)

        def closer(handle=handle):
            torch.cuda.synchronize(self.device)
            self.comm.barrier()                 # nobody still reads a peer's memory when the owners let go
            if handle in self._handles:
                self._handles.remove(handle)

        buf = SymmBuffer(self, nbytes, ptrs, tensors, closer, guard)
        buf.multicast_ptr = int(getattr(handle, "multicast_ptr", 0) or 0)
        self._buffers.append(buf)
        return buf


# ----------------------------------------------------------------------------- CPU shared memory
class ShmWorld(World):
    """CPU ranks of one node; allocations are shared files under /dev/shm."""

    def __init__(self, group=None, shm_dir: str = "/dev/shm", comm=None):
        self.comm = comm if comm is not None else DistComm(group)
        self.group = self.comm.group
        self.rank = self.comm.rank
        self.size = self.comm.size
        self.device = torch.device("cpu")
        self._dir = shm_dir
        self._token = self.comm.all_gather(uuid.uuid4().hex[:12])[0]
        self._count = 0
        self._paths: list[str] = []

    def _path(self, index: int, rank: int) -> str:
        return os.path.join(self._dir, f"ugemm_{self._token}_{index}_{rank}")

    def _alloc_raw(self, nbytes: int, guard: int) -> SymmBuffer:
        nbytes = _round_up(max(int(nbytes), 1), _ALIGN)
        index = self._count
        self._count += 1
        mine = self._path(index, self.rank)
        with open(mine, "wb") as f:
            f.truncate(nbytes)
        self._paths.append(mine)
        self.comm.barrier()
        tensors = [torch.from_file(self._path(index, r), shared=True, size=nbytes, dtype=torch.uint8)
                   for r in range(self.size)]
        self.comm.barrier()
        return SymmBuffer(self, nbytes, [t.data_ptr() for t in tensors], tensors, None, guard)

    def barrier(self) -> None:
        self.comm.barrier()

    def device_barrier(self, clear_ptr: int = 0, num_clear: int = 0) -> int:
        self.barrier()
        return 0

    def lock_path(self, rank: int) -> str:
        return os.path.join(self._dir, f"ugemm_{self._token}_lock_{rank}")

    def close(self) -> None:
        self.barrier()
        for p in self._paths:
            try:
                os.unlink(p)
            except OSError:
                pass
        self._paths.clear()
        if self.rank == 0:
            for r in range(self.size):
                try:
                    os.unlink(self.lock_path(r))
                except OSError:
                    pass


# ----------------------------------------------------------------------------- emulation
class EmulatedCluster:
    """``size`` ranks inside this process.  ``cluster.world(r)`` is rank r's view."""

    def __init__(self, size: int, device: torch.device | str = "cpu", guard_bytes: int | None = None):
        self.size = int(size)
        self.device = torch.device(device)
        self._allocs: list[list[torch.Tensor]] = []
        self._worlds = [EmulatedWorld(self, r) for r in range(self.size)]
        if guard_bytes is not None:
            for w in self._worlds:
                w.guard_bytes = int(guard_bytes)

    def check_guards(self) -> int:
        """Check every rank's guard regions; returns the number of allocations checked."""
        return sum(w.check_guards() for w in self._worlds)

    def world(self, rank: int) -> "EmulatedWorld":
        return self._worlds[rank]

    def worlds(self) -> list["EmulatedWorld"]:
        return list(self._worlds)

    def _get(self, index: int, nbytes: int) -> list[torch.Tensor]:
        if index == len(self._allocs):
            self._allocs.append([torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
                                 for _ in range(self.size)])
        tensors = self._allocs[index]
        if tensors[0].numel() != nbytes:
            raise RuntimeError("ranks of an emulated cluster must allocate in the same order and size")
        return tensors


class EmulatedWorld(World):
    emulated = True

    def __init__(self, cluster: EmulatedCluster, rank: int):
        self.cluster = cluster
        self.rank = rank
        self.size = cluster.size
        self.device = cluster.device
        self._count = 0
        self.timeout_ns = 4_000_000_000

    def _alloc_raw(self, nbytes: int, guard: int) -> SymmBuffer:
        nbytes = _round_up(max(int(nbytes), 1), _ALIGN)
        tensors = self.cluster._get(self._count, nbytes)
        self._count += 1
        return SymmBuffer(self, nbytes, [t.data_ptr() for t in tensors], tensors, None, guard)

    def barrier(self) -> None:
        pass

    def device_barrier(self, clear_ptr: int = 0, num_clear: int = 0) -> int:
        # Ranks run one after the other, so only the local clearing part of the barrier remains.
        if num_clear and self.is_cuda:
            from ..ops.device import DeviceState

            DeviceState.get(self.device).zero_2d(clear_ptr, num_clear * 4, 1, num_clear * 4)
            return 1
        return 0


class SingleWorld(EmulatedWorld):
    """A world of one rank (no peers); used on one GPU or one CPU process."""

    def __init__(self, device: torch.device | str = "cpu"):
        super().__init__(EmulatedCluster(1, device), 0)


# ----------------------------------------------------------------------------- bump heap
class SymmHeap:
    """Bump allocator over one symmetric buffer (scratch for fetched tiles).

    Like the reference heap (dtensor_scratch.py:9-53) it wraps around when full;
    unlike it, it refuses to hand out memory that overlaps a view which is still
    registered as live (``release`` ends a view's life).
    """

    def __init__(self, world: World, capacity_elements: int, dtype: torch.dtype):
        if capacity_elements <= 0:
            raise ValueError("capacity_elements must be positive")
        self.world = world
        self.dtype = dtype
        self.itemsize = torch.empty(0, dtype=dtype).element_size()
        self._capacity = int(capacity_elements)
        self.buffer = world.alloc(self._capacity * self.itemsize)
        self._cursor = 0
        self._live: dict[int, tuple[int, int]] = {}

    @property
    def capacity(self) -> int:
        return self._capacity

    def reset(self) -> None:
        self._cursor = 0
        self._live.clear()

    def alloc(self, shape: Sequence[int]) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        if numel == 0:
            return self.buffer.local[:0].view(self.dtype).view(*shape)
        step = _round_up(numel, max(1, 256 // self.itemsize))     # keep every view 256-byte aligned
        if numel > self._capacity:
            raise RuntimeError(f"SymmHeap exhausted: requested={numel} elements, capacity={self._capacity} elements")
        start = self._cursor
        if start + numel > self._capacity:
            start = 0
        end = start + numel
        for lo, hi in self._live.values():
            if lo < end and start < hi:
                raise RuntimeError("SymmHeap wrapped onto a tile that is still in use; release tiles or grow the heap")
        view = self.buffer.local[start * self.itemsize:end * self.itemsize].view(self.dtype).view(*shape)
        self._live[view.data_ptr()] = (start, end)
        self._cursor = min(start + step, self._capacity)
        return view

    def release(self, view: torch.Tensor) -> None:
        self._live.pop(view.data_ptr(), None)

    def close(self) -> None:
        self._live.clear()
        self.buffer.free()
