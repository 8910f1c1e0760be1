"""B200-native universal distributed GEMM.

``C += A @ B`` for matrices partitioned by rows, columns or 2-D blocks (with an
optional replication factor) across the GPUs of one node, using Stationary-B /
Stationary-C plans executed by one persistent tcgen05 kernel per rank that pulls
remote operand tiles and pushes partial results over NVLink.

Typical use (one process per GPU, launched with torchrun)::

    import universal_gemm_b200 as ug
    world = ug.init()                                  # NCCL process group + symmetric memory
    a = ug.distribute_tensor(full_a, world, "row")     # bf16 shards in symmetric memory
    b = ug.distribute_tensor(full_b, world, "column")
    c = ug.zeros(world, (m, n), "row")                 # fp32 accumulator
    ug.matmul(a, b, c, method="auto")                  # stream-ordered, no host sync
    ug.check_status()                                  # raises if a kernel reported an error
"""
from __future__ import annotations

__version__ = "0.1.0"

from .parallel.tiles import (  # noqa: F401
    Layout, Partial, Replicate, Shard, Slice1D, Slice2D, grid_shape, intersect_1d, intersect_2d, matrix_numel,
    my_replica, overlapping_tiles, replication_factor, subtract_offset, tile_bounds, tile_offset, tile_rank,
    tile_shape,
)
from .parallel.partition import (  # noqa: F401
    Partitioning, closest_factors, column_partitioning, get_nprocs_from_env, get_partitioning, get_rank_from_env,
    materialized_placements, one_dimensional_partitioning, row_partitioning, two_dimensional_partitioning,
)
from .parallel.plan import (  # noqa: F401
    MultiplyOp, build_stationary_b_ops, build_stationary_c_ops, clear_plan_cache, clear_stationary_b_plan_cache,
    clear_stationary_c_plan_cache, format_op, format_plan, format_stationary_b_op, format_stationary_b_plan,
    group_ops, plan_traffic, select_method,
)
from .parallel.symm import (  # noqa: F401
    CudaIpcWorld, DistComm, EmulatedCluster, FileComm, GuardViolation, ShmWorld, SingleWorld, SymmHeap, SymmMemWorld, World,
)
from .parallel.matrix import DistMatrix, distribute_tensor, empty, resolve, zeros  # noqa: F401
from .parallel.runtime import (  # noqa: F401
    accumulate_tile, clear_peer_tensor_cache, default_world, free_get_tile_scratch, get_tile, get_tile_async,
    init_scratch, put_tile, redistribute, reduce_replicas, reduce_replicas_async, release_tile, set_default_world, tile, SignalPad,
)
from .parallel.exec import (  # noqa: F401
    execute_stationary_b, execute_stationary_b_ops, execute_stationary_b_ops_async, execute_stationary_c,
    execute_stationary_c_ops, execute_stationary_c_ops_async, matmul, row_partitioned_matmul,
)
from .parallel.prepared import MatmulPlan, prepare_matmul  # noqa: F401
from .parallel import handler as mm_handler  # noqa: F401
from .utils import profile, trace  # noqa: F401


def init(backend: str | None = None, device=None, timeout_s: float = 10.0, world: str | None = None) -> World:
    """Create the world for this process and make it the default.

    Under ``torchrun`` (``RANK`` / ``WORLD_SIZE`` set) this initialises ``torch.distributed``
    (``nccl`` when CUDA is available, else ``gloo``) and returns a :class:`CudaIpcWorld` or
    :class:`ShmWorld`; without a launcher it returns a single-rank world.  ``world="symm_mem"`` (or
    ``UGEMM_WORLD=symm_mem``) takes the symmetric allocations from torch's symmetric memory instead of CUDA IPC.
    """
    import os

    import torch
    import torch.distributed as dist

    use_cuda = torch.cuda.is_available() if device is None else torch.device(device).type == "cuda"
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        if use_cuda:
            local = int(os.environ.get("LOCAL_RANK", os.environ["RANK"])) % max(torch.cuda.device_count(), 1)
            torch.cuda.set_device(local)
        if not dist.is_initialized():
            if use_cuda:
                dist.init_process_group(backend or "nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
            else:
                dist.init_process_group(backend or "gloo")
        kind = world or os.environ.get("UGEMM_WORLD", "")
        if use_cuda and kind == "symm_mem":
            made: World = SymmMemWorld(timeout_s=timeout_s)
        else:
            made = CudaIpcWorld(timeout_s=timeout_s) if use_cuda else ShmWorld()
    else:
        made = SingleWorld(torch.device("cuda", torch.cuda.current_device()) if use_cuda else "cpu")
    set_default_world(made)
    return made


def check_status(device=None) -> None:
    """Raise ``KernelStatusError`` if a kernel on ``device`` reported an error since the last check."""
    from .ops.device import DeviceState

    DeviceState.get(device).check()
