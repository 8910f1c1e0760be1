"""Partition helpers in the form the torch DTensor API wants: ``(DeviceMesh, placements)``.

Thin adapters over ``universal_gemm_b200.parallel.partition`` (which works without a process
group); used by the plain-DTensor method of the benchmark worker and by user scripts written
against the reference's ``benchmark/util.py``.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from universal_gemm_b200.parallel import partition as _p  # noqa: E402
from universal_gemm_b200.parallel.partition import (  # noqa: E402,F401
    closest_factors, get_nprocs_from_env, get_rank_from_env,
)

DEVICE_TYPE = "cuda"


def materialized_placements(device_mesh, placements):
    return _p.materialized_placements(placements)


def one_dimensional_partitioning(dimension="row", replication_factor=1, mesh_type=DEVICE_TYPE):
    return _p.one_dimensional_partitioning(dimension, replication_factor).to_torch(mesh_type)


def row_partitioning(replication_factor=1, mesh_type=DEVICE_TYPE):
    return _p.row_partitioning(replication_factor).to_torch(mesh_type)


def column_partitioning(replication_factor=1, mesh_type=DEVICE_TYPE):
    return _p.column_partitioning(replication_factor).to_torch(mesh_type)


def two_dimensional_partitioning(process_grid=None, replication_factor=1, mesh_type=DEVICE_TYPE):
    return _p.two_dimensional_partitioning(process_grid, replication_factor).to_torch(mesh_type)


def get_partitioning(partition, replication_factor=1, mesh_type=DEVICE_TYPE):
    return _p.get_partitioning(partition, replication_factor).to_torch(mesh_type)
