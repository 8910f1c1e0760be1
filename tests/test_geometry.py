"""Tile geometry and partition helpers (CPU)."""
import numpy as np
import pytest

import universal_gemm_b200 as ug
from universal_gemm_b200.parallel import tiles as T
from universal_gemm_b200.parallel.partition import get_partitioning, materialized_placements


def test_slice_validation():
    with pytest.raises(ValueError):
        ug.Slice1D(3, 2)
    with pytest.raises(ValueError):
        ug.Slice1D(-1, 2)
    s = ug.Slice2D(ug.Slice1D(1, 4), ug.Slice1D(0, 2))
    assert s.shape == (3, 2) and s.as_slices() == (slice(1, 4), slice(0, 2))


def test_closest_factors():
    assert ug.closest_factors(8) == (4, 2)
    assert ug.closest_factors(4) == (2, 2)
    assert ug.closest_factors(2) == (2, 1)
    assert ug.closest_factors(1) == (1, 1)
    assert ug.closest_factors(7) == (7, 1)


def test_row_partition_geometry():
    lay = ug.row_partitioning(1, 8).layout((8192, 8192))
    assert ug.grid_shape(lay) == (8, 1)
    assert ug.tile_shape(lay) == (1024, 8192)
    assert ug.tile_bounds(lay, (3, 0)).rows == ug.Slice1D(3072, 4096)
    assert [ug.tile_rank(lay, (i, 0), rank=0) for i in range(8)] == list(range(8))
    assert ug.replication_factor(lay) == 1 and ug.my_replica(lay, rank=5) == 0


def test_block_partition_mesh_matches_reference_layout():
    p = ug.two_dimensional_partitioning(world_size=8)
    assert p.mesh.tolist() == [[0, 1], [2, 3], [4, 5], [6, 7]]
    lay = p.layout((8192, 8192))
    assert ug.grid_shape(lay) == (4, 2) and ug.tile_shape(lay) == (2048, 4096)
    assert ug.tile_rank(lay, (2, 1), rank=0) == 5
    assert T.local_tile_coord(lay, 5) == (2, 1)


def test_block_partition_single_rank_is_valid():
    lay = ug.two_dimensional_partitioning(world_size=1).layout((10, 12))
    assert ug.grid_shape(lay) == (1, 1) and ug.tile_shape(lay, (0, 0)) == (10, 12)


def test_replication_meshes():
    p = ug.row_partitioning(2, 8)
    assert p.mesh.tolist() == [[0, 1, 2, 3], [4, 5, 6, 7]]
    lay = p.layout((8192, 8192))
    assert ug.replication_factor(lay) == 2 and ug.grid_shape(lay) == (4, 1)
    assert ug.my_replica(lay, rank=5) == 1
    assert ug.tile_rank(lay, (1, 0), replica=0, rank=5) == 1
    assert ug.tile_rank(lay, (1, 0), rank=5) == 5
    full = ug.row_partitioning(8, 8)
    assert full.mesh.ndim == 1 and ug.replication_factor(full.layout((4, 4))) == 8
    blk = ug.two_dimensional_partitioning(replication_factor=2, world_size=8)
    assert blk.mesh.shape == (2, 2, 2) and ug.grid_shape(blk.layout((64, 64))) == (2, 2)
    with pytest.raises(RuntimeError):
        ug.row_partitioning(3, 8)


def test_empty_trailing_tiles_are_empty_not_errors():
    lay = ug.row_partitioning(1, 8).layout((9, 5))      # ceil(9/8) = 2 rows per tile -> tiles 5..7 empty
    assert ug.tile_shape(lay, (4, 0)) == (1, 5)
    assert ug.tile_shape(lay, (5, 0)) == (0, 5)
    assert ug.tile_bounds(lay, (7, 0)).rows == ug.Slice1D(9, 9)


def test_overlapping_tiles_and_clamping():
    lay = ug.two_dimensional_partitioning(world_size=8).layout((100, 50))   # tiles 25 x 25
    region = ug.Slice2D(ug.Slice1D(20, 60), ug.Slice1D(24, 200))
    assert ug.overlapping_tiles(lay, region) == [(0, 0), (0, 1), (1, 0), (1, 1), (2, 0), (2, 1)]
    assert ug.overlapping_tiles(lay, ug.Slice2D(ug.Slice1D(5, 5), ug.Slice1D(0, 10))) == []


def test_tiles_cover_matrix_exactly():
    for world in (1, 2, 4, 8):
        for part in ("row", "col", "block"):
            lay = get_partitioning(part, 1, world).layout((37, 29))
            cover = np.zeros((37, 29), dtype=int)
            gr, gc = ug.grid_shape(lay)
            owners = set()
            for i in range(gr):
                for j in range(gc):
                    b = ug.tile_bounds(lay, (i, j))
                    cover[b.rows.as_slice(), b.cols.as_slice()] += 1
                    owners.add(ug.tile_rank(lay, (i, j), rank=0))
            assert (cover == 1).all()
            assert owners == set(range(world))


def test_materialized_placements():
    has, out = materialized_placements([ug.Partial(), ug.Shard(1)])
    assert has and out == [ug.Shard(0), ug.Shard(1)]
    has, out = materialized_placements([ug.Shard(0)])
    assert not has and out == [ug.Shard(0)]
    has, out = materialized_placements([ug.Partial()])
    assert has and out == [ug.Shard(0)]


def test_dtensor_layout_roundtrip():
    import torch
    import torch.distributed as dist
    from torch.testing._internal.distributed.fake_pg import FakeStore

    dist.init_process_group("fake", rank=3, world_size=8, store=FakeStore())
    try:
        mesh, placements = ug.two_dimensional_partitioning(replication_factor=2).to_torch("cpu")
        from torch.distributed.tensor import DTensor

        dt = DTensor.from_local(torch.zeros(4, 4), mesh, placements, run_check=False, shape=torch.Size((8, 8)),
                                stride=(8, 1))
        assert ug.grid_shape(dt) == (2, 2) and ug.replication_factor(dt) == 2
        assert ug.my_replica(dt) == 0 and ug.tile_rank(dt, (1, 1)) == 3
    finally:
        dist.destroy_process_group()
