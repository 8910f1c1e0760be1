"""Host-side lowering logic that needs no GPU: tile raster, tile-variant model, tail splitting."""
import pytest

from universal_gemm_b200.ops import native
from universal_gemm_b200.ops.fused import FusedProgramBuilder, OperandSlice, TaskSpec, tile_coords_for_test


def _task(m, n, k, *, remote=False, mode=native.C_STORE):
    return TaskSpec(c_ptr=4096, ldc=n, m=m, n=n, c_mode=mode, c_dtype=native.DT_F32,
                    segments=[(OperandSlice(1024, k, 0, 0, m, k), OperandSlice(2048, n, 0, 0, k, n))], c_remote=remote)


def _locate(row, idx):
    """The kernels' raster formula (fused_common.cuh: locate)."""
    gm = row["group_m"] if row["group_m"] > 0 else row["m_tiles"]
    band_tiles = gm * row["n_tiles"]
    band = idx // band_tiles
    first_m = band * gm
    band_m = min(gm, row["m_tiles"] - first_m)
    rem = idx - band * band_tiles
    return first_m + rem % band_m, rem // band_m


@pytest.mark.parametrize("m_tiles,n_tiles,group_m", [(1, 7, 1), (8, 24, 8), (20, 5, 8), (33, 3, 16)])
def test_host_raster_matches_kernel_formula(m_tiles, n_tiles, group_m):
    row = {"m_tiles": m_tiles, "n_tiles": n_tiles, "group_m": group_m}
    coords = tile_coords_for_test([row])
    assert len(coords) == m_tiles * n_tiles and len(set(coords)) == len(coords)
    for idx, (t, mt, nt) in enumerate(coords):
        assert t == 0 and (mt, nt) == _locate(row, idx)


def test_tile_variant_model_prefers_hidden_epilogue_for_remote_c():
    b = FusedProgramBuilder("cpu", num_sms=148)
    for _ in range(8):
        b.add_task(_task(1024, 6144, 12288, remote=True))
    assert b.choose_tile_m() in (128, "pair")            # never the variant whose epilogue is exposed
    small = FusedProgramBuilder("cpu", num_sms=148)
    small.add_task(_task(300, 200, 157))
    assert small.choose_tile_m() == 128
    forced = FusedProgramBuilder("cpu", num_sms=148, tile_m=256)
    forced.add_task(_task(300, 200, 157))
    assert forced.choose_tile_m() == 256
    with pytest.raises(ValueError):
        FusedProgramBuilder("cpu", num_sms=148, tile_m=192)


def test_tail_split_keeps_coverage_and_halves_the_last_wave():
    tasks = [_task(1024, 6144, 12288) for _ in range(8)]        # 8 x 96 = 768 tiles of 256 x 256 on 74 workers
    out = FusedProgramBuilder._split_tail(tasks, 256, 74)
    assert len(out) == 9 and [t.tile_n for t in out] == [256] * 8 + [128]
    left, right = out[-2], out[-1]
    assert left.n + right.n == 6144 and right.n == 7 * 256      # 28 tail tiles = 7 tile columns x 4 tile rows
    assert right.c_ptr == left.c_ptr + left.n * 4
    assert right.segments[0][1].col0 == left.n and right.segments[0][1].cols == right.n
    tiles = sum(((t.m + 255) // 256) * ((t.n + t.tile_n - 1) // t.tile_n) for t in out)
    assert tiles == 740 + 56
    # no split when the tail is more than half a wave, when there is less than one wave, or with several raster bands
    assert FusedProgramBuilder._split_tail([_task(256, 6144, 64) for _ in range(8)], 256, 74) \
        == [_task(256, 6144, 64) for _ in range(8)]
    assert len(FusedProgramBuilder._split_tail([_task(512, 512, 64)], 256, 74)) == 1
    assert len(FusedProgramBuilder._split_tail([_task(8192, 49152, 64)], 256, 74)) == 1


def test_add_task_validates_shapes():
    b = FusedProgramBuilder("cpu", num_sms=4)
    bad = _task(128, 256, 64)
    bad.segments = [(OperandSlice(0, 64, 0, 0, 128, 64), OperandSlice(0, 256, 0, 0, 32, 256))]
    with pytest.raises(ValueError):
        b.add_task(bad)
    b.add_task(TaskSpec(c_ptr=0, ldc=8, m=0, n=8, c_mode=0, c_dtype=0, segments=[]))     # empty tasks are dropped
    assert b.tasks == []


def test_operand_alignment_rules():
    ok = OperandSlice(base=4096, ld=128, row0=3, col0=8, rows=10, cols=20)
    assert ok.tma_ok() and ok.vector_ok() and ok.address(1, 2) == 4096 + ((3 + 1) * 128 + 8 + 2) * 2
    assert not OperandSlice(base=4096, ld=128, row0=0, col0=3, rows=1, cols=8).tma_ok()        # odd column start
    assert not OperandSlice(base=4096, ld=100, row0=0, col0=0, rows=1, cols=8).tma_ok()        # pitch not 16 B
    assert not OperandSlice(base=4096, ld=128, row0=0, col0=0, rows=1, cols=8, remote=True).tma_ok()
    assert OperandSlice(base=4096, ld=128, row0=0, col0=0, rows=1, cols=8, remote=True).vector_ok()


def test_tail_split_of_wide_pair_tiles():
    """256 x 512 tiles: 82 tiles on 74 pairs leave 8 tail tiles = 4 trailing tile columns of 2 tile rows, re-cut to 256."""
    from dataclasses import replace

    tasks = [replace(_task(512, 41 * 512, 128), tile_n=512)]
    out = FusedProgramBuilder._split_tail(tasks, 256, 74, 512)
    assert [t.tile_n for t in out] == [512, 256]
    assert out[0].n == 37 * 512 and out[1].n == 4 * 512 and out[1].c_ptr == out[0].c_ptr + out[0].n * 4
    tiles = sum(((t.m + 255) // 256) * ((t.n + t.tile_n - 1) // t.tile_n) for t in out)
    assert tiles == 74 + 16


def test_tile_variant_model_long_k_prefers_the_256_row_tile_locally():
    """Local C, long K: the exposed epilogue of the 256-row tile costs less than the pair tile's slower main loop;
    with few K blocks per tile the hidden epilogue wins."""
    long_k = FusedProgramBuilder("cpu", num_sms=148)
    long_k.add_task(_task(8192, 49152, 12288))
    assert long_k.choose_tile_m() == 256
    short_k = FusedProgramBuilder("cpu", num_sms=148)
    short_k.add_task(_task(8192, 8192, 1024))
    assert short_k.choose_tile_m() == "pair"
    explicit = FusedProgramBuilder("cpu", num_sms=148, tile_m="pair512")
    explicit.add_task(_task(300, 200, 157))
    assert explicit.choose_tile_m() == "pair512"


def test_model_time_matches_the_measured_scale():
    """The time model reproduces the measured 8192^3 kernel times of the variants within 10 % (0.69 / 0.73 / 0.88 ms)."""
    for variant, measured_us in ((256, 690.0), ("pair", 725.0), (128, 880.0)):
        b = FusedProgramBuilder("cpu", num_sms=148)
        b.add_task(_task(8192, 8192, 8192))
        assert abs(b.model_us(variant) - measured_us) / measured_us < 0.10, (variant, b.model_us(variant))
    assert FusedProgramBuilder("cpu", num_sms=1).model_us("pair") is None
