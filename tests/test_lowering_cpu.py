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


def test_split_k_cuts_atomic_tasks_into_whole_k_blocks():
    """8 tiles on 148 workers with 256 K blocks each: every task becomes parts of whole K blocks that cover K once."""
    t = _task(64, 2048, 16383, mode=native.C_ATOMIC)
    out = FusedProgramBuilder._split_k([t], 128, 148)
    assert len(out) == 18                                    # 148 // 8 tiles = 18 parts
    spans = [(a.col0, a.cols, b.row0, b.rows) for part in out for a, b in part.segments]
    assert all(a0 == b0 and ac == br for a0, ac, b0, br in spans)
    assert sorted(a0 for a0, *_ in spans) == [a0 for a0, *_ in spans] and spans[0][0] == 0
    assert sum(ac for _, ac, _, _ in spans) == 16383 and all(ac % 64 == 0 for _, ac, _, _ in spans[:-1])
    assert all(p.c_ptr == t.c_ptr and p.m == 64 and p.n == 2048 and p.c_mode == native.C_ATOMIC for p in out)
    # stores cannot be split (parts would overwrite each other), nor can plans that fill the GPU already
    assert FusedProgramBuilder._split_k([_task(64, 2048, 16383, mode=native.C_STORE)], 128, 148)[0].segments == \
        _task(64, 2048, 16383, mode=native.C_STORE).segments
    many = [_task(1024, 6144, 12288, mode=native.C_ATOMIC) for _ in range(8)]
    assert FusedProgramBuilder._split_k(many, 256, 74) == many


def test_row_tasks_that_share_b_are_merged_into_a_stacked_task():
    """Eight tasks of 8 rows each (A row tiles of a skinny problem on 8 ranks) with the same B slice become one task of
    64 rows whose A is the stack of the eight slices and whose output rows go to eight places."""
    from universal_gemm_b200.ops.fused import StackedSlice

    k, n = 2048, 512
    bslice = OperandSlice(base=1 << 20, ld=n, row0=0, col0=0, rows=k, cols=n)
    b = FusedProgramBuilder("cpu", num_sms=148, split_k=True)
    for i in range(8):
        a = OperandSlice(base=(2 + i) << 20, ld=k, row0=0, col0=0, rows=8, cols=k, remote=i != 3)
        b.add_task(TaskSpec(c_ptr=(64 + i) << 20, ldc=n, m=8, n=n, c_mode=native.C_ATOMIC, c_dtype=native.DT_F32,
                            segments=[(a, bslice)], c_remote=i != 3))
    other = _task(300, 200, 157, mode=native.C_ATOMIC)           # 300 rows: left alone
    b.add_task(other)
    assert b.merge_row_tasks() == 7
    merged, untouched = b.tasks
    assert untouched is other
    a_stack, b_same = merged.segments[0]
    assert isinstance(a_stack, StackedSlice) and a_stack.rows == 64 and a_stack.cols == k and b_same == bslice
    assert merged.m == 64 and merged.c_rows == tuple(((64 + i) << 20, n, 8) for i in range(8)) and merged.c_remote
    assert [off for _, off in a_stack.row_parts()] == list(range(0, 64, 8)) and not a_stack.tma_ok()
    assert a_stack.with_cols(128, 64).parts[5].col0 == 128 and a_stack.remote_bytes() == 7 * 8 * k * 2
    # tasks whose B slices differ are not merged
    b2 = FusedProgramBuilder("cpu", num_sms=148)
    for i in range(2):
        b2.add_task(TaskSpec(c_ptr=(64 + i) << 20, ldc=n, m=8, n=n, c_mode=native.C_ATOMIC, c_dtype=native.DT_F32,
                             segments=[(OperandSlice((2 + i) << 20, k, 0, 0, 8, k),
                                        OperandSlice(1 << 20, 2 * n, 0, i * n, k, n))]))
    assert b2.merge_row_tasks() == 0 and len(b2.tasks) == 2


def test_split_fp32_slices_are_always_staged():
    hi = OperandSlice(base=4096, ld=128, row0=0, col0=0, rows=16, cols=64, elem_bytes=4, split=1)
    assert not hi.tma_ok() and hi.vector_ok() and hi.with_split(2).split == 2
    assert hi.address(1, 2) == 4096 + (128 + 2) * 4
