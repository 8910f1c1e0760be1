"""Planner semantics (CPU): golden op lists and the sum-of-ops property.

The golden strings are op lists of the reference planners for world size 8
(M = N = K = 8192 unless noted); the property test checks that the ops of all
ranks and replicas add up to A @ B for every partition triple.
"""
import itertools

import pytest
import torch

import universal_gemm_b200 as ug
from universal_gemm_b200.parallel import plan as P
from universal_gemm_b200.parallel.partition import get_partitioning

from helpers import ALL_TRIPLES


def layouts(triple, rep, world, m, n, k):
    return (get_partitioning(triple[0], rep, world).layout((m, k)),
            get_partitioning(triple[1], rep, world).layout((k, n)),
            get_partitioning(triple[2], rep, world).layout((m, n)))


def test_golden_stationary_c_row_row_row_rank3():
    a, b, c = layouts(("row", "row", "row"), 1, 8, 8192, 8192, 8192)
    ops = ug.build_stationary_c_ops(a, b, c, rank=3)
    assert len(ops) == 8
    assert ug.format_op(ops[0]) == ("C.tile(3, 0)[0:1024, 0:8192] += A.tile(3, 0)[0:1024, 3072:4096] * "
                                    "B.tile(3, 0)[0:1024, 0:8192]")
    assert [op.b_idx[0] for op in ops] == [3, 4, 5, 6, 7, 0, 1, 2]
    assert [op.a_slice.cols.start for op in ops] == [3072, 4096, 5120, 6144, 7168, 0, 1024, 2048]
    text = ug.format_plan(ops, 3)
    assert text.splitlines()[0] == "Stationary-C plan (rank=3): 8 ops"
    assert text.splitlines()[1].startswith("  0000: C.tile(3, 0)")


def test_golden_stationary_b_row_row_row_rank3():
    a, b, c = layouts(("row", "row", "row"), 1, 8, 8192, 8192, 8192)
    ops = ug.build_stationary_b_ops(a, b, c, rank=3)
    assert [op.c_idx[0] for op in ops] == [3, 4, 5, 6, 7, 0, 1, 2]
    assert all(op.b_idx == (3, 0) and op.a_slice.cols == ug.Slice1D(3072, 4096) for op in ops)
    assert ug.format_stationary_b_plan(ops, 3).startswith("Stationary-B plan (rank=3): 8 ops")


def test_golden_block_rank5():
    a, b, c = layouts(("block", "block", "block"), 1, 8, 8192, 8192, 8192)
    ops = ug.build_stationary_c_ops(a, b, c, rank=5)
    got = [(op.a_idx, (op.a_slice.cols.start, op.a_slice.cols.stop), op.b_idx) for op in ops]
    assert got == [((2, 1), (2048, 4096), (3, 1)), ((2, 0), (0, 2048), (0, 1)), ((2, 0), (2048, 4096), (1, 1)),
                   ((2, 1), (0, 2048), (2, 1))]
    assert all(op.c_idx == (2, 1) and op.c_slice.shape == (2048, 4096) for op in ops)
    ops_b = ug.build_stationary_b_ops(a, b, c, rank=5)
    assert [(op.c_idx, op.a_idx) for op in ops_b] == [((3, 1), (3, 1)), ((0, 1), (0, 1)), ((1, 1), (1, 1)),
                                                      ((2, 1), (2, 1))]
    assert all(op.b_idx == (2, 1) and op.a_slice.cols == ug.Slice1D(0, 2048) for op in ops_b)


def test_golden_replication2_rank5():
    a, b, c = layouts(("row", "row", "row"), 2, 8, 8192, 8192, 8192)
    ops = ug.build_stationary_c_ops(a, b, c, rank=5)
    assert [ug.format_op(o) for o in ops] == [
        "C.tile(1, 0)[0:2048, 0:8192] += A.tile(1, 0)[0:2048, 6144:8192] * B.tile(3, 0)[0:2048, 0:8192]",
        "C.tile(1, 0)[0:2048, 0:8192] += A.tile(1, 0)[0:2048, 0:2048] * B.tile(0, 0)[0:2048, 0:8192]",
    ]
    ops_b = ug.build_stationary_b_ops(a, b, c, rank=5)
    assert [(o.c_idx, o.a_idx, o.a_slice.cols.start, o.b_idx) for o in ops_b] == [
        ((3, 0), (3, 0), 2048, (1, 0)), ((0, 0), (0, 0), 2048, (1, 0))]


def test_golden_gpt3_shapes_rank2():
    a, b, c = layouts(("row", "column", "row"), 1, 8, 8192, 49152, 12288)
    ops = ug.build_stationary_c_ops(a, b, c, rank=2)
    assert ug.format_op(ops[0]) == ("C.tile(2, 0)[0:1024, 12288:18432] += A.tile(2, 0)[0:1024, 0:12288] * "
                                    "B.tile(0, 2)[0:12288, 0:6144]")
    assert [o.b_idx[1] for o in ops] == [2, 3, 4, 5, 6, 7, 0, 1]
    ops_b = ug.build_stationary_b_ops(a, b, c, rank=2)
    assert [o.c_idx[0] for o in ops_b] == [2, 3, 4, 5, 6, 7, 0, 1]
    assert all(o.b_idx == (0, 2) and o.c_slice.cols == ug.Slice1D(12288, 18432) for o in ops_b)
    a, b, c = layouts(("column", "row", "row"), 1, 8, 8192, 12288, 49152)
    ops = ug.build_stationary_c_ops(a, b, c, rank=2)
    assert [(o.a_idx, o.b_idx) for o in ops] == [((0, k), (k, 0)) for k in (2, 3, 4, 5, 6, 7, 0, 1)]
    assert all(o.a_slice.rows == ug.Slice1D(2048, 3072) and o.a_slice.cols == ug.Slice1D(0, 6144) for o in ops)
    ops_b = ug.build_stationary_b_ops(a, b, c, rank=2)
    assert [o.c_idx[0] for o in ops_b] == [2, 3, 4, 5, 6, 7, 0, 1]
    assert all(o.a_idx == (0, 2) for o in ops_b)


def test_golden_odd_rank7_has_expected_op():
    a, b, c = layouts(("row", "block", "column"), 1, 8, 3001, 3001, 3001)
    ops = ug.build_stationary_c_ops(a, b, c, rank=7)
    assert len(ops) == 32
    assert ("C.tile(0, 7)[2632:3001, 0:369] += A.tile(7, 0)[0:369, 1502:2253] * B.tile(2, 1)[0:751, 1131:1500]"
            in [ug.format_op(o) for o in ops])


def test_op_counts_small_shapes():
    m, n, k = 301, 203, 157
    count = lambda tr, kind: [len((ug.build_stationary_c_ops if kind == "c" else ug.build_stationary_b_ops)(
        *layouts(tr, 1, 8, m, n, k), rank=r)) for r in range(8)]
    assert count(("row", "row", "row"), "c") == [8] * 8
    assert count(("row", "row", "column"), "c") == [64] * 8
    assert count(("column", "column", "row"), "c") == [64] * 8
    assert count(("block", "block", "block"), "c") == [5] * 8
    assert all(4 <= x <= 8 for x in count(("block", "block", "block"), "b"))


def _accumulate_plan(ops, a_lay, b_lay, c_lay, full_a, full_b, out):
    for op in ops:
        ab, bb, cb = ug.tile_bounds(a_lay, op.a_idx), ug.tile_bounds(b_lay, op.b_idx), ug.tile_bounds(c_lay, op.c_idx)
        av = full_a[ab.rows.as_slice(), ab.cols.as_slice()][op.a_slice.as_slices()]
        bv = full_b[bb.rows.as_slice(), bb.cols.as_slice()][op.b_slice.as_slices()]
        assert av.shape == op.a_slice.shape and bv.shape == op.b_slice.shape
        cv = out[cb.rows.as_slice(), cb.cols.as_slice()][op.c_slice.as_slices()]
        assert cv.shape == op.c_slice.shape
        cv += av @ bv


@pytest.mark.parametrize("world,rep", [(1, 1), (2, 1), (2, 2), (4, 1), (4, 2), (4, 4), (8, 1), (8, 2), (8, 4), (8, 8)])
def test_sum_of_all_ops_is_a_times_b(world, rep):
    torch.manual_seed(1)
    for (m, n, k) in ((67, 45, 83), (9, 7, 5)):
        full_a, full_b = torch.randn(m, k, dtype=torch.float64), torch.randn(k, n, dtype=torch.float64)
        for triple in ALL_TRIPLES:
            a, b, c = layouts(triple, rep, world, m, n, k)
            for kind, build in (("c", ug.build_stationary_c_ops), ("b", ug.build_stationary_b_ops)):
                out = torch.zeros(m, n, dtype=torch.float64)
                anchor = c if kind == "c" else b
                for r in range(world):
                    ops = build(a, b, c, rank=r)
                    for op in ops:   # anchored on an owned tile
                        idx = op.c_idx if kind == "c" else op.b_idx
                        assert ug.tile_rank(anchor, idx, rank=r) == r
                    _accumulate_plan(ops, a, b, c, full_a, full_b, out)
                torch.testing.assert_close(out, full_a @ full_b, rtol=1e-10, atol=1e-10,
                                           msg=lambda s: f"{kind} {triple} world={world} rep={rep}: {s}")


def test_regions_are_disjoint_and_cover_ops():
    a, b, c = layouts(("block", "row", "column"), 1, 8, 301, 203, 157)
    for r in range(8):
        ops = ug.build_stationary_c_ops(a, b, c, rank=r)
        regions = ug.group_ops(ops)
        assert sum(len(x.ops) for x in regions) == len(ops)
        for x in regions:
            assert all(o.c_idx == x.c_idx and o.c_slice == x.c_slice for o in x.ops)


def test_auto_rule_and_cache():
    a, b, c = layouts(("row", "column", "row"), 1, 8, 8192, 49152, 12288)
    assert ug.select_method("auto", b, c) == "stationary_b"        # K > M
    a2, b2, c2 = layouts(("row", "column", "row"), 1, 8, 32768, 49152, 12288)
    assert ug.select_method("auto", b2, c2) == "stationary_c"
    assert ug.select_method("stationary_c", b, c) == "stationary_c"
    with pytest.raises(ValueError):
        ug.select_method("stationary_a", b, c)
    first = ug.build_stationary_c_ops(a, b, c, rank=1)
    assert ug.build_stationary_c_ops(a, b, c, rank=1) is first
    ug.clear_stationary_c_plan_cache()
    assert ug.build_stationary_c_ops(a, b, c, rank=1) is not first
    with pytest.raises(ValueError):
        ug.build_stationary_c_ops(a, b, c2, rank=0)


def test_min_traffic_method_selection():
    """GPT-3 up-projection with B split along K (row / row / row) on 8 ranks: Stationary-B ships 7/8 of an fp32 partial C
    per rank (1.4 GB), Stationary-C pulls 7/8 of B (1.06 GB), so ``min_traffic`` takes Stationary-C where the reference's
    size rule (K > M) takes Stationary-B; with a bf16 C the push halves and Stationary-B wins.  With a column-split B
    (row / column / row) both rules agree on Stationary-B."""
    from universal_gemm_b200.parallel import partition as PT, plan as PL

    m, n, k = 8192, 49152, 12288
    lay = lambda shape, part: PT.get_partitioning(part, 1, 8).layout(shape)  # noqa: E731
    a, b, c = lay((m, k), "row"), lay((k, n), "row"), lay((m, n), "row")
    assert PL.select_method("auto", b, c) == "stationary_b"
    tb, tc = PL.plan_traffic("stationary_b", a, b, c), PL.plan_traffic("stationary_c", a, b, c)
    assert tb == (7 * 1024 * 1536 * 2, 7 * 1024 * n * 4) and tc == (7 * 1536 * n * 2, 0)
    assert PL.select_method("min_traffic", b, c, a) == "stationary_c"
    assert PL.select_method("min_traffic", b, c, a, c_bytes=2) == "stationary_b"
    b_col = lay((k, n), "column")
    assert PL.select_method("min_traffic", b_col, c, a) == PL.select_method("auto", b_col, c) == "stationary_b"
    with pytest.raises(ValueError):
        PL.select_method("min_traffic", b, c)
