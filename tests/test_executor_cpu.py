"""Executors on emulated CPU clusters: every partition triple, both methods, replication."""
import pytest
import torch

import universal_gemm_b200 as ug
from universal_gemm_b200.parallel import tiles as T

from helpers import ALL_TRIPLES, build_cluster_matrices, make_inputs, oracle, run_cluster


@pytest.mark.parametrize("world,rep", [(1, 1), (2, 1), (4, 2), (8, 1), (8, 2), (8, 4)])
@pytest.mark.parametrize("method", ["stationary_c", "stationary_b", "auto"])
def test_all_triples_cpu(world, rep, method):
    m, n, k = 37, 29, 41
    full_a, full_b, full_c = make_inputs(m, n, k, seed=world * 10 + rep)
    triples = ALL_TRIPLES if world in (1, 8) else ALL_TRIPLES[::4]
    for triple in triples:
        cluster = ug.EmulatedCluster(world, "cpu")
        mats = build_cluster_matrices(cluster, full_a, full_b, full_c, triple, rep, torch.float32, torch.float32)
        run_cluster(cluster, mats, method)
        got = mats[0][2].full_tensor(replica=0)
        torch.testing.assert_close(got.double(), oracle(full_a, full_b, full_c, torch.float32), rtol=1e-4, atol=1e-4,
                                   msg=lambda s: f"{method} {triple} world={world} rep={rep}: {s}")


def test_repeated_calls_accumulate():
    full_a, full_b, full_c = make_inputs(16, 24, 32, seed=3)
    cluster = ug.EmulatedCluster(4, "cpu")
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c, ("row", "column", "block"), 1, torch.float32,
                                  torch.float32)
    for _ in range(3):
        run_cluster(cluster, mats, "stationary_b")
    want = full_c.double() + 3 * (full_a.double() @ full_b.double())
    torch.testing.assert_close(mats[0][2].full_tensor().double(), want, rtol=1e-4, atol=1e-4)


def test_tile_api_cpu():
    cluster = ug.EmulatedCluster(4, "cpu")
    full = torch.arange(8 * 6, dtype=torch.float32).reshape(8, 6)
    mats = [ug.distribute_tensor(full, w, "row") for w in cluster.worlds()]
    dm = mats[1]
    assert ug.tile(dm, (1, 0)).tolist() == full[2:4].tolist()
    with pytest.raises(RuntimeError):
        ug.tile(dm, (0, 0))
    got = ug.get_tile(dm, (3, 0))
    assert got.tolist() == full[6:8].tolist()
    part = ug.get_tile(dm, (2, 0), region=ug.Slice2D(ug.Slice1D(1, 2), ug.Slice1D(2, 5)))
    assert part.tolist() == full[5:6, 2:5].tolist()
    fut = ug.get_tile_async(dm, (0, 0))
    assert fut.get().tolist() == full[0:2].tolist()
    ug.accumulate_tile(dm, (2, 0), torch.ones(1, 2), slice_=ug.Slice2D(ug.Slice1D(0, 1), ug.Slice1D(4, 6))).wait()
    assert mats[2].local[0].tolist() == [24, 25, 26, 27, 29, 30]
    with pytest.raises(ValueError):
        ug.accumulate_tile(dm, (2, 0), torch.ones(3, 3))
    with pytest.raises(RuntimeError):
        ug.accumulate_tile(dm, (2, 0), torch.ones(2, 6, dtype=torch.float64))
    with pytest.raises(ValueError):
        ug.get_tile(dm, (4, 0))


def test_reduce_replicas_cpu():
    cluster = ug.EmulatedCluster(4, "cpu")
    mats = [ug.zeros(w, (4, 4), "row", torch.float32, replication_factor=2) for w in cluster.worlds()]
    for dm in mats:
        dm.local.fill_(float(dm.rank + 1))
    for dm in mats:
        ug.reduce_replicas(dm)
    # replica 0 = ranks 0,1; replica 1 = ranks 2,3 ; rank 2 adds into rank 0, rank 3 into rank 1
    assert mats[0].local.unique().tolist() == [4.0] and mats[1].local.unique().tolist() == [6.0]
    assert mats[2].local.unique().tolist() == [3.0]


def test_scratch_heap_lifetimes():
    world = ug.SingleWorld("cpu")
    heap = ug.SymmHeap(world, 1024, torch.float32)
    x = heap.alloc((16, 32))
    y = heap.alloc((16, 32))
    assert x.data_ptr() != y.data_ptr()
    with pytest.raises(RuntimeError):
        heap.alloc((16, 32))           # would wrap onto x which is still live
    heap.release(x)
    z = heap.alloc((16, 32))
    assert z.data_ptr() == x.data_ptr()
    with pytest.raises(RuntimeError):
        heap.alloc((64, 64))           # larger than the heap
    heap.reset()
    assert heap.alloc((4, 4)).data_ptr() == x.data_ptr()
    heap.close()


def test_profile_counters(capsys):
    from universal_gemm_b200 import profile

    profile.reset_stats()
    profile.add_comm_issue(0.25)
    profile.add_comm_sync(0.25)
    profile.add_compute(0.5)
    profile.set_total_runtime(2.0)
    profile.print_stats()
    out = capsys.readouterr().out
    assert "comm_issue: 0.25, comm_sync: 0.25, compute: 0.5" in out
    assert "total_runtime: 2.0, accounted: 1.0, unaccounted: 1.0" in out
    assert "accounted: 50.0%, unaccounted: 50.0%" in out
    profile.reset_stats()
    assert profile.snapshot() == {"comm_issue": 0.0, "comm_sync": 0.0, "compute": 0.0, "total_runtime": 0.0}


def test_beta_zero_cpu():
    full_a, full_b, full_c = make_inputs(20, 24, 28, seed=8)
    cluster = ug.EmulatedCluster(4, "cpu")
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c, ("row", "column", "row"), 1, torch.float32,
                                  torch.float32)
    for a, b, c in mats:
        ug.matmul(a, b, c, method="stationary_c", beta=0)
    torch.testing.assert_close(mats[0][2].full_tensor().double(), full_a.double() @ full_b.double(), rtol=1e-4, atol=1e-4)
    with pytest.raises(ValueError):
        ug.matmul(*mats[0], beta=2)


def test_put_tile_and_signal_cpu():
    cluster = ug.EmulatedCluster(3, "cpu")
    wins = [ug.zeros(w, (3, 8), "row", torch.float32) for w in cluster.worlds()]
    pads = [ug.SignalPad(w, slots=2) for w in cluster.worlds()]
    for r, (win, pad) in enumerate(zip(wins, pads)):
        ug.put_tile(win, ((r + 1) % 3, 0), torch.full((1, 4), float(r + 1)), slice_=ug.Slice2D(ug.Slice1D(0, 1), ug.Slice1D(2, 6)))
        pad.signal((r + 1) % 3, slot=1)
    for r, (win, pad) in enumerate(zip(wins, pads)):
        pad.wait(slot=1, value=1)
        assert win.local[0].tolist() == [0, 0] + [float((r - 1) % 3 + 1)] * 4 + [0, 0]
    pads[0].timeout_ns = int(0.05e9)
    with pytest.raises(TimeoutError):
        pads[0].wait(slot=0, value=1)


def test_distributed_mlp_cpu():
    from universal_gemm_b200.models import DistributedMLP

    cluster = ug.EmulatedCluster(4, "cpu")
    full_x = torch.randn(24, 16)
    blocks = [DistributedMLP(w, 24, 16, 48, seed=3) for w in cluster.worlds()]
    for blk in blocks:
        blk.set_input(full_x)
    for blk in blocks:        # phase 1 on every rank, then phase 2 (ranks of an emulated cluster run in turn)
        ug.matmul(blk.x, blk.w1, blk.h, beta=0)
    for blk in blocks:
        blk.act.local.copy_(torch.nn.functional.gelu(blk.h.local))
    for blk in blocks:        # K-split GEMM: several ranks add into y, so emulated ranks clear first, then add
        blk.y.zero_()
    for blk in blocks:
        ug.matmul(blk.act, blk.w2, blk.y, beta=1)
    torch.testing.assert_close(blocks[0].y.full_tensor(), blocks[0].reference(full_x), rtol=1e-4, atol=1e-4)
    single = DistributedMLP(ug.SingleWorld("cpu"), 24, 16, 48, seed=3)
    single.set_input(full_x)
    torch.testing.assert_close(single.forward().full_tensor(), single.reference(full_x), rtol=1e-4, atol=1e-4)


def test_redistribute_and_ring_matmul_cpu():
    full = torch.randn(37, 29)
    cluster = ug.EmulatedCluster(4, "cpu")
    srcs = [ug.distribute_tensor(full, w, "row") for w in cluster.worlds()]
    for target, rep in (("column", 1), ("block", 1), ("row", 2)):
        outs = [ug.redistribute(s, target, rep) for s in srcs]
        torch.testing.assert_close(outs[0].full_tensor(), full)
        assert ug.grid_shape(outs[0]) == ug.grid_shape(ug.get_partitioning(target, rep, 4).layout((37, 29)))
    halves = [ug.redistribute(s, "block", dtype=torch.bfloat16) for s in srcs]
    torch.testing.assert_close(halves[0].full_tensor().float(), full.bfloat16().float())
    full_a, full_b, full_c = make_inputs(16, 12, 20, seed=1)
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c, ("row", "row", "row"), 1, torch.float32, torch.float32)
    for a, b, c in mats:
        ug.row_partitioned_matmul(a, b, c)
    torch.testing.assert_close(mats[0][2].full_tensor().double(), oracle(full_a, full_b, full_c, torch.float32),
                               rtol=1e-4, atol=1e-4)
    with pytest.raises(ValueError):
        ug.row_partitioned_matmul(halves[0], mats[0][1], mats[0][2])


def test_guard_regions_detect_writes_outside_an_allocation():
    """With guard regions on, a full plan leaves them intact; a write past the end of a shard is reported."""
    full_a, full_b, full_c = make_inputs(37, 29, 41, seed=11)
    cluster = ug.EmulatedCluster(4, "cpu", guard_bytes=512)
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c, ("block", "row", "column"), 1, torch.float32,
                                  torch.float32)
    run_cluster(cluster, mats, "stationary_b")
    run_cluster(cluster, mats, "stationary_c")
    assert cluster.check_guards() == 3 * 4                      # A, B and C of every rank
    torch.testing.assert_close(mats[0][2].full_tensor().double(),
                               2 * oracle(full_a, full_b, full_c, torch.float32) - full_c.double(), rtol=1e-4, atol=1e-4)
    c2 = mats[2][2]
    raw = c2.buffer._raw_local
    assert raw.numel() == c2.buffer.nbytes + 2 * 512 and c2.buffer.ptr(2) == raw.data_ptr() + 512
    raw[512 + c2.buffer.nbytes + 7] = 0                          # one byte past the payload of rank 2's C
    with pytest.raises(ug.GuardViolation, match="rank 2.*above.*payload offset"):
        cluster.check_guards()
    plain = ug.EmulatedCluster(2, "cpu")
    ug.empty(plain.world(0), (8, 8), "row", torch.float32)
    assert plain.check_guards() == 0                             # no guards unless asked for
