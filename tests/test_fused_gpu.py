"""GPU tests: the fused tcgen05 kernel and the tile kernels against fp32 PyTorch references,
and the fused executors on an emulated multi-rank cluster that lives on one GPU (ranks run
one after the other; remote tiles are other buffers of the same GPU, so every fetch / push
path of the kernel is exercised without a second device)."""
import pytest
import torch

import universal_gemm_b200 as ug

from helpers import ALL_TRIPLES, build_cluster_matrices, make_inputs, oracle, run_cluster

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _status_ok():
    from universal_gemm_b200.ops.device import DeviceState

    torch.cuda.synchronize()
    DeviceState.get(_dev()).check()


def _native_loaded():
    from universal_gemm_b200.ops import build

    with open("/proc/self/maps") as f:
        return str(build.library_path()) in f.read()


def test_native_library_is_loaded():
    from universal_gemm_b200.ops import native

    assert native.lib().ug_version() >= 1
    assert _native_loaded()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (512, 1024, 512), (300, 520, 200), (375, 1000, 376),
                                   (64, 4099, 1024), (2048, 4096, 1024), (1, 8, 8)])
@pytest.mark.parametrize("mode", ["store", "add", "atomic"])
@pytest.mark.parametrize("tile_m", [128, 256, "pair", "pair512"])
def test_gemm_kernel_fp32_out(m, n, k, mode, tile_m):
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import gemm

    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c0 = torch.randn(m, n, device=_dev())
    c = c0.clone()
    gemm(a, b, c, mode={"store": native.C_STORE, "add": native.C_ADD, "atomic": native.C_ATOMIC}[mode], tile_m=tile_m)
    _status_ok()
    ref = a.float() @ b.float() + (0 if mode == "store" else c0)
    torch.testing.assert_close(c, ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("mode", ["store", "add", "atomic"])
def test_gemm_kernel_bf16_out(mode):
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import gemm

    torch.manual_seed(5)
    m, n, k = 384, 777, 320
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c0 = torch.randn(m, n, device=_dev()).bfloat16()
    c = c0.clone()
    gemm(a, b, c, mode={"store": native.C_STORE, "add": native.C_ADD, "atomic": native.C_ATOMIC}[mode])
    _status_ok()
    ref = a.float() @ b.float() + (0 if mode == "store" else c0.float())
    torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=3e-2)


@pytest.mark.parametrize("stage_a,stage_b", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("tile_m", [128, 256, "pair", "pair512"])
def test_gemm_kernel_segments_and_staging(stage_a, stage_b, tile_m):
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import build_gemm_program, run_program

    torch.manual_seed(9)
    m, n, k = 640, 1290, 1500
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c = torch.zeros(m, n, device=_dev())
    cuts = [0, 500, 1001, 1500]          # 1001 is not a multiple of 8: that segment is staged and re-aligned
    prog = build_gemm_program([a[:, cuts[i]:cuts[i + 1]] for i in range(3)], [b[cuts[i]:cuts[i + 1]] for i in range(3)],
                              c, mode=native.C_STORE, stage_a=stage_a, stage_b=stage_b, tile_m=tile_m)
    assert prog.num_pieces > 0
    for _ in range(2):                   # second launch checks that the counters are reset
        run_program(prog, _dev())
    _status_ok()
    torch.testing.assert_close(c, a.float() @ b.float(), rtol=2e-3, atol=2e-3)


def test_tile_kernels():
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.device import DeviceState

    st = DeviceState.get(_dev())
    torch.manual_seed(0)
    for dtype, code in ((torch.float32, native.DT_F32), (torch.bfloat16, native.DT_BF16)):
        es = torch.empty(0, dtype=dtype).element_size()
        for rows, cols, off in ((64, 128, 0), (37, 53, 0), (37, 53, 3), (1, 8, 0)):
            src = torch.randn(rows + 2, cols + 16, device=_dev()).to(dtype)
            dst = torch.zeros(rows + 2, cols + 24, device=_dev(), dtype=dtype)
            sv, dv = src[1:1 + rows, off:off + cols], dst[1:1 + rows, 8:8 + cols]
            st.pull_2d(dv.data_ptr(), dst.stride(0) * es, sv.data_ptr(), src.stride(0) * es, rows, cols * es, es)
            torch.cuda.synchronize()
            outside = dst.clone()
            outside[1:1 + rows, 8:8 + cols] = 0
            assert torch.equal(dv, sv) and outside.abs().max().item() == 0
            before = dv.clone()
            st.accumulate_2d(dv.data_ptr(), dst.stride(0), sv.data_ptr(), src.stride(0), rows, cols, code)
            torch.cuda.synchronize()
            torch.testing.assert_close(dv.float(), before.float() * 2, rtol=1e-2, atol=1e-2)
            st.zero_2d(dv.data_ptr(), dst.stride(0) * es, rows, cols * es)
            torch.cuda.synchronize()
            assert dst.abs().sum() == 0
    f = torch.randn(33, 47, device=_dev())
    h = torch.zeros(33, 64, device=_dev(), dtype=torch.bfloat16)
    st.convert_2d(h.data_ptr(), 64, native.DT_BF16, f.data_ptr(), 47, native.DT_F32, 33, 47)
    torch.cuda.synchronize()
    assert torch.equal(h[:, :47], f.bfloat16())
    f2 = torch.randn(40, 96, device=_dev())                       # aligned: the 16-byte vector kernels
    h2 = torch.zeros(40, 128, device=_dev(), dtype=torch.bfloat16)
    st.convert_2d(h2.data_ptr(), 128, native.DT_BF16, f2.data_ptr(), 96, native.DT_F32, 40, 96)
    back = torch.zeros(40, 96, device=_dev())
    st.convert_2d(back.data_ptr(), 96, native.DT_F32, h2.data_ptr(), 128, native.DT_BF16, 40, 96)
    torch.cuda.synchronize()
    assert torch.equal(h2[:, :96], f2.bfloat16()) and torch.equal(back, f2.bfloat16().float()) and h2[:, 96:].abs().sum() == 0


@pytest.mark.parametrize("world,rep", [(1, 1), (2, 1), (4, 2), (8, 1), (8, 2), (8, 4)])
@pytest.mark.parametrize("method", ["stationary_c", "stationary_b"])
def test_fused_all_triples_emulated(world, rep, method):
    m, n, k = 301, 203, 157
    full_a, full_b, full_c = make_inputs(m, n, k, seed=world + rep, device=_dev())
    triples = ALL_TRIPLES if world == 8 and rep == 1 else ALL_TRIPLES[::3]
    for triple in triples:
        cluster = ug.EmulatedCluster(world, _dev())
        mats = build_cluster_matrices(cluster, full_a, full_b, full_c, triple, rep, torch.bfloat16, torch.float32)
        run_cluster(cluster, mats, method, executor="fused")
        _status_ok()
        got = mats[0][2].full_tensor(replica=0)
        torch.testing.assert_close(got.double(), oracle(full_a, full_b, full_c, torch.bfloat16), rtol=2e-3, atol=2e-3,
                                   msg=lambda s: f"{method} {triple} world={world} rep={rep}: {s}")


@pytest.mark.parametrize("triple", [("row", "row", "row"), ("row", "column", "row"), ("column", "row", "row"),
                                    ("block", "block", "block")])
@pytest.mark.parametrize("method", ["stationary_c", "stationary_b", "auto"])
def test_fused_medium_shapes_emulated(triple, method):
    m, n, k = 1024, 1536, 2048
    full_a, full_b, full_c = make_inputs(m, n, k, seed=11, device=_dev())
    for rep, out_dtype in ((1, torch.float32), (2, torch.float32), (1, torch.bfloat16)):
        cluster = ug.EmulatedCluster(8, _dev())
        mats = build_cluster_matrices(cluster, full_a, full_b, full_c, triple, rep, torch.bfloat16, out_dtype)
        for _ in range(2):
            run_cluster(cluster, mats, method, executor="fused")
        _status_ok()
        got = mats[0][2].full_tensor(replica=0).double()
        want = full_c.to(out_dtype).double() + 2 * (full_a.bfloat16().double() @ full_b.bfloat16().double())
        tol = 3e-3 if out_dtype == torch.float32 else 6e-2
        torch.testing.assert_close(got, want, rtol=tol, atol=tol,
                                   msg=lambda s: f"{method} {triple} rep={rep} {out_dtype}: {s}")


def test_unfused_replica_reduce_and_tilewise_on_gpu():
    m, n, k = 256, 320, 512
    full_a, full_b, full_c = make_inputs(m, n, k, seed=2, device=_dev())
    for executor in ("fused", "tilewise"):
        cluster = ug.EmulatedCluster(4, _dev())
        mats = build_cluster_matrices(cluster, full_a, full_b, full_c, ("row", "row", "row"), 2, torch.bfloat16,
                                      torch.float32)
        run_cluster(cluster, mats, "stationary_c", executor=executor, fuse_replica_reduce=False)
        _status_ok()
        torch.testing.assert_close(mats[0][2].full_tensor().double(), oracle(full_a, full_b, full_c, torch.bfloat16),
                                   rtol=3e-3, atol=3e-3)


def test_tile_api_on_gpu():
    cluster = ug.EmulatedCluster(4, _dev())
    full = torch.randn(64, 48, device=_dev())
    mats = [ug.distribute_tensor(full, w, "row") for w in cluster.worlds()]
    dm = mats[1]
    ug.init_scratch(4 * 16 * 64, torch.float32, world=dm.world)
    t = ug.get_tile(dm, (3, 0))
    fut = ug.get_tile_async(dm, (0, 0), region=ug.Slice2D(ug.Slice1D(3, 9), ug.Slice1D(5, 40)))
    part = fut.get()
    torch.cuda.synchronize()
    assert torch.equal(t, full[48:64]) and torch.equal(part, full[3:9, 5:40])
    ug.release_tile(t)
    ug.accumulate_tile(dm, (2, 0), torch.ones(16, 48, device=_dev())).wait()
    torch.testing.assert_close(mats[2].local, full[32:48] + 1)
    ug.free_get_tile_scratch()


def test_bounded_wait_reports_timeout_instead_of_hanging():
    """A cross-rank barrier whose peer never signals runs out after its limit and reports a
    status code; the context stays usable."""
    import ctypes

    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.device import DeviceState, KernelStatusError

    st = DeviceState.get(_dev())
    slots = torch.zeros(2, 8, dtype=torch.int32, device=_dev())      # "rank 1" never adds to our slot
    table = torch.tensor([slots[0].data_ptr(), slots[1].data_ptr()], dtype=torch.int64, device=_dev())
    rounds = torch.zeros(1, dtype=torch.int32, device=_dev())
    native.check(native.lib().ug_signal_barrier(table.data_ptr(), 2, 0, rounds.data_ptr(), st.status_ptr, 50_000_000, 0, 0,
                                                ctypes.c_void_p(st.stream())), "ug_signal_barrier")
    torch.cuda.synchronize()
    with pytest.raises(KernelStatusError) as err:
        st.check()
    assert err.value.code == native.ERR_TIMEOUT_PEER
    assert slots[1, 0].item() == 1 and rounds.item() == 1             # our own signal was delivered
    st.check()                                                        # status cleared, context alive
    assert torch.ones(4, device=_dev()).sum().item() == 4


@pytest.mark.parametrize("method,triple", [("stationary_c", ("row", "row", "row")), ("stationary_c", ("block", "column", "block")),
                                           ("stationary_b", ("row", "column", "row")), ("stationary_b", ("block", "column", "row"))])
def test_beta_zero_overwrites_without_zeroing(method, triple):
    """beta=0 on single-writer plans stores C = A @ B whatever C held before (no zeroing pass)."""
    m, n, k = 520, 390, 450
    full_a, full_b, full_c = make_inputs(m, n, k, seed=4, device=_dev())
    cluster = ug.EmulatedCluster(4, _dev())
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c * 100, triple, 1, torch.bfloat16, torch.float32)
    for a, b, c in mats:
        ug.matmul(a, b, c, method=method, beta=0)
    _status_ok()
    want = full_a.bfloat16().double() @ full_b.bfloat16().double()
    torch.testing.assert_close(mats[0][2].full_tensor().double(), want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("tile_m,m,n", [("pair", 512, 10240 - 17), (256, 512, 19712 - 5), (128, 256, 19712),
                                        ("pair512", 512, 20480 - 17)])
def test_gemm_kernel_tail_wave_uses_narrow_tiles(tile_m, m, n):
    """Tile counts just above a multiple of the worker count: the trailing tile columns run as 128-wide tiles."""
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import build_gemm_program, run_program

    torch.manual_seed(n)
    k = 320
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c = torch.full((m, n), 3.0, device=_dev())
    prog = build_gemm_program([a], [b], c, mode=native.C_ADD, tile_m=tile_m)
    assert prog.stats["tasks"] == 2                      # the task was split into a wide and a narrow part
    run_program(prog, _dev())
    _status_ok()
    torch.testing.assert_close(c, a.float() @ b.float() + 3.0, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("method", ["stationary_b", "stationary_c"])
def test_fused_tail_split_with_remote_tiles(method, monkeypatch):
    """Two emulated ranks with 80 tiles each on 74 CTA pairs: the last three tile columns run as narrow tiles,
    with the A slices staged from the 'peer' and (Stationary-B) the result stored into the peer's C."""
    from universal_gemm_b200.parallel import exec as X

    monkeypatch.setenv("UGEMM_TILE_M", "pair")
    m, n, k = 1024, 10240, 256
    full_a, full_b, full_c = make_inputs(m, n, k, seed=6, device=_dev())
    cluster = ug.EmulatedCluster(2, _dev())
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c, ("row", "column", "row"), 1, torch.bfloat16,
                                  torch.float32)
    X.clear_program_cache()
    for a, b, c in mats:
        ug.matmul(a, b, c, method=method, beta=0)
    _status_ok()
    stats = [v[2][0].stats for v in X._program_cache.values()]
    assert all(s["tiles"] == 86 and s["tasks"] == 3 for s in stats), stats   # 74 wide + 12 narrow tiles
    want = full_a.bfloat16().double() @ full_b.bfloat16().double()
    torch.testing.assert_close(mats[0][2].full_tensor().double(), want, rtol=2e-3, atol=2e-3)
    X.clear_program_cache()


def test_redistribute_on_gpu():
    full = torch.randn(301, 203, device=_dev())
    cluster = ug.EmulatedCluster(4, _dev())
    srcs = [ug.distribute_tensor(full, w, "block") for w in cluster.worlds()]
    outs = [ug.redistribute(s, "column") for s in srcs]
    halves = [ug.redistribute(s, "row", dtype=torch.bfloat16) for s in srcs]
    torch.cuda.synchronize()
    assert torch.equal(outs[2].full_tensor(), full)
    assert torch.equal(halves[1].full_tensor().float(), full.bfloat16().float())


def test_prepared_matmul_and_cuda_graph():
    """A prepared plan gives the same result eagerly and when replayed from a CUDA graph."""
    m, n, k = 512, 768, 640
    full_a, full_b, full_c = make_inputs(m, n, k, seed=12, device=_dev())
    world = ug.SingleWorld(_dev())
    a = ug.distribute_tensor(full_a, world, "row", dtype=torch.bfloat16)
    b = ug.distribute_tensor(full_b, world, "column", dtype=torch.bfloat16)
    c = ug.distribute_tensor(full_c, world, "row", dtype=torch.float32)
    plan = ug.prepare_matmul(a, b, c, method="stationary_c", beta=1)
    plan.run()
    _status_ok()
    prod = full_a.bfloat16().double() @ full_b.bfloat16().double()
    torch.testing.assert_close(c.full_tensor().double(), full_c.double() + prod, rtol=2e-3, atol=2e-3)
    plan.capture(warmup=1)              # two more accumulations: warm-up + capture run nothing new... capture does not execute
    torch.cuda.synchronize()
    before = c.full_tensor().double()
    for _ in range(3):
        plan()
    _status_ok()
    torch.testing.assert_close(c.full_tensor().double(), before + 3 * prod, rtol=2e-3, atol=4e-3)


@pytest.mark.parametrize("tile_m", [128, 256, "pair", "pair512"])
def test_kernel_timeline_records_every_tile(tile_m):
    """With tracing on, every tile leaves a record whose stamps are ordered, the fetch warps account for every
    staged piece, and the result is unchanged."""
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import build_gemm_program, run_program
    from universal_gemm_b200.utils import trace as TR

    torch.manual_seed(21)
    m, n, k = 1024, 1536, 768
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c = torch.zeros(m, n, device=_dev())
    prog = build_gemm_program([a], [b], c, mode=native.C_STORE, stage_a=True, tile_m=tile_m)
    assert prog.read_trace() is None
    prog.enable_trace()
    run_program(prog, _dev())
    _status_ok()
    torch.testing.assert_close(c, a.float() @ b.float(), rtol=2e-3, atol=2e-3)
    arr = prog.read_trace()
    pair = str(tile_m).startswith("pair")
    slots = arr.shape[1] - 1
    tiles = arr[:, :slots]
    leaders = tiles[::2] if pair else tiles
    seen = sorted(int(t) - 1 for t in leaders[:, :, TR.TILE].ravel() if t > 0)
    assert seen == list(range(prog.stats["tiles"]))
    rec = leaders[leaders[:, :, TR.TILE] > 0]
    assert (rec[:, TR.PROD_BEGIN] <= rec[:, TR.PROD_END]).all()
    assert (rec[:, TR.MMA_BEGIN] <= rec[:, TR.MMA_ISSUED]).all() and (rec[:, TR.MMA_BEGIN] > 0).all()
    assert (rec[:, TR.MMA_BEGIN] <= rec[:, TR.EPI_BEGIN]).all() and (rec[:, TR.EPI_BEGIN] <= rec[:, TR.EPI_END]).all()
    summ = arr[:, slots]
    assert (summ[:, TR.S_START] > 0).all() and (summ[:, TR.S_END] >= summ[:, TR.S_START]).all()
    assert int(summ[:, TR.S_PIECES].sum()) == prog.num_pieces
    s = TR.summarize(arr, pair=pair)
    assert s["recorded_tiles"] == prog.stats["tiles"] and s["pieces_copied"] == prog.num_pieces
    assert 0 < s["main_us_mean"] < s["kernel_us"] < 1e5
    assert 0.1 < s["sm_clock_ghz"] < 3.0               # SM cycles per globaltimer nanosecond
    assert TR.to_chrome_trace(arr)
    prog.disable_trace()
    run_program(prog, _dev())
    _status_ok()


@pytest.mark.parametrize("tile_m", [128, 256, "pair", "pair512"])
def test_dynamic_tile_claiming_many_tiles_per_worker(tile_m, monkeypatch):
    """Dynamic tile claiming with more than 16 tiles per worker (the in-CTA tile queue wraps around), launched
    several times in a row (the kernel re-arms its claim counters itself)."""
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import build_gemm_program, run_program

    monkeypatch.setenv("UGEMM_DYNAMIC_TILES", "1")
    torch.manual_seed(5)
    m, n, k = 8192, 24576, 128
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c = torch.zeros(m, n, device=_dev())
    prog = build_gemm_program([a], [b], c, mode=native.C_STORE, tile_m=tile_m)
    workers = prog.grid // 2 if str(tile_m).startswith("pair") else prog.grid
    assert prog.params.sched != 0 and prog.stats["tiles"] > 16 * workers
    for _ in range(3):
        run_program(prog, _dev())
    _status_ok()
    torch.testing.assert_close(c, a.float() @ b.float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("method", ["stationary_b", "stationary_c"])
def test_fused_kernels_stay_inside_their_allocations(method):
    """Odd shapes on an emulated 4-rank cluster whose symmetric allocations carry guard regions: fetch warps,
    epilogue stores / red.add into 'peers' and the zeroing kernels must leave every guard byte alone."""
    m, n, k = 389, 517, 263
    full_a, full_b, full_c = make_inputs(m, n, k, seed=17, device=_dev())
    for triple in [("row", "column", "block"), ("block", "block", "block"), ("column", "row", "row")]:
        cluster = ug.EmulatedCluster(4, _dev(), guard_bytes=4096)
        mats = build_cluster_matrices(cluster, full_a, full_b, full_c, triple, 1, torch.bfloat16, torch.float32)
        run_cluster(cluster, mats, method)
        _status_ok()
        assert cluster.check_guards() == 12
        torch.testing.assert_close(mats[0][2].full_tensor().double(), oracle(full_a, full_b, full_c, torch.bfloat16),
                                   rtol=2e-3, atol=2e-3)


def test_beta_zero_with_separate_replica_reduction_clears_every_replica():
    """beta=0, Stationary-B with a column-partitioned B (no K split), replication 2 and the replica reduction as a
    separate pass: every replica fills only its share of its own copy of C, so the plan must report that all copies
    start at zero (stale rows of replica 0 would otherwise survive into the sum)."""
    from universal_gemm_b200.ops.device import DeviceState
    from universal_gemm_b200.parallel import exec as X, plan as P, runtime as R

    m, n, k = 512, 384, 320
    full_a, full_b, full_c = make_inputs(m, n, k, seed=23, device=_dev())
    cluster = ug.EmulatedCluster(4, _dev())
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c * 100, ("row", "column", "row"), 2, torch.bfloat16,
                                  torch.float32)
    X.clear_program_cache()
    progs = []
    for a, b, c in mats:
        ops = P.build_stationary_b_ops(a.layout, b.layout, c.layout, rank=c.rank)
        prog, needs_zero = X._program("b", a, b, c, ops, False, 0)
        assert needs_zero
        progs.append(prog)
    st = DeviceState.get(_dev())
    for _, _, c in mats:                 # what every rank's executor does before its entry barrier
        c.local_padded.zero_()
    for prog in progs:                   # the ranks' kernels, one after the other
        prog.reset_flags(st.stream())
        prog.launch(st.stream())
    for _, _, c in mats:
        R.reduce_replicas(c)
    _status_ok()
    want = full_a.bfloat16().double() @ full_b.bfloat16().double()
    torch.testing.assert_close(mats[0][2].full_tensor(replica=0).double(), want, rtol=2e-3, atol=2e-3)
    X.clear_program_cache()
    with pytest.raises(ValueError):      # prepared plans run only the fused kernel: no separate reduction pass
        ug.prepare_matmul(*mats[0], method="stationary_b", beta=0, fuse_replica_reduce=False)


@pytest.mark.parametrize("tile_m", [128, "pair"])
@pytest.mark.parametrize("field,value", [("a_map", 4000), ("b_flag", 100000), ("seg_count", 77)])
def test_corrupt_table_entry_is_reported_not_followed(tile_m, field, value):
    """An index in the device tables that points outside the tables the launch declared (written here by the host,
    as a truncated or stale table would) is caught by the kernel's own check: it reports UG_ERR_BAD_TABLE, touches
    nothing through that index and returns; C is left alone and the next launch with intact tables works."""
    import numpy as np

    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.device import DeviceState, KernelStatusError
    from universal_gemm_b200.ops.gemm import build_gemm_program, run_program

    torch.manual_seed(3)
    m, n, k = 512, 512, 256
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c = torch.full((m, n), 5.0, device=_dev())
    prog = build_gemm_program([a], [b], c, mode=native.C_STORE, stage_b=True, tile_m=tile_m)
    tables = prog._tables
    is_task = field == "seg_count"
    dtype = native.TASK_DTYPE if is_task else native.SEGMENT_DTYPE
    off = (prog.params.tasks if is_task else prog.params.segs) - tables.data_ptr()
    good = tables[off:off + dtype.itemsize].clone()
    row = np.frombuffer(good.cpu().numpy().tobytes(), dtype=dtype).copy()
    row[0][field] = value
    tables[off:off + dtype.itemsize].copy_(torch.from_numpy(np.frombuffer(row.tobytes(), dtype=np.uint8).copy()))
    prog.params.timeout_ns = 200_000_000
    run_program(prog, _dev())
    torch.cuda.synchronize()
    with pytest.raises(KernelStatusError) as err:
        DeviceState.get(_dev()).check()
    assert err.value.code == native.ERR_BAD_TABLE
    tables[off:off + dtype.itemsize].copy_(good)
    run_program(prog, _dev())
    _status_ok()
    torch.testing.assert_close(c, a.float() @ b.float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("offset,n", [(1, 1537), (2, 700), (3, 256), (1, 5), (3, 67)])
@pytest.mark.parametrize("mode", ["store", "add", "atomic"])
@pytest.mark.parametrize("tile_m", [128, 256, "pair", "pair512"])
def test_gemm_kernel_c_region_on_odd_columns(offset, n, mode, tile_m):
    """C is a column range that starts on an odd column of a wider, 16-byte-pitched matrix (what a column or block
    partition of an odd-sized C gives): the epilogue writes head columns singly and the rest as 16-byte vectors, and
    must not touch the columns next to the region."""
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import gemm

    torch.manual_seed(offset * 1000 + n)
    m, k = 300, 200
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    pitch = (offset + n + 7 + 63) // 64 * 64
    big0 = torch.randn(m, pitch, device=_dev())
    big = big0.clone()
    c = big[:, offset:offset + n]
    gemm(a, b, c, mode={"store": native.C_STORE, "add": native.C_ADD, "atomic": native.C_ATOMIC}[mode], tile_m=tile_m)
    _status_ok()
    ref = a.float() @ b.float() + (0 if mode == "store" else big0[:, offset:offset + n])
    torch.testing.assert_close(c, ref, rtol=2e-3, atol=2e-3)
    assert torch.equal(big[:, :offset], big0[:, :offset]) and torch.equal(big[:, offset + n:], big0[:, offset + n:])


@pytest.mark.parametrize("method", ["stationary_c", "stationary_b"])
@pytest.mark.parametrize("triple", [("row", "column", "row"), ("column", "row", "row"), ("block", "block", "block")])
def test_skinny_problem_splits_k_across_the_gpu(method, triple):
    """M = 64 against a long K: a rank has a handful of output tiles, so the lowering cuts K into parts that add into
    C atomically (all ranks zero C first when beta = 0).  Result and beta = 1 accumulation must be unchanged."""
    from universal_gemm_b200.parallel import exec as X

    m, n, k = 64, 2100, 4500
    full_a, full_b, full_c = make_inputs(m, n, k, seed=31, device=_dev())
    cluster = ug.EmulatedCluster(8, _dev())
    mats = build_cluster_matrices(cluster, full_a, full_b, full_c, triple, 1, torch.bfloat16, torch.float32)
    X.clear_program_cache()
    prod = full_a.bfloat16().double() @ full_b.bfloat16().double()
    for _, _, c in mats:                                   # beta = 0: every rank clears its C, then all ranks add
        c.local_padded.fill_(3.0)
    progs = []
    from universal_gemm_b200.parallel import plan as P
    for a, b, c in mats:
        kind = "b" if method == "stationary_b" else "c"
        build = P.build_stationary_b_ops if kind == "b" else P.build_stationary_c_ops
        ops = build(a.layout, b.layout, c.layout, rank=c.rank)
        prog, needs_zero = X._program(kind, a, b, c, ops, True, 0)
        assert needs_zero
        progs.append((prog, c))
    assert any(p.stats["tasks"] >= 2 and p.stats["tiles"] >= 16 for p, _ in progs), [p.stats for p, _ in progs]
    if triple[0] != "column" and method == "stationary_b":   # A rows spread over the ranks and one B tile per rank:
        # the 8-row tasks of a rank share their B slices and were merged into stacked ones
        assert all(p.stats["indirect_rows"] > 0 for p, _ in progs), [p.stats for p, _ in progs]
    from universal_gemm_b200.ops.device import DeviceState
    st = DeviceState.get(_dev())
    for _, c in progs:
        c.local_padded.zero_()
    for prog, _ in progs:
        prog.reset_flags(st.stream())
        prog.launch(st.stream())
    _status_ok()
    torch.testing.assert_close(mats[0][2].full_tensor().double(), prod, rtol=2e-3, atol=2e-3)
    X.clear_program_cache()
    for a, b, c in mats:                                   # beta = 1 through the public call
        ug.matmul(a, b, c, method=method)
    _status_ok()
    torch.testing.assert_close(mats[0][2].full_tensor().double(), 2 * prod, rtol=2e-3, atol=2e-3)
    X.clear_program_cache()


@pytest.mark.parametrize("m,n,k", [(256, 512, 384), (300, 520, 200), (375, 1000, 1001), (64, 4099, 1024)])
@pytest.mark.parametrize("tile_m", [128, "pair"])
def test_gemm_kernel_fp32_operands_as_three_bf16_products(m, n, k, tile_m):
    """fp32 A and B: the fetch warps split every element into a bf16 high and low part while staging and the
    kernel accumulates lo x hi + hi x lo + hi x hi in fp32.  The result must be far closer to the fp64 product
    than a single bf16 product is (and within the reference example's tolerance for fp32 results)."""
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import gemm

    torch.manual_seed(m + k)
    a = torch.randn(m, k, device=_dev())
    b = torch.randn(k, n, device=_dev()) / k ** 0.5
    c = torch.full((m, n), 9.0, device=_dev())
    gemm(a, b, c, mode=native.C_STORE, tile_m=tile_m)
    _status_ok()
    want = a.double() @ b.double()
    err = (c.double() - want).abs().max().item()
    bf16_err = ((a.bfloat16().double() @ b.bfloat16().double()) - want).abs().max().item()
    assert err < 1e-4 and err < bf16_err / 50, (err, bf16_err)


@pytest.mark.parametrize("method", ["stationary_c", "stationary_b"])
def test_fused_fp32_operands_emulated(method):
    m, n, k = 301, 203, 517
    full_a, full_b, full_c = make_inputs(m, n, k, seed=41, device=_dev())
    for triple in [("row", "column", "row"), ("block", "block", "block"), ("column", "row", "row")]:
        cluster = ug.EmulatedCluster(4, _dev(), guard_bytes=4096)
        mats = build_cluster_matrices(cluster, full_a, full_b, full_c, triple, 1, torch.float32, torch.float32)
        run_cluster(cluster, mats, method)
        _status_ok()
        assert cluster.check_guards() == 12
        want = full_c.double() + full_a.double() @ full_b.double()
        torch.testing.assert_close(mats[0][2].full_tensor().double(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("m,n,k,tile_m", [(3001, 3001, 3001, "pair"), (3001, 3001, 3001, 256), (12289, 1537, 3001, 128),
                                          (64, 16383, 16383, None), (1537, 12289, 12289, "pair512")])
def test_gemm_kernel_large_odd_shapes(m, n, k, tile_m):
    """Odd sizes of the benchmark sweep at kernel level: odd pitches put A and B on the 2-byte gather path of the
    fetch warps, C is written with ragged right and bottom edges, M = 64 leaves most tensor rows empty."""
    from universal_gemm_b200.ops import native
    from universal_gemm_b200.ops.gemm import gemm

    torch.manual_seed(m + n)
    a = torch.randn(m, k, device=_dev()).bfloat16()
    b = (torch.randn(k, n, device=_dev()) / k ** 0.5).bfloat16()
    c = torch.full((m, n), 2.0, device=_dev())
    gemm(a, b, c, mode=native.C_ADD, tile_m=tile_m)
    _status_ok()
    torch.testing.assert_close(c, a.float() @ b.float() + 2.0, rtol=3e-3, atol=3e-3)


@pytest.mark.parametrize("case", ["aligned", "odd", "skinny", "bf16_c", "replicated"])
def test_epilogue_checksum_adds_up_to_the_sum_of_the_product(case):
    """``checksum=``: every rank's kernel adds the sum of all values it writes into (or adds to) C to a running
    double; over all ranks that is sum(A @ B), whatever path the epilogue takes (vector, shifted for odd columns,
    row table of merged skinny tasks with K split, bf16 output, pushes into replica 0) and over repeated calls."""
    m, n, k, triple, rep, c_dtype, world = {
        "aligned": (1024, 1536, 512, ("row", "column", "row"), 1, torch.float32, 4),
        "odd": (389, 517, 263, ("block", "column", "block"), 1, torch.float32, 4),
        "skinny": (64, 2100, 4500, ("row", "column", "row"), 1, torch.float32, 8),
        "bf16_c": (512, 777, 320, ("column", "row", "row"), 1, torch.bfloat16, 4),
        "replicated": (512, 768, 640, ("row", "row", "row"), 2, torch.float32, 4),
    }[case]
    full_a, full_b, full_c = make_inputs(m, n, k, seed=51, device=_dev())
    want = float((full_a.bfloat16().double() @ full_b.bfloat16().double()).sum().item())
    scale = float((full_a.bfloat16().double() @ full_b.bfloat16().double()).abs().sum().item())
    for method in ("stationary_c", "stationary_b"):
        cluster = ug.EmulatedCluster(world, _dev())
        mats = build_cluster_matrices(cluster, full_a, full_b, full_c, triple, rep, torch.bfloat16, c_dtype)
        sums = [torch.zeros(1, dtype=torch.float64, device=_dev()) for _ in mats]
        calls = 2
        for _ in range(calls):
            for (a, b, c), chk in zip(mats, sums):
                ug.matmul(a, b, c, method=method, checksum=chk)
        _status_ok()
        got = sum(float(x.item()) for x in sums)
        assert abs(got - calls * want) <= 1e-5 * scale + 1e-6, (case, method, got, calls * want)
