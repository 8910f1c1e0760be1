"""Compare this package's planners with the reference's, op for op (run as a script by test_plan_reference.py).

The reference's ``build_stationary_{b,c}_ops`` (stationary_c_plan.py:182-283, stationary_b_plan.py:153-255) are run on
CPU from a verbatim copy of the reference tree given as ``argv[1]``: its module-level imports of nvshmem4py /
``cuda.core`` are satisfied with empty modules (the planners never call into them) and torch's ``fake`` process group
lets one process stand in for any rank of any world size.  Every (world, rank, replication, partition triple, shape)
is planned by both sides; op lists must be identical, including their order.  Configurations on which the reference
itself raises (its ``tile_bounds`` rejects empty trailing tiles) are counted and skipped.  Prints one JSON line.
"""
import itertools
import json
import os
import sys
import types


def main(ref_root: str, quick: bool) -> int:
    for name in ["nvshmem", "nvshmem.core", "cuda.core", "cuda.core.experimental", "cuda.core.experimental._stream",
                 "cuda.core.experimental._memory"]:
        sys.modules[name] = types.ModuleType(name)
    sys.modules["nvshmem"].core = sys.modules["nvshmem.core"]
    nt = types.ModuleType("nvshmem_types")
    nt.NvshmemStream = object
    sys.modules["nvshmem.core"].nvshmem_types = nt
    sys.modules["cuda.core.experimental"].Device = object
    sys.modules["cuda.core.experimental._stream"].Stream = object
    sys.modules["cuda.core.experimental._memory"].Buffer = object
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

    import torch
    import torch.distributed as dist
    from torch.distributed.tensor import DTensor
    from torch.distributed.tensor._utils import compute_local_shape_and_global_offset
    from torch.testing._internal.distributed.fake_pg import FakeStore

    # the reference's modules, by file path, under private names (its "benchmark" package name collides with ours)
    import importlib.util

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    sys.path.insert(0, ref_root)            # the reference's flat modules import each other by bare name
    ref_util = load("_ref_bench_util", os.path.join("benchmark", "util.py"))
    import dtensor_utils as rdt             # noqa: E402  (the reference's facade)

    from universal_gemm_b200.parallel import partition as P, plan as PL

    def ref_part(name, rep):
        if name == "row":
            return ref_util.row_partitioning(rep, "cpu")
        if name == "column":
            return ref_util.column_partitioning(rep, "cpu")
        return ref_util.two_dimensional_partitioning(None, rep, "cpu")

    def mk(shape, part):
        mesh, pl = part
        ls, _ = compute_local_shape_and_global_offset(shape, mesh, pl)
        return DTensor.from_local(torch.zeros(ls), mesh, pl, shape=torch.Size(shape), stride=(shape[1], 1),
                                  run_check=False)

    def conv(op):
        f = lambda s: ((s.rows.start, s.rows.stop), (s.cols.start, s.cols.stop))  # noqa: E731
        return (tuple(op.a_idx), tuple(op.b_idx), tuple(op.c_idx), f(op.a_slice), f(op.b_slice), f(op.c_slice))

    mismatches, compared, ref_errors = [], 0, 0
    shapes = [(301, 203, 157), (67, 45, 83)]
    worlds = (2, 8) if quick else (2, 4, 8)
    triples = list(itertools.product(("row", "column", "block"), repeat=3))
    for world in worlds:
        ranks = range(world) if not quick else sorted({0, 1, world - 1, world // 2})
        for rank in ranks:
            dist.init_process_group("fake", rank=rank, world_size=world, store=FakeStore())
            try:
                for rep in (1, 2, 4, 8):
                    if world % rep:
                        continue
                    for (pa, pb, pc), (m, n, k) in itertools.product(triples, shapes):
                        try:
                            ra, rb, rc = mk((m, k), ref_part(pa, rep)), mk((k, n), ref_part(pb, rep)), mk((m, n), ref_part(pc, rep))
                            r_c = [conv(o) for o in rdt.build_stationary_c_ops(ra, rb, rc)]
                            r_b = [conv(o) for o in rdt.build_stationary_b_ops(ra, rb, rc)]
                        except Exception:  # noqa: BLE001  (the reference rejects this configuration)
                            ref_errors += 1
                            continue
                        la = P.get_partitioning(pa, rep, world).layout((m, k))
                        lb = P.get_partitioning(pb, rep, world).layout((k, n))
                        lc = P.get_partitioning(pc, rep, world).layout((m, n))
                        m_c = [conv(o) for o in PL.build_stationary_c_ops(la, lb, lc, rank=rank)]
                        m_b = [conv(o) for o in PL.build_stationary_b_ops(la, lb, lc, rank=rank)]
                        compared += 2
                        if r_c != m_c:
                            mismatches.append(("stationary_c", world, rank, rep, pa, pb, pc, m, n, k))
                        if r_b != m_b:
                            mismatches.append(("stationary_b", world, rank, rep, pa, pb, pc, m, n, k))
            finally:
                dist.destroy_process_group()
    print(json.dumps({"compared": compared, "mismatches": mismatches[:20], "num_mismatches": len(mismatches),
                      "reference_errors": ref_errors}))
    return 1 if mismatches else 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1], len(sys.argv) > 2 and sys.argv[2] == "quick"))
