"""Shared helpers: emulated clusters, CPU oracle, plan checks."""
from __future__ import annotations

import itertools

import torch

import universal_gemm_b200 as ug
from universal_gemm_b200.parallel import tiles as T

PARTS = ("row", "column", "block")
ALL_TRIPLES = list(itertools.product(PARTS, repeat=3))


def make_inputs(m, n, k, seed=0, scale=None, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g)
    b = torch.randn(k, n, generator=g) * (scale if scale is not None else 1.0 / max(k, 1) ** 0.5)
    c0 = torch.randn(m, n, generator=g)
    return a.to(device), b.to(device), c0.to(device)


def build_cluster_matrices(cluster, full_a, full_b, full_c, triple, rep, in_dtype, out_dtype):
    """Distribute A, B, C on every rank of an emulated cluster; returns per-rank (a, b, c)."""
    out = []
    for w in cluster.worlds():
        a = ug.distribute_tensor(full_a, w, triple[0], rep, dtype=in_dtype)
        b = ug.distribute_tensor(full_b, w, triple[1], rep, dtype=in_dtype)
        c = ug.distribute_tensor(full_c, w, triple[2], rep, dtype=out_dtype)
        out.append((a, b, c))
    return out


def run_cluster(cluster, mats, method, **kwargs):
    """Execute one distributed GEMM on an emulated cluster, rank after rank."""
    rep_c = T.replication_factor(mats[0][2].layout)
    fused_reduce = kwargs.get("fuse_replica_reduce", True) and kwargs.get("executor") != "tilewise" \
        and mats[0][2].world.is_cuda and mats[0][0].dtype == torch.bfloat16
    if rep_c > 1 and not fused_reduce:
        # phases must be separated across ranks: zero -> compute -> reduce
        for a, b, c in mats:
            if T.my_replica(c.layout, c.rank) != 0:
                c.local_padded.zero_()
        from universal_gemm_b200.parallel import exec as X, plan as P, runtime as R

        for a, b, c in mats:
            kind = "b" if P.select_method(method, b.layout, c.layout) == "stationary_b" else "c"
            build = P.build_stationary_b_ops if kind == "b" else P.build_stationary_c_ops
            ops = build(a.layout, b.layout, c.layout, rank=c.rank)
            if kwargs.get("executor") == "fused":
                X._run_fused(kind, a, b, c, ops, fuse_replica_reduce=False)
            else:
                X._run_tilewise(kind, a, b, c, ops)
        for a, b, c in mats:
            R.reduce_replicas(c)
        return
    for a, b, c in mats:
        ug.matmul(a, b, c, method=method, **kwargs)


def oracle(full_a, full_b, full_c, in_dtype):
    a = full_a.to(in_dtype).double()
    b = full_b.to(in_dtype).double()
    return full_c.double() + a @ b
