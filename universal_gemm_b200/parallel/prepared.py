"""Prepared distributed GEMMs: resolve the plan and the lowered program once, then run it with three
launches per call, optionally replayed from a CUDA graph.

``ug.matmul`` looks its plan and program up in caches on every call, which costs tens of microseconds of
host time; for small, latency-bound GEMMs that is comparable to the GPU time.  ``prepare_matmul`` does the
look-ups once.  ``MatmulPlan.capture()`` records ``[zero C] -> barrier -> fused kernel -> barrier`` into a
``torch.cuda.CUDAGraph``; the barrier keeps its round counter in device memory, so replays stay in step
across ranks (every rank must replay the same number of times).
"""
from __future__ import annotations

from typing import Any

import torch

from . import exec as X
from . import plan as P
from .matrix import resolve


class MatmulPlan:
    def __init__(self, a: Any, b: Any, c: Any, *, method: str = "auto", beta: int = 1, fuse_replica_reduce: bool = True):
        self.a, self.b, self.c = resolve(a), resolve(b), resolve(c)
        if not X._can_fuse(self.a, self.b, self.c):
            raise RuntimeError("prepare_matmul needs a CUDA world and bfloat16 A / B (use ug.matmul otherwise)")
        self.method = P.select_method(method, self.b.layout, self.c.layout)
        self.kind = "b" if self.method == "stationary_b" else "c"
        build = P.build_stationary_b_ops if self.kind == "b" else P.build_stationary_c_ops
        self.ops = build(self.a.layout, self.b.layout, self.c.layout, rank=self.c.rank)
        self.beta = beta
        self.fuse = fuse_replica_reduce
        if not fuse_replica_reduce and X.T.replication_factor(self.c.layout) > 1:
            # run() / capture() queue only the fused kernel and its barriers; the separate reduction pass of the
            # executor (zero the non-origin replicas, reduce_replicas, barrier) is not part of a prepared plan.
            raise ValueError("a prepared plan of a replicated C needs fuse_replica_reduce=True "
                             "(use ug.matmul(..., fuse_replica_reduce=False) for the separate reduction pass)")
        # lowering happens here; later calls hit the program cache by identity of the op list
        self.program, self.needs_zero = X._program(self.kind, self.a, self.b, self.c, self.ops, self.fuse, beta)
        self._graph: torch.cuda.CUDAGraph | None = None

    def run(self) -> None:
        """Queue one ``C (+)= A @ B`` on the current stream."""
        if self._graph is not None:
            self._graph.replay()
            return
        X._run_fused(self.kind, self.a, self.b, self.c, self.ops, fuse_replica_reduce=self.fuse, beta=self.beta)

    __call__ = run

    def capture(self, warmup: int = 2) -> "MatmulPlan":
        """Record one call into a CUDA graph (after ``warmup`` eager calls on a side stream, which also perform
        the one-time kernel attribute set-up that must not happen during capture).  Collective in the sense that
        every rank has to capture and later replay in the same order."""
        dev = self.c.device
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                X._run_fused(self.kind, self.a, self.b, self.c, self.ops, fuse_replica_reduce=self.fuse, beta=self.beta)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.c.world.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            X._run_fused(self.kind, self.a, self.b, self.c, self.ops, fuse_replica_reduce=self.fuse, beta=self.beta)
        self._graph = graph
        return self


def prepare_matmul(a: Any, b: Any, c: Any, *, method: str = "auto", beta: int = 1, **kwargs) -> MatmulPlan:
    return MatmulPlan(a, b, c, method=method, beta=beta, **kwargs)
