"""A tensor-parallel transformer MLP block built from two distributed GEMMs.

    H = X @ W1        X [tokens, hidden] row-partitioned (token-sharded activations),
                      W1 [hidden, ffn] column-partitioned (column-parallel up-projection), H row-partitioned
    Y = gelu(H) @ W2  W2 [ffn, hidden] row-partitioned (K split), Y row-partitioned

These are the "GPT-3 expansion / shrinking" GEMMs of the benchmark suite with the partition triples
row,column,row and row,row,row.  The reference has no model code; this block shows how the partition
triples compose into a layer and serves as the smoke-test workload.  Forward only.
"""
from __future__ import annotations

import torch

from ..parallel.exec import matmul
from ..parallel.matrix import DistMatrix, distribute_tensor, empty, zeros
from ..parallel.symm import World


class DistributedMLP:
    def __init__(self, world: World, tokens: int, hidden: int, ffn: int, *, dtype: torch.dtype | None = None,
                 method: str = "auto", seed: int = 0):
        self.world = world
        self.method = method
        self.dtype = dtype or (torch.bfloat16 if world.is_cuda else torch.float32)
        g = torch.Generator().manual_seed(seed)
        w1 = torch.randn(hidden, ffn, generator=g) * hidden ** -0.5
        w2 = torch.randn(ffn, hidden, generator=g) * ffn ** -0.5
        self.w1 = distribute_tensor(w1, world, "column", dtype=self.dtype)
        self.w2 = distribute_tensor(w2, world, "row", dtype=self.dtype)
        self.x = empty(world, (tokens, hidden), "row", self.dtype)
        self.h = zeros(world, (tokens, ffn), "row", torch.float32)
        self.act = empty(world, (tokens, ffn), "row", self.dtype)
        self.y = zeros(world, (tokens, hidden), "row", torch.float32)

    def set_input(self, full_x: torch.Tensor) -> None:
        self.x.local_padded.zero_()
        self.x.fill_from_full(full_x)

    def forward(self) -> DistMatrix:
        """``y = gelu(x @ w1) @ w2``; every call is stream-ordered, the result is the row-partitioned ``self.y``."""
        matmul(self.x, self.w1, self.h, method=self.method, beta=0)
        # activation on the local token rows (elementwise, no communication), cast to the GEMM input dtype
        self.act.local.copy_(torch.nn.functional.gelu(self.h.local))
        matmul(self.act, self.w2, self.y, method=self.method, beta=0)
        return self.y

    def reference(self, full_x: torch.Tensor) -> torch.Tensor:
        """Same computation on one device from the gathered weights (for checks)."""
        w1 = self.w1.full_tensor().float()
        w2 = self.w2.full_tensor().float()
        x = full_x.to(self.world.device).to(self.dtype).float()
        return torch.nn.functional.gelu(x @ w1).to(self.dtype).float() @ w2
