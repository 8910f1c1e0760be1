"""Workload definitions (GEMM shape families) and small model blocks built on the distributed GEMM."""
from .workloads import (  # noqa: F401
    GPT3_FFN, GPT3_HIDDEN, MethodCase, ShapeCase, build_shape_suite, case_key, gpt3_expansion, gpt3_shrinking,
    merged_row, odd, square,
)
from .mlp import DistributedMLP  # noqa: F401,E402
