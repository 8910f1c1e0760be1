"""GEMM workload families of the benchmark suite.

The "models" of this framework are matrix shapes: the two GEMMs of a GPT-3-175B MLP block
(hidden 12288, FFN 49152) swept over the token count, square matrices, and odd / skinny
shapes with one large dimension.  Same families, labels and case keys as the reference's suite
(benchmark/run_matmul_experiments.py:74-158, :175-181) so that result files are interchangeable.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

GPT3_HIDDEN = 12 * 1024
GPT3_FFN = 48 * 1024


@dataclass(frozen=True)
class ShapeCase:
    experiment_group: str
    experiment_label: str
    varied_dim: str
    varied_value: int
    m: int
    n: int
    k: int


@dataclass(frozen=True)
class MethodCase:
    method: str
    a_partition: str
    b_partition: str
    c_partition: str
    replication_factor: int


def gpt3_expansion(m: int) -> ShapeCase:
    """Up-projection ``[m, 12288] @ [12288, 49152]``."""
    return ShapeCase("gpt3_expansion", f"GPT-3 expansion (k={GPT3_HIDDEN}, n={GPT3_FFN})", "m", m, m, GPT3_FFN, GPT3_HIDDEN)


def gpt3_shrinking(m: int) -> ShapeCase:
    """Down-projection ``[m, 49152] @ [49152, 12288]``."""
    return ShapeCase("gpt3_shrinking", f"GPT-3 shrinking (k={GPT3_FFN}, n={GPT3_HIDDEN})", "m", m, m, GPT3_HIDDEN, GPT3_FFN)


def square(size: int) -> ShapeCase:
    return ShapeCase("square", "Square matrices", "size", size, size, size, size)


def odd(which: str, big: int, small: int) -> ShapeCase:
    dims = {"m": small, "n": small, "k": small}
    dims[which] = big
    others = "=".join(d for d in "mnk" if d != which)
    return ShapeCase(f"odd_{which}_large", f"Odd-dimension: large {which} ({others}={small})", which, big,
                     dims["m"], dims["n"], dims["k"])


def build_shape_suite(*, gpt3_m_values, square_sizes, odd_large_values, odd_small_value) -> list[ShapeCase]:
    suite = [gpt3_expansion(m) for m in gpt3_m_values]
    suite += [gpt3_shrinking(m) for m in gpt3_m_values]
    suite += [square(s) for s in square_sizes]
    for big in odd_large_values:
        suite += [odd(w, big, odd_small_value) for w in ("m", "n", "k")]
    return suite


def case_key(shape: ShapeCase, method: MethodCase) -> str:
    return (f"{shape.experiment_group}_m{shape.m}_n{shape.n}_k{shape.k}_{method.method}"
            f"_A{method.a_partition}B{method.b_partition}C{method.c_partition}_rep{method.replication_factor}")


def merged_row(shape: ShapeCase, method: MethodCase, worker_result: dict) -> dict:
    row = {"experiment_group": shape.experiment_group, "experiment_label": shape.experiment_label,
           "varied_dim": shape.varied_dim, "varied_value": shape.varied_value, "case_key": case_key(shape, method)}
    row.update(asdict(shape))
    row.update(asdict(method))
    row.update(worker_result)
    return row
