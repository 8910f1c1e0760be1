"""Real multi-process runs: gloo ranks on CPU (shared-memory world) here, one rank per GPU on
a multi-GPU box."""
import os
import subprocess
import sys

import pytest
import torch

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mgpu_worker.py")


def _launch(nproc, device, cases, port, timeout=900, extra_env=None, extra_args=()):
    env = dict(os.environ)
    env.update({"MASTER_ADDR": "127.0.0.1", "OMP_NUM_THREADS": "2"})
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), WORKER, "--device", device, "--cases", cases,
           *extra_args]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("nproc", [2, 4])
def test_cpu_gloo_shared_memory_world(nproc):
    proc = _launch(nproc, "cpu", "tiny", 29610 + nproc, extra_env={"UGEMM_GUARD_BYTES": "1024"})
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "failures=0" in proc.stdout
    assert "guarded allocations checked on rank 0: 0" not in proc.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("cases", ["small", "large"])
def test_multi_gpu_ipc_world(cases):
    """``small``: all 27 partition triples on an odd shape.  ``large``: shapes with several waves of tiles per rank
    and megabytes of staged remote operands, for every tile variant, static and dynamic tile order, replication 1
    and 2, fp32 and bf16 C, plus redistribute and put + signal between GPUs (see mgpu_worker.large_cases)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    nproc = 8 if n >= 8 else 4 if n >= 4 else 2
    proc = _launch(nproc, "cuda", cases, 29650 if cases == "small" else 29660,
                   extra_env={"NCCL_NVLS_ENABLE": "0", "UGEMM_GUARD_BYTES": "4096"})
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "failures=0" in proc.stdout


@pytest.mark.gpu
def test_multi_gpu_torch_symmetric_memory_world():
    """The same worker on a world whose symmetric allocations come from ``torch.distributed._symmetric_memory``
    (multicast binding switched off): the kernels only ever see a table of peer pointers."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    proc = _launch(2, "cuda", "tiny", 29670, extra_env={"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"},
                   extra_args=("--world", "symm_mem"))
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "failures=0" in proc.stdout
