"""Host-side failure detection: a control plane that does not depend on a process group, and ranks that
never arrive.  No GPU is involved; the GPU-side counterpart (a device wait that runs out and reports a
status code) is tests/test_fused_gpu.py::test_bounded_wait_reports_timeout_instead_of_hanging."""
import os
import subprocess
import sys

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "filecomm_worker.py")


def _spawn(directory, size, mode):
    procs = [subprocess.Popen([sys.executable, WORKER, str(directory), str(r), str(size), mode],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(size)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    return [p.returncode for p in procs], outs


def test_file_rendezvous_world_runs_a_gemm(tmp_path):
    codes, outs = _spawn(tmp_path, 3, "ok")
    assert codes == [0, 0, 0], "\n".join(outs)
    assert all("ok" in o for o in outs)


def test_absent_rank_is_reported_not_waited_for(tmp_path):
    codes, outs = _spawn(tmp_path, 3, "absent")
    assert codes == [3, 3, 0], "\n".join(outs)
    assert "rank 2 did not reach collective #0" in outs[0]
