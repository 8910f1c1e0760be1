"""The planners produce the reference planner's op lists, op for op and in the same order, for all 27 partition
triples x replication factors x world sizes on odd shapes (see ref_planner_compare.py).  Needs the verbatim copy of
the reference tree under ``baseline/_ref`` (git-ignored); skipped when it is absent."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(os.path.dirname(HERE), "baseline", "_ref")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "stationary_c_plan.py")), reason="baseline/_ref is absent")
def test_planners_match_the_reference_planners_op_for_op():
    proc = subprocess.run([sys.executable, os.path.join(HERE, "ref_planner_compare.py"), REF],
                          capture_output=True, text=True, timeout=1500)
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert lines, proc.stdout[-2000:] + proc.stderr[-2000:]
    res = json.loads(lines[-1])
    assert res["num_mismatches"] == 0, res["mismatches"]
    assert res["compared"] >= 4000, res
    assert proc.returncode == 0
