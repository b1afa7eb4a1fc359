"""The checked build of the kernel library (``-DRA_BOUNDS_CHECK``) and canary-padded outputs: the stand-in for
a memory checker. The checked library is a separate shared object, so the kernels run in a child process."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(env_extra):
    env = dict(os.environ, **env_extra)
    p = subprocess.run([sys.executable, os.path.join(HERE, "bounds_worker.py")], capture_output=True, text=True,
                       timeout=900, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("BOUNDS ")][-1]
    return json.loads(line[len("BOUNDS "):])


def test_checked_build_finds_nothing_at_ragged_shapes_and_canaries_survive():
    rep = _run({"RINGATTN_B200_BOUNDS_CHECK": "1"})
    assert rep["clean"]["checked"] is True
    assert rep["clean"]["violations"] == 0, rep["clean"]
    assert rep["canaries_intact"] is True
    # the recorder works: the out-of-vocabulary token of the last step was counted and named
    assert rep["seeded"]["violations"] >= 1
    assert rep["seeded"]["first"]["access"] == "embedding token id"
    assert rep["seeded"]["first"]["index"] == 5000 and rep["seeded"]["first"]["limit"] == 1000


def test_normal_build_reports_unchecked_and_canaries_survive():
    rep = _run({"RINGATTN_B200_BOUNDS_CHECK": "0"})
    assert rep["clean"]["checked"] is False and rep["clean"]["violations"] == 0
    assert rep["canaries_intact"] is True
