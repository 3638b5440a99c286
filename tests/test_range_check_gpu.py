"""The debug build (-DSP_RANGE_CHECK, chosen for a process by SPISSA_B200_RANGE_CHECK=1): kernels check the indices they
take from the tables the host packed, record a code and leave the access out. It stands in for a memory checker.
Both tests run child processes, because the build is chosen when the libraries are loaded."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def run(args, timeout=900):
    env = dict(os.environ, SPISSA_B200_RANGE_CHECK="1", PYTHONPATH=os.pathsep.join([ROOT, HERE]))
    return subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_an_index_beyond_the_declared_bounds_is_reported_and_the_access_left_out():
    proc = run([os.path.join(HERE, "range_check_cases.py")])
    assert proc.returncode == 0 and "range check cases ok" in proc.stdout, (proc.stdout + proc.stderr)[-3000:]


def test_the_replay_cuts_run_green_in_the_debug_build():
    proc = run(["-m", "pytest", os.path.join(HERE, "test_replay_gpu.py"), "-q", "-x", "-m", "gpu",
                "-k", "cuts_agree and (A- or B- or E-)"])
    assert proc.returncode == 0 and " passed" in proc.stdout, (proc.stdout + proc.stderr)[-3000:]
    assert "6 passed" in proc.stdout
