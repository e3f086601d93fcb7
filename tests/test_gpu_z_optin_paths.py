"""Paths that were written after the last GPU session: round gating, the simta data path, symmetric buffers.

Their tests in test_gpu_emulated.py / test_gpu_symmetric.py are switched on by environment variables.  Here each
group runs in a process of its own (so that a CUDA error stays in that process) and is reported as an expected
failure when it fails and as an unexpected pass when it passes: the run tells which of the new paths work on the
machine at hand without letting them decide the outcome of the suite.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

GROUPS = {
    "round_gating": ({"STRAGGLAR_TEST_GATE": "1"}, ["tests/test_gpu_emulated.py", "-k", "round_gating"]),
    "simta_path": ({"STRAGGLAR_TEST_SIMTA": "1"}, ["tests/test_gpu_emulated.py", "-k", "simta"]),
    "symmetric_buffers": ({"STRAGGLAR_TEST_SYMM": "1"}, ["tests/test_gpu_symmetric.py", "-k", "plain or single_rank"]),
}


@pytest.mark.xfail(strict=False, reason="written after the last GPU session; not yet exercised on a GPU")
@pytest.mark.parametrize("group", sorted(GROUPS))
def test_new_path_in_a_process_of_its_own(group):
    env_extra, args = GROUPS[group]
    env = dict(os.environ, **env_extra)
    p = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", *args], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=600)
    tail = (p.stdout or "")[-1500:]
    print(tail)
    assert p.returncode == 0, tail
    assert " passed" in tail and " failed" not in tail
