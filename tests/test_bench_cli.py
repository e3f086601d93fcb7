"""Command lines of the benchmark programs: argument checks that need no GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
AR = os.path.join(ROOT, "bin", "allreduce")
RS = os.path.join(ROOT, "bin", "reducescatter")



@pytest.fixture(scope="module", autouse=True)
def _programs():
    """The programs are build products (not in the source tree): build them when they are missing."""
    if not (os.path.exists(AR) and os.path.exists(RS)):
        import shutil
        import sys
        if not (shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc")):
            pytest.skip("bin/allreduce is not built and there is no nvcc to build it")
        sys.path.insert(0, ROOT)
        from stragglar_b200 import build
        build.build_bench()


def test_allreduce_usage():
    p = subprocess.run([AR], capture_output=True, text=True)
    assert p.returncode != 0 and "Usage:" in p.stderr and "<bufferSize> <algorithm> <numIters> <sleepTimeMs>" in p.stderr


def test_allreduce_rejects_unknown_algorithm():
    p = subprocess.run([AR, "1024", "tree", "1", "-1"], capture_output=True, text=True)
    assert p.returncode != 0 and "Invalid algorithm: tree" in p.stderr


def test_reducescatter_usage():
    p = subprocess.run([RS], capture_output=True, text=True)
    assert p.returncode != 0 and "Usage:" in p.stderr and "<bufferSize> <numIters>" in p.stderr


def test_bench_py_reference_arm_without_the_program(tmp_path):
    # 2 GPUs: the reference has no program for that count and says so in one JSON line
    import json
    import sys
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, env={**os.environ, "RANK": "0", "WORLD_SIZE": "1"})
    assert p.returncode == 0
    out = json.loads(p.stdout.strip().splitlines()[-1])
    assert out["impl"] == "reference" and "unavailable" in out
