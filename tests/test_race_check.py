"""The table protocol under ThreadSanitizer: csrc/core/tests/host_exec_race_check.cpp
runs every algorithm and lowering with several host threads per rank; any
access to a buffer element that the flags do not order is reported as a data
race and fails the test."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_no_data_race_in_any_table(tmp_path):
    core = os.path.join(ROOT, "csrc", "core")
    exe = str(tmp_path / "race_check")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-pthread", "-Wno-nonnull",
                            os.path.join(core, "tests", "host_exec_race_check.cpp"), os.path.join(core, "plan.cpp"),
                            os.path.join(core, "host_exec.cpp"), "-o", exe], capture_output=True, text=True)
    if build.returncode != 0 and "tsan" in (build.stderr or "").lower():
        pytest.skip("ThreadSanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600,
                         env={**os.environ, "TSAN_OPTIONS": "halt_on_error=0 exitcode=66"})
    out = run.stdout + run.stderr
    assert "ThreadSanitizer" not in out, out[-3000:]
    assert run.returncode == 0 and "0 failures" in out, out[-2000:]
