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


def test_both_arms_describe_the_same_configuration():
    """bench.py: the two arms use the same byte count and print the same `config` entry."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_main", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for n in (1, 2, 4, 8):
        b = bench.bench_bytes(0, n)
        assert b % (4 * max(n - 1, 1)) == 0 and abs(b - (1 << 30)) < 8192
        assert bench.bench_config("stragglar", n, b, 5.0, n - 1) == bench.bench_config("stragglar", n, b, 5.0, n - 1)
    assert bench.bench_bytes(1000, 8) == 980
    assert set(bench.bench_config("ring", 8, 64, 0.0, 7)) == {"model", "bytes_per_gpu", "delay_ms", "straggler_rank",
                                                               "global_batch", "seq_len", "parallelism", "l2"}


def test_summarize_reads_old_and_new_csv_rows(tmp_path, capsys):
    """bench/summarize.py: rows of the reference (6 columns), of earlier runs (14) and of the current program (15, with the
    in-kernel time) summarise side by side; the delay is taken off the net time."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("summarize", os.path.join(ROOT, "bench", "summarize.py"))
    sm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sm)
    f = tmp_path / "mixed.csv"
    f.write_text("algorithm,buffer_size_bytes,iteration,delay,runtime_ms,BW(GB/s)\n"
                 "stragglar,1048576,1,5.000,6.000,1.0\n"
                 "ring,1048576,1,-1.000,2.000,1.0,8,float32,tma,2000.0,0.5,0.9,0.800,0.000\n"
                 "rsag:blocks=64,1048576,1,5.000,7.500,1.0,8,float32,tma,7500.0,0.4,0.7,0.700,5.005,123.4\n"
                 "Rank 0, done\n")
    sm.main([str(f)])
    out = capsys.readouterr().out
    rows = {l.split()[1]: l.split() for l in out.strip().splitlines()[1:]}
    assert abs(float(rows["stragglar/ref"][5]) - 1.0) < 1e-9            # nominal delay taken off the reference's row
    assert abs(float(rows["rsag:blocks=64/tma"][5]) - 2.495) < 1e-9     # measured delay taken off
    assert rows["rsag:blocks=64/tma"][8] == "123.4" and rows["ring/tma"][8] == "nan"
