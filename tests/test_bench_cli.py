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


def test_tune_ranks_settings_with_a_fake_program(tmp_path, monkeypatch, capsys):
    """bench/tune.py: runs one program per setting, reads the CSV, ranks the settings per algorithm and size."""
    import importlib.util
    import stat
    import sys
    spec = importlib.util.spec_from_file_location("tune", os.path.join(ROOT, "bench", "tune.py"))
    tune = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tune)
    fake = tmp_path / "allreduce"
    # time = size / blocks, gating takes a fifth off; one setting fails
    fake.write_text("#!/usr/bin/env python3\n"
                    "import os, sys\n"
                    "sizes, alg, iters, delay = sys.argv[1].split(','), sys.argv[2], int(sys.argv[3]), sys.argv[4]\n"
                    "b = int(os.environ.get('STRAGGLAR_BLOCKS', '128'))\n"
                    "if os.environ.get('STRAGGLAR_PATH') == 'simta': sys.stderr.write('collective failed\\n'); sys.exit(2)\n"
                    "print('algorithm,buffer_size_bytes,iteration,delay,runtime_ms,BW(GB/s),n,dtype,path,time_us_max,algbw_GBps,busbw_GBps,roofline_frac,real_delay_ms')\n"
                    "for s in sizes:\n"
                    "    for i in range(iters):\n"
                    "        ms = int(s) / 1e6 / b * (0.8 if os.environ.get('STRAGGLAR_GATE') == '1' else 1.0)\n"
                    "        print(f'{alg},{s},{i+1},{delay},{ms:.3f},1.0,8,float32,tma,0,0,0,0,0.000')\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setattr(tune, "EXE", str(fake))
    monkeypatch.setattr(sys, "argv", ["tune.py", "--sizes", "1048576,2097152", "--iters", "3", "--out", str(tmp_path / "raw")])
    assert tune.main() == 0
    out = capsys.readouterr().out
    block = out.split("stragglar, 1 MiB (net ms, best first)")[1].split("stragglar, 2 MiB")[0]
    ranked = [l.split(None, 1)[1] for l in block.strip().splitlines()]
    assert ranked[0] == "blocks=128 gate=1" and ranked[1] == "blocks=128"
    assert "path=simta blocks=64 [FAILED: collective failed]" in out
    assert (tmp_path / "raw" / "stragglar_blocks128_gate1.csv").exists()


def test_bench_py_times_experimental_lowerings_with_the_benchmark_program(tmp_path, monkeypatch):
    """bench.py asks bin/allreduce for the lowerings that are not the default yet; a failing run is reported, not fatal."""
    import importlib.util
    import stat
    spec = importlib.util.spec_from_file_location("bench_main", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    (tmp_path / "bin").mkdir()
    fake = tmp_path / "bin" / "allreduce"
    fake.write_text("#!/usr/bin/env python3\n"
                    "import os, sys\n"
                    "size, alg, iters, delays = int(sys.argv[1]), sys.argv[2], int(sys.argv[3]), sys.argv[4].split(',')\n"
                    "assert os.environ['STRAGGLAR_NGPUS'] == '8' and 'RANK' not in os.environ\n"
                    "if os.environ.get('STRAGGLAR_LANE1_EIGHTHS'): sys.stderr.write('collective failed in iteration 0\\n'); sys.exit(2)\n"
                    "ms = 2.0 if os.environ.get('STRAGGLAR_GATE') == '1' else 2.5\n"
                    "print('algorithm,buffer_size_bytes,iteration,delay,runtime_ms,BW(GB/s),n,dtype,path,time_us_max,algbw_GBps,busbw_GBps,roofline_frac,real_delay_ms')\n"
                    "for d in delays:\n"
                    "    real = max(float(d), 0.0)\n"
                    "    for i in range(iters):\n"
                    "        print(f'{alg},{size},{i+1},{float(d):.3f},{ms + real:.3f},1.0,8,float32,tma,0,0,0,0,{real:.3f}')\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    monkeypatch.setenv("RANK", "0")
    out = bench.experimental_lowerings(8, 1 << 30, 5.0)
    assert abs(out["stragglar_gated"]["delay_-1.000"]["time_us_net"] - 2000.0) < 1e-6
    assert abs(out["stragglar_gated"]["delay_5.000"]["time_us_net"] - 2000.0) < 1e-6
    assert abs(out["stragglar_default_lowering"]["delay_-1.000"]["time_us_net"] - 2500.0) < 1e-6
    assert "collective failed" in out["stragglar_a2a_lane1_5of8"]["error"]
    assert bench.experimental_lowerings(2, 1 << 30, 5.0) == {}          # nothing to try below four ranks
    monkeypatch.setenv("STRAGGLAR_BENCH_EXPERIMENTS", "0")
    assert bench.experimental_lowerings(8, 1 << 30, 5.0) == {}
