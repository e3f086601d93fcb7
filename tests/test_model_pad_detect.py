"""Analytical model, padding helper and straggler detection."""
import io
from contextlib import redirect_stdout

import pytest

from stragglar_b200 import detect, pad, simulate


def test_reference_speedups():
    sp, rhd, direct, ring = simulate.compute_speedups(simulate.POWERS_OF_TWO)
    assert [round(float(x), 3) for x in sp] == [1.127, 1.363, 1.565, 1.718, 1.826, 1.897, 1.941]
    assert [round(float(x), 3) for x in rhd] == [1.002, 1.006, 1.016, 1.036, 1.078, 1.162, 1.331]
    assert [round(float(x), 3) for x in direct] == [0.753, 0.589, 0.478, 0.404, 0.356, 0.332, 0.335]
    sp, rhd, direct, ring = simulate.compute_speedups(simulate.IN_BETWEEN)
    assert [round(float(x), 3) for x in sp] == [1.192, 1.346, 1.635, 1.617, 1.743, 1.829]
    assert [round(float(x), 3) for x in rhd] == [0.670, 0.675, 0.685, 0.706, 0.748, 0.833]


def test_absolute_times_n8():
    s, rhd, ring, direct = simulate.compute_costs([8])
    assert round(float(s[0]), 3) == 2.884 and round(float(ring[0]), 3) == 3.931
    assert round(float(rhd[0]), 3) == 3.907 and round(float(direct[0]), 3) == 6.676


def test_model_rounds_match_synthesizer():
    from stragglar_b200.synth import synthesize
    for n in (4, 8, 16):
        assert len(synthesize(n)) == simulate.stragglar_rounds(n)
    assert len(synthesize(6)) == simulate.NONPOW2_ROUNDS[6]


def test_printed_lines():
    buf = io.StringIO()
    with redirect_stdout(buf):
        simulate.main([])
    lines = buf.getvalue().splitlines()
    assert lines[0].startswith("Speedups for powers of two: [") and lines[1].startswith(
        "Speedups for non-power-of-two values: [")
    assert len(lines) == 2


def test_b200_model_is_faster_link():
    a = simulate.compute_costs([8], simulate.LinkModel.b200())[0][0]
    b = simulate.compute_costs([8])[0][0]
    assert a < b


def test_padding_values():
    assert pad.padded_sizes(8)[-1] == 1073744896 and pad.padded_sizes(4)[-1] == 1073743872
    assert pad.padded_sizes(8)[0] == 265216
    for n in (2, 4, 6, 8):
        for raw, p in zip(pad.BUFFER_SIZES, pad.padded_sizes(n)):
            assert p >= raw and p % ((n - 1) * 1024) == 0 and p // (n - 1) > raw // (n - 1)


def test_pad_cli():
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert pad.main(["pad", "8"]) == 0
    assert buf.getvalue().splitlines()[1].startswith("Padded buffer sizes:  265216 1053696")
    assert pad.main(["pad"]) == 1


LOG = """noise
\x1b[92mRank 1 | Step 0 | Forward Time: 1.0 ms | Backward Time: 2.0 ms  | Loss: 5.5 | Iteration Time: 6.0 ms | AR Time: 900.00 ms | AR Buffer Size: 1.00 KB\x1b[0m
Rank 0 | Step 0 | Forward Time: 1.0 ms | AR Time: 1000.00 ms | x Rank 2 | Step 0 | Forward Time: 1.0 ms | AR Time: 800.00 ms | y
Rank 0 | Step 1 | Forward Time: 1.0 ms | AR Time: 141.00 ms | x
Rank 1 | Step 1 | Forward Time: 1.0 ms | AR Time: 146.00 ms | x
Rank 2 | Step 1 | Forward Time: 1.0 ms | AR Time: 118.00 ms | x
Rank 0 | Step 2 | Forward Time: 1.0 ms | AR Time: 145.00 ms | x
Rank 1 | Step 2 | Forward Time: 1.0 ms | AR Time: 139.00 ms | x
Rank 2 | Step 2 | Forward Time: 1.0 ms | AR Time: 118.50 ms | x
"""


def test_detect_from_log():
    table = detect.parse_ar_times(LOG.splitlines(True))
    assert table[0] == {1: 900.0, 0: 1000.0, 2: 800.0}
    rep = detect.analyse(table)
    assert rep.straggler == 2 and rep.share[2] == 100.0
    assert rep.delays_ms == [pytest.approx(23.0), pytest.approx(20.5)]
    assert rep.median_delay_ms == pytest.approx(21.75)


def test_online_detector():
    d = detect.OnlineDetector(4, window=5, threshold=0.8)
    for _ in range(4):
        d.update([140, 139, 118, 130])
    assert d.recommendation() is None
    d.update([140, 100, 118, 130])
    assert d.recommendation() == 2
    a = detect.OnlineDetector(3, window=2, arrival=True)
    a.update([0.1, 0.2, 5.0]); a.update([0.1, 0.3, 7.0])
    assert a.recommendation() == 2


def test_log_line_round_trip_and_detection():
    from stragglar_b200.utils.logfmt import format_step, parse_step
    line = format_step(2, 7, 1499.21, 3032.68, 5.3932, 4815.84, 117.94, 12850999296)
    rec = parse_step(line)
    assert rec["rank"] == 2 and rec["step"] == 7 and rec["ar_ms"] == 117.94 and rec["forward_ms"] == 1499.21
    table = detect.parse_ar_times([line + "\n", format_step(0, 7, 1.0, 2.0, 5.0, 9.0, 141.09, 1024) + "\n"])
    assert table == {7: {2: 117.94, 0: 141.09}}


def test_env_report_runs_without_a_gpu():
    from stragglar_b200.utils import env_check
    info = env_check.report()
    assert "torch" in info and isinstance(info["gpus"], list)


def test_detect_on_the_shipped_training_log():
    import os
    log = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "logs",
                       "log_8_b200_llama1b_stragglar.txt")
    with open(log) as f:
        rep = detect.analyse(detect.parse_ar_times(f), skip_delay_steps=3)
    assert rep.straggler == 7            # the rank that was held back 20 ms per step
    assert 15.0 < rep.median_delay_ms < 25.0


def test_detect_cli_writes_the_delay_cdf(tmp_path, capsys):
    log = tmp_path / "train.log"
    log.write_text(LOG)
    out = tmp_path / "cdf.csv"
    assert detect.main([str(log), "--cdf", str(out), "--skip", "0"]) == 0
    assert "straggler: rank 2" in capsys.readouterr().out
    rows = out.read_text().strip().splitlines()
    assert rows[0] == "delay_ms,fraction"
    pts = [tuple(map(float, r.split(","))) for r in rows[1:]]
    assert pts == sorted(pts) and pts[-1][1] == 1.0 and len(pts) == 3


def test_online_detector_reports_when_nobody_is_persistently_late():
    d = detect.OnlineDetector(4, window=4, threshold=0.75)
    for times in ([9, 1, 9, 9], [9, 1, 9, 9], [9, 1, 9, 9]):
        d.update(times)
    assert not d.no_straggler()              # the window is not full yet
    d.update([9, 1, 9, 9])
    assert d.recommendation() == 1 and not d.no_straggler()
    for times in ([1, 9, 9, 9], [9, 9, 1, 9], [9, 9, 9, 1]):
        d.update(times)
    assert d.recommendation() is None and d.no_straggler()
    d.update([9, 9, 9, 1])
    assert d.recommendation() is None and not d.no_straggler()   # between the two fractions nothing changes


def test_cpu_affinity_from_a_fake_nvml(monkeypatch):
    import os

    from stragglar_b200.utils import affinity

    assert affinity.cpus_from_masks([0b1011, 0b1]) == [0, 1, 3, 64]

    class FakeNvml:
        def __init__(self, masks):
            self.masks, self.calls = masks, []
        def nvmlInit(self): self.calls.append("init")
        def nvmlShutdown(self): self.calls.append("shutdown")
        def nvmlDeviceGetHandleByIndex(self, i): self.calls.append(("handle", i)); return i
        def nvmlDeviceGetCpuAffinity(self, h, words): return self.masks

    mine = sorted(os.sched_getaffinity(0))
    keep = mine[: max(1, len(mine) // 2)]
    mask = 0
    for c in keep:
        mask |= 1 << c
    words = [(mask >> (64 * i)) & (2**64 - 1) for i in range(max(keep) // 64 + 1)]
    try:
        monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,5")
        fake = FakeNvml(words)
        assert affinity.bind_to_gpu(1, fake) == keep and sorted(os.sched_getaffinity(0)) == keep
        assert ("handle", 5) in fake.calls and fake.calls[-1] == "shutdown"
        # CPUs the process may not use, or no answer at all: nothing changes
        assert affinity.bind_to_gpu(0, FakeNvml([0, 0, 0, 1 << 62])) is None
        assert affinity.bind_to_gpu(0, object()) is None
        assert sorted(os.sched_getaffinity(0)) == keep
    finally:
        os.sched_setaffinity(0, mine)


def test_simulate_table_with_the_switched_algorithms(capsys):
    from stragglar_b200 import simulate
    assert simulate.main(["--b200", "--table"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert lines[0].split()[:4] == ["n", "stragglar", "a2a", "ring"] and len(lines) == 1 + 13
    row8 = dict(zip(lines[0].split(), lines[[l.split()[0] for l in lines].index("8")].split()))
    # 1 GiB at 770 GB/s: S*b = 1.394 ms; a2a moves S per direction, the ring 1.75 S, StragglAR 9/7 S
    assert abs(float(row8["a2a"]) - 1.400) < 2e-3 and abs(float(row8["ring"]) - 2.468) < 2e-3
    assert abs(float(row8["stragglar"]) - (9 * 0.002 + 9 / 7 * 1.39445)) < 2e-3
    a2a, rsag = simulate.compute_costs_switched([4, 8], simulate.LinkModel.b200())
    assert a2a[0] == a2a[1] and rsag[0] < rsag[1]


