"""Synthesizers: byte-identical output to the reference tools for the sizes
they handle, working n = 2 and n = 4, and valid schedules everywhere."""
import hashlib
import io
import os
import subprocess
import sys
from contextlib import redirect_stdout

import pytest

from stragglar_b200.schedule import (OneWayMatching, Schedule, ScheduleError, StragglerMatching, TwoWayMatching)
from stragglar_b200.synth import nonpow2, pow2, synthesize

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _printed(mod, n):
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert mod.main(["prog", str(n)]) == 0
    return "".join(l for l in buf.getvalue().splitlines(True) if not l.startswith("Time taken"))


@pytest.mark.parametrize("n", [8, 16])
def test_pow2_matches_reference_text(n):
    assert _printed(pow2, n) == open(os.path.join(GOLD, f"pow2_{n}.txt")).read()


@pytest.mark.parametrize("n", [6, 10, 12])
def test_nonpow2_matches_reference_text(n):
    pytest.importorskip("networkx")
    assert _printed(nonpow2, n) == open(os.path.join(GOLD, f"nonpow2_{n}.txt")).read()


def test_large_outputs_match_reference_digest():
    want = dict(reversed(l.split()) for l in open(os.path.join(GOLD, "big_md5.txt")))
    assert hashlib.md5(_printed(pow2, 32).encode()).hexdigest() == want["pow2_32.txt"]
    import networkx
    if networkx.__version__ == "3.6.1":  # the matcher's tie-breaks are version dependent
        assert hashlib.md5(_printed(nonpow2, 14).encode()).hexdigest() == want["nonpow2_14.txt"]


def test_n4_is_the_hand_schedule():
    # the 4-round schedule hand-coded in stragglar/allreduce_4GPU.cu:307-363
    s = synthesize(4)
    assert s.rounds == [
        [StragglerMatching(0, 3, 0)],
        [StragglerMatching(1, 3, 1), OneWayMatching(0, 2, 0)],
        [StragglerMatching(2, 3, 2), TwoWayMatching(0, 1, 0, 1)],
        [TwoWayMatching(0, 2, 1, 2), OneWayMatching(3, 1, 2)],
    ]


def test_n2_single_round():
    assert synthesize(2).rounds == [[StragglerMatching(0, 1, 0)]]


@pytest.mark.parametrize("n", [2, 4, 8, 16, 32, 64])
def test_pow2_round_count_is_optimal(n):
    s = synthesize(n).validate()
    assert len(s) == s.optimal_rounds()


@pytest.mark.parametrize("n,rounds", [(6, 7), (10, 12), (24, 27)])
def test_nonpow2_round_counts(n, rounds):
    pytest.importorskip("networkx")
    assert len(synthesize(n).validate()) == rounds


@pytest.mark.parametrize("n", [6, 10, 12, 14])
def test_nonpow2_without_networkx_is_valid(n):
    s = nonpow2.synthesize(n, use_networkx=False).validate()
    assert len(s) <= s.optimal_rounds() + 2


def test_bad_arguments():
    with pytest.raises(ValueError):
        pow2.synthesize(6)
    with pytest.raises(ValueError):
        nonpow2.synthesize(8)
    with pytest.raises(ValueError):
        nonpow2.synthesize(7)
    assert pow2.main(["prog"]) == 1


def test_parse_round_trip():
    s = synthesize(8)
    again = Schedule.parse(s.format())
    assert again.n == 8 and again.rounds == s.rounds
    assert again.format() == s.format()


def test_validator_catches_errors():
    s = synthesize(8)
    broken = Schedule(8, [list(r) for r in s.rounds])
    broken.rounds[1].append(OneWayMatching(2, 5, 0))  # rank 2 does not hold chunk 0 yet
    with pytest.raises(ScheduleError):
        broken.validate()
    broken = Schedule(8, [list(r) for r in s.rounds])
    broken.rounds[2].append(OneWayMatching(0, 4, 0))  # rank 0 sends twice, rank 4 receives twice
    with pytest.raises(ScheduleError):
        broken.validate()
    with pytest.raises(ScheduleError):
        Schedule(8, s.rounds[:-1]).validate()


def test_straggler_never_sends_more_than_needed():
    s = synthesize(8)
    assert s.chunks_sent_by(7) == 9  # 7 matchings + 2 one-way sends of the last chunk


def test_cli_module_runs():
    out = subprocess.run([sys.executable, "-m", "stragglar_b200.synth.pow2", "8"], capture_output=True, text=True,
                         cwd=os.path.dirname(os.path.dirname(__file__)))
    assert out.returncode == 0
    assert "Actual number of rounds 9" in out.stdout and "Optimal number of rounds 9.0" in out.stdout


def test_rank_map_and_compact_form():
    s = synthesize(8)
    assert s.rank_map_for_straggler(2) == [0, 1, 7, 3, 4, 5, 6, 2]
    assert s.rank_map_for_straggler(7) == list(range(8))
    with pytest.raises(ScheduleError):
        s.rank_map_for_straggler(8)
    lines = s.compact().splitlines()
    assert lines[0] == "R0: 0<->7 c0" and lines[1] == "R1: 1<->7 c1 | 0->3 c0" and len(lines) == 9


def test_matchers_agree_on_cardinality_and_weight():
    from stragglar_b200.synth.matching import _exact, _greedy, max_weight_matching
    nodes = list(range(8))
    edges = [(0, 1, 2), (1, 2, 1), (2, 3, 2), (3, 4, 1), (4, 5, 2), (5, 6, 1), (6, 7, 2), (0, 7, 1), (1, 6, 1)]
    exact = _exact(nodes, edges)
    assert len(exact) == 4 and sum(w for u, v, w in edges if (u, v) in exact or (v, u) in exact) == 8
    nxm = max_weight_matching(nodes, edges)
    assert len(nxm) == 4
    g = _greedy(nodes, edges)
    assert len(g) == 4 and len({x for p in g for x in p}) == 8


def test_builtin_schedule_export_is_current():
    import contextlib
    from stragglar_b200.synth import export
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        export.main()
    path = os.path.join(os.path.dirname(os.path.dirname(__file__)), "csrc", "core", "builtin_schedules.inc")
    assert buf.getvalue() == open(path).read(), "run: python -m stragglar_b200.synth.export > csrc/core/builtin_schedules.inc"


@pytest.mark.parametrize("script,args,needle", [("synthesizer_pow2.py", ["8"], "Actual number of rounds 9"),
                                                ("synthesizer_nonpow2.py", ["6"], "Actual number of rounds 7"),
                                                ("pad_buffers.py", ["8"], "1073744896"),
                                                ("simulation.py", [], "Speedups for powers of two:")])
def test_reference_named_scripts(script, args, needle):
    root = os.path.dirname(os.path.dirname(__file__))
    out = subprocess.run([sys.executable, os.path.join(root, "stragglar", script), *args], capture_output=True, text=True)
    assert out.returncode == 0 and needle in out.stdout
