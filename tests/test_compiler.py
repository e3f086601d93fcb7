"""Schedule compiler: every algorithm lowers to hazard-free tables whose
execution (host threads walking the tables like the kernels do) gives the
fp64 oracle's sum; wrong plans and wrong schedules are refused."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from helpers import chunk_bounds, emulate_prephase, oracle_sum, seeded_inputs
from stragglar_b200 import compiler as sc
from stragglar_b200.schedule import OneWayMatching, Schedule
from stragglar_b200.synth import synthesize

BUILTIN_N = (2, 4, 6, 8, 10, 12, 16)


def _run(alg, n, count, prephase=True, straggler=None, scale=1.0, dtype=np.float32, blocks=3, tile=64, delay=None):
    prog = sc.compile_program(alg, n, prephase, straggler)
    bufs = seeded_inputs(n, count, dtype)
    want = oracle_sum(bufs) * scale
    if not prephase:
        emulate_prephase(bufs, alg, n - 1 if straggler is None else straggler)
    status = sc.host_allreduce(prog, bufs, scale=scale, blocks=blocks, tile_elems=tile, delay_ms=delay)
    assert status == 0, sc.status_string(status)
    return prog, bufs, want


@pytest.mark.parametrize("alg", ["stragglar", "stragglar_a2a", "ring", "rhd", "direct", "rsag"])
@pytest.mark.parametrize("n", [2, 4, 6, 8])
def test_allreduce_algorithms(alg, n):
    if alg == "rhd" and n & (n - 1):
        with pytest.raises(sc.CompileError):
            sc.compile_program(alg, n)
        return
    prog, bufs, want = _run(alg, n, 4099)
    for b in bufs:
        np.testing.assert_allclose(b, want, atol=1e-5)


@pytest.mark.parametrize("alg", ["stragglar", "stragglar_a2a", "direct"])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_prephase_already_done(alg, n):
    prog, bufs, want = _run(alg, n, 2050, prephase=False)
    for b in bufs:
        np.testing.assert_allclose(b, want, atol=1e-5)


def test_round_counts():
    assert sc.compile_table("stragglar", 8, prephase=False).num_rounds == 9
    assert sc.compile_table("stragglar", 8).num_rounds == 10      # + the reduce-scatter pre-phase
    assert sc.compile_table("stragglar", 4, prephase=False).num_rounds == 4
    assert sc.compile_table("stragglar", 6, prephase=False).num_rounds == 7
    assert sc.compile_table("ring", 8).num_rounds == 14
    assert sc.compile_table("rhd", 8).num_rounds == 6
    assert sc.compile_table("direct", 8, prephase=False).num_rounds == 3
    assert [p.channel for p in sc.compile_program("direct", 8).phases] == [1, 0]


def test_link_traffic():
    # straggler: 7 matchings (1 chunk each way) + 2 one-way sends -> 9 chunks out
    t = sc.compile_table("stragglar", 8, prephase=False)
    assert t.ranks[7].chunks_out == 9 and t.link_chunks() == 9
    assert sc.compile_table("ring", 8).link_chunks() == 14
    assert sc.compile_table("stragglar_a2a", 8, prephase=False).link_chunks() == 7


@pytest.mark.parametrize("straggler", [0, 2, 5])
def test_straggler_swap(straggler):
    # the late rank plays logical rank n-1; with a real delay on that physical rank
    n = 8
    delay = [0.0] * n
    delay[straggler] = 20.0
    prog, bufs, want = _run("stragglar", n, 3001, straggler=straggler, delay=delay)
    for b in bufs:
        np.testing.assert_allclose(b, want, atol=1e-5)
    t = prog.main
    pushes = [int((r.ops["kind"] == sc.REDUCE_PUSH).sum()) for r in t.ranks]
    assert pushes[straggler] == n - 1 and sorted(pushes)[:-1] == [1] * (n - 1)


def test_fused_scale_applies_once():
    for alg in ("stragglar", "ring", "rhd", "direct", "rsag", "stragglar_a2a"):
        prog, bufs, want = _run(alg, 8, 1027, scale=0.125)
        for b in bufs:
            np.testing.assert_allclose(b, want, atol=1e-5, err_msg=alg)


def test_single_rank_scale():
    prog, bufs, want = _run("stragglar", 1, 1001, scale=0.5)
    np.testing.assert_allclose(bufs[0], want, atol=1e-6)


def test_reduce_scatter():
    n, count = 7, 5003
    t = sc.compile_table("reducescatter", n)
    bufs = seeded_inputs(n, count)
    want = oracle_sum(bufs)
    assert sc.host_allreduce(t, bufs, blocks=2, tile_elems=128) == 0
    for r, (b, e) in enumerate(chunk_bounds(count, 4, n)):
        np.testing.assert_allclose(bufs[r][b:e], want[b:e], atol=1e-5)


def test_bf16_bits():
    import torch
    n, count = 4, 1030
    xs = [torch.empty(count).uniform_(-1, 1, generator=torch.Generator().manual_seed(r)).bfloat16() for r in range(n)]
    want = torch.stack([x.double() for x in xs]).sum(0)
    bufs = [x.view(torch.uint16).numpy().copy() for x in xs]
    assert sc.host_allreduce(sc.compile_program("stragglar", n), bufs, blocks=2, tile_elems=64) == 0
    for b in bufs:
        got = torch.from_numpy(b.copy()).view(torch.bfloat16).double()
        torch.testing.assert_close(got, want, atol=0.05, rtol=0.02)
    # both sides of a straggler matching store the same rounded sum: all ranks agree bit for bit
    assert all((b == bufs[0]).all() for b in bufs)


def test_repeated_collectives_reuse_flags():
    n = 4
    t = sc.compile_table("ring", n)
    bufs = [np.full(515, float(r + 1), dtype=np.float32) for r in range(n)]
    assert sc.host_allreduce(t, bufs, blocks=2, tile_elems=32, repeats=3) == 0
    for b in bufs:
        np.testing.assert_allclose(b, 10.0 * n * n)  # sum, then twice more n times the previous


def test_tiny_and_ragged_sizes():
    for count in (1, 3, 4, 7, 29, 33):
        prog, bufs, want = _run("stragglar", 8, count, tile=4)
        for b in bufs:
            np.testing.assert_allclose(b, want, atol=1e-5)


def test_custom_schedule_text():
    s = synthesize(8)
    prog = sc.compile_program("stragglar", 8, schedule=s)
    assert prog.main.num_rounds == len(s) + 1
    # a schedule that forwards a chunk before its holder has it must be refused
    bad = Schedule(8, [list(r) for r in s.rounds])
    bad.rounds[0].append(OneWayMatching(3, 4, 0))
    with pytest.raises(sc.CompileError):
        sc.compile_program("stragglar", 8, schedule=bad)


def test_missing_last_round_is_refused():
    s = synthesize(8)
    with pytest.raises(sc.CompileError, match="ends without the full sum"):
        sc.compile_program("stragglar", 8, schedule=Schedule(8, s.rounds[:-1]))


def test_unknown_algorithm():
    with pytest.raises(sc.CompileError, match="Invalid algorithm"):
        sc.compile_program("tree", 8)


def test_late_rank_times_out_instead_of_hanging():
    # rank 3 "arrives" after the deadline: everybody returns a timeout status
    n = 4
    prog = sc.compile_program("stragglar", n)
    bufs = seeded_inputs(n, 512)
    status = sc.host_allreduce(prog, bufs, blocks=1, tile_elems=64, delay_ms=[0, 0, 0, 1500.0], timeout_s=0.3)
    assert status != 0 and "timeout" in sc.status_string(status) or "aborted" in sc.status_string(status)


@settings(max_examples=25, deadline=None)
@given(n=st.sampled_from(BUILTIN_N), count=st.integers(1, 3000), straggler=st.integers(0, 15),
       alg=st.sampled_from(["stragglar", "stragglar_a2a", "ring", "direct", "rsag"]),
       tile=st.sampled_from([4, 16, 64, 1024]), blocks=st.integers(1, 4))
def test_property_any_size_any_straggler(n, count, straggler, alg, tile, blocks):
    straggler %= n
    prog, bufs, want = _run(alg, n, count, straggler=straggler, blocks=blocks, tile=tile)
    for b in bufs:
        np.testing.assert_allclose(b, want, atol=2e-5)


def test_forwarding_lane_and_merged_pushes(monkeypatch):
    monkeypatch.setenv("STRAGGLAR_COPY", "push")
    monkeypatch.setenv("STRAGGLAR_LANES", "2")
    t = sc.compile_table("stragglar_a2a", 8)
    ops = t.ranks[0].ops
    kinds = [(int(o["kind"]), int(o["round"]), int(o["lane"]), int(o["nsrc"]), int(o["part"]), int(o["parts"])) for o in ops]
    # pre-phase reduce (6 peers), the rank's half of its matching, then its final chunk pushed to the
    # six other non-stragglers as two interleaved half-chunk ops in the forwarding lane
    assert kinds == [(sc.REDUCE, 0, 0, 6, 0, 1), (sc.REDUCE_PUSH, 1, 0, 1, 0, 2),
                     (sc.PUSH, 2, 1, 6, 0, 2), (sc.PUSH, 2, 1, 6, 1, 2)]
    # the straggler only has matchings: no forwarding lane, all of its blocks serve them
    assert all(int(o["lane"]) == 0 and int(o["kind"]) == sc.REDUCE_PUSH for o in t.ranks[7].ops)
    # within a round lane 0 comes first
    s = sc.compile_table("stragglar", 8)
    for r in s.ranks:
        key = [(int(o["round"]), int(o["lane"])) for o in r.ops]
        assert key == sorted(key)
    # ring has no matchings: one lane, whole-chunk ops
    assert all(int(o["lane"]) == 0 and int(o["parts"]) == 1 for r in sc.compile_table("ring", 8).ranks for o in r.ops)


@pytest.mark.parametrize("copy,lanes", [("pull", "1"), ("pull", "2"), ("push", "1"), ("push", "2")])
def test_every_lowering_gives_the_same_sum(monkeypatch, copy, lanes):
    monkeypatch.setenv("STRAGGLAR_COPY", copy)
    monkeypatch.setenv("STRAGGLAR_LANES", lanes)
    for alg in ("stragglar", "stragglar_a2a", "direct"):
        for blocks in (1, 2, 5):
            prog, bufs, want = _run(alg, 8, 3001, blocks=blocks, tile=32)
            for b in bufs:
                np.testing.assert_allclose(b, want, atol=1e-5, err_msg=f"{alg} {copy} {lanes} {blocks}")


def test_block_count_hints():
    assert sc.compile_table("stragglar", 8).blocks_hint == 64
    a2a = sc.compile_table("stragglar_a2a", 8)
    assert a2a.blocks_hint == 48 and a2a.stages_hint == 3
    assert sc.compile_table("ring", 8).blocks_hint == 0
    assert sc.compile_table("stragglar", 2).blocks_hint == 0 and sc.compile_table("stragglar", 1).blocks_hint == 0
    assert [t.blocks_hint for t in sc.compile_program("direct", 8).phases] == [0, 0]


def test_table_listing_cli(capsys):
    assert sc.main(["stragglar", "4", "--no-prephase"]) == 0
    text = capsys.readouterr().out
    assert "phase 0" in text and "match" in text and "rank 3" in text
    assert sc.main(["rhd", "6"]) == 1 and "power-of-two" in capsys.readouterr().out


def test_round_gating_attribute_and_host_execution(monkeypatch):
    """STRAGGLAR_GATE marks tables for round gating (rounds one after the other); the host executor runs gated
    tables of every algorithm to the same sums, with several threads per rank and a late straggler."""
    import numpy as np
    from helpers import oracle_sum, seeded_inputs

    monkeypatch.delenv("STRAGGLAR_GATE", raising=False)
    assert sc.compile_program("stragglar", 8).main.gate_rounds           # the default for the synthesized schedule
    assert not sc.compile_program("stragglar_a2a", 8).main.gate_rounds
    monkeypatch.setenv("STRAGGLAR_GATE", "1")
    assert sc.compile_program("stragglar", 8).main.gate_rounds
    assert not sc.compile_program("stragglar", 2).main.gate_rounds       # one round: nothing to gate
    assert not sc.compile_program("ring", 8).main.gate_rounds            # "1" gates the synthesized schedule only
    monkeypatch.setenv("STRAGGLAR_GATE", "all")
    for alg, n, slack in (("stragglar", 8, 0), ("stragglar", 8, 5), ("stragglar", 6, 0), ("stragglar_a2a", 4, 2), ("ring", 4, 0),
                          ("rhd", 8, 0), ("direct", 4, 0), ("rsag", 4, 3)):
        # slack 0: a full barrier between rounds, gated items skip their flag waits; slack s: a round opens when
        # all but s items before it are done and items wait for their flags as usual
        monkeypatch.setenv("STRAGGLAR_GATE_SLACK", str(slack))
        prog = sc.compile_program(alg, n)
        assert prog.main.gate_rounds, alg
        bufs = seeded_inputs(n, 20_011)
        want = oracle_sum(bufs)
        delay = [0.0] * n
        delay[n - 1] = 3.0
        assert sc.host_allreduce(prog, bufs, blocks=3, tile_elems=256, delay_ms=delay) == 0
        for b in bufs:
            np.testing.assert_allclose(b.astype(np.float64), want, atol=2e-5)
        if len(prog.phases) == 1:
            # twice in a row on the same control words (the second epoch): the sum of n equal sums
            assert sc.host_allreduce(prog.main, bufs, blocks=3, tile_elems=256, repeats=2) == 0
            for b in bufs:
                np.testing.assert_allclose(b.astype(np.float64), want * n * n, rtol=1e-5, atol=1e-3)
    monkeypatch.setenv("STRAGGLAR_GATE", "0")
    assert not sc.compile_program("stragglar", 8).main.gate_rounds


def test_lane_split_share(monkeypatch):
    """STRAGGLAR_LANE1_EIGHTHS moves blocks between the two lanes: every split runs to the same sums and the
    default (half, alternating) is unchanged."""
    import numpy as np
    from helpers import oracle_sum, seeded_inputs
    monkeypatch.delenv("STRAGGLAR_LANE1_EIGHTHS", raising=False)
    assert sc.compile_program("stragglar_a2a", 8).main.lane1_eighths == 4
    for e in ("2", "5", "7"):
        monkeypatch.setenv("STRAGGLAR_LANE1_EIGHTHS", e)
        prog = sc.compile_program("stragglar_a2a", 6)
        assert prog.main.lane1_eighths == int(e)
        bufs = seeded_inputs(6, 12_345)
        want = oracle_sum(bufs)
        assert sc.host_allreduce(prog, bufs, blocks=5, tile_elems=128) == 0
        for b in bufs:
            np.testing.assert_allclose(b.astype(np.float64), want, atol=2e-5)


def test_final_versions_match_the_ops():
    """The final version of every slot (what staged launches wait for) is the newest version any op gives it."""
    for alg, n in (("stragglar", 8), ("stragglar_a2a", 6), ("ring", 4), ("rsag", 4), ("rhd", 8)):
        t = sc.compile_table(alg, n)
        newest = [[0] * t.num_chunks for _ in range(n)]
        for r in range(n):
            for op in t.ranks[r].ops:
                kind, chunk = int(op["kind"]), int(op["chunk"])
                if kind != 3:                                   # everything but a push rewrites the own slot
                    newest[r][chunk] = max(newest[r][chunk], int(op["post_ver"]))
                if kind in (2, 3):                              # REDUCE_PUSH / PUSH rewrite the peers' slots
                    for q in range(int(op["nsrc"])):
                        peer = int(op["src"][q])
                        newest[peer][chunk] = max(newest[peer][chunk], int(op["push_ver"]))
        for r in range(n):
            assert t.final_versions(r) == newest[r], (alg, n, r)
            assert all(v >= 1 for v in newest[r])               # every slot ends rewritten (the sum lands everywhere)
