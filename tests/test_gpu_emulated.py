"""The CUDA table executor with all ranks emulated on one device (a single
cooperative launch), against a plain PyTorch fp32/fp64 reference.  Both data
paths (simt loads/stores and the bulk-copy pipeline) run the same tables."""
import os

import pytest
import torch

from stragglar_b200 import compiler as sc

pytestmark = pytest.mark.gpu

# simt: every thread moves vectors; tma: the bulk-copy pipeline; simta: the simt data path with control and
# signalling in threads of their own
PATHS = ["simt", "tma", "simta"]


def _inputs(n, count, dtype, dev="cuda:0"):
    from stragglar_b200 import ops
    xs = [torch.empty(count, dtype=dtype, device=dev) for _ in range(n)]
    for r, x in enumerate(xs):
        ops.fill_uniform(x, seed=r)
    torch.cuda.synchronize()
    return xs


def _prephase(xs, alg, straggler):
    n = len(xs)
    non = [r for r in range(n) if r != straggler]
    part = torch.stack([xs[r].float() for r in non]).sum(0).to(xs[0].dtype)
    if alg == "direct":
        for r in non:
            xs[r].copy_(part)
        return
    from helpers import chunk_bounds
    l2p = list(range(n))
    l2p[n - 1], l2p[straggler] = straggler, n - 1
    for i, (b, e) in enumerate(chunk_bounds(xs[0].numel(), xs[0].element_size(), n - 1)):
        xs[l2p[i]][b:e] = part[b:e]


def _run(alg, n, count, dtype=torch.float32, path="simt", prephase=True, straggler=None, scale=1.0, blocks=2,
         tile_bytes=4096, delay_ms=None):
    from stragglar_b200 import ops
    comm = ops.LocalComm(n, emulate=True)
    prog = sc.compile_program(alg, n, prephase, straggler)
    xs = _inputs(n, count, dtype)
    want = torch.stack([x.double() for x in xs]).sum(0) * scale
    if not prephase:
        _prephase(xs, alg, n - 1 if straggler is None else straggler)
    comm.run(prog, xs, path=path, blocks=blocks, tile_bytes=tile_bytes, scale=scale, delay_ms=delay_ms, timeout_s=5.0)
    comm.sync()
    comm.close()
    return xs, want


TOL = {torch.float32: dict(atol=1e-5, rtol=1e-6), torch.bfloat16: dict(atol=6e-2, rtol=2e-2),
       torch.float16: dict(atol=8e-3, rtol=4e-3)}


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("alg", ["stragglar", "stragglar_a2a", "ring", "rhd", "direct", "rsag"])
def test_algorithms_n8(alg, path):
    xs, want = _run(alg, 8, 40_003, path=path)
    for x in xs:
        torch.testing.assert_close(x.double(), want, **TOL[torch.float32])


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("n", [1, 2, 4, 6])
def test_stragglar_other_sizes(n, path):
    xs, want = _run("stragglar", n, 20_001, path=path, scale=0.5)
    for x in xs:
        torch.testing.assert_close(x.double(), want, **TOL[torch.float32])


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_precisions(dtype, path):
    xs, want = _run("stragglar", 8, 30_005, dtype=dtype, path=path)
    for x in xs:
        torch.testing.assert_close(x.double(), want, **TOL[dtype])
    # one rounding per reduction, the same on both sides of a matching: all ranks agree bit for bit
    for x in xs[1:]:
        assert torch.equal(x, xs[0])


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("alg", ["stragglar", "stragglar_a2a", "direct"])
def test_prephase_done_mode(alg, path):
    xs, want = _run(alg, 8, 25_000, path=path, prephase=False)
    for x in xs:
        torch.testing.assert_close(x.double(), want, atol=2e-5, rtol=1e-6)


@pytest.mark.parametrize("path", PATHS)
def test_late_straggler_swapped_to_last_rank(path):
    # physical rank 2 is 3 ms late and plays logical rank n-1
    delay = [0.0] * 8
    delay[2] = 3.0
    xs, want = _run("stragglar", 8, 50_000, path=path, straggler=2, delay_ms=delay)
    for x in xs:
        torch.testing.assert_close(x.double(), want, **TOL[torch.float32])


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("count", [1, 5, 17, 4099])
def test_small_and_ragged(count, path):
    xs, want = _run("stragglar", 4, count, path=path, tile_bytes=2048)
    for x in xs:
        torch.testing.assert_close(x.double(), want, **TOL[torch.float32])


@pytest.mark.parametrize("path", PATHS)
def test_back_to_back_collectives_reuse_flags(path):
    from stragglar_b200 import ops
    n, count = 4, 100_000
    comm = ops.LocalComm(n, emulate=True)
    prog = sc.compile_program("ring", n)
    xs = [torch.full((count,), float(r + 1), device="cuda:0") for r in range(n)]
    for _ in range(3):
        comm.run(prog, xs, path=path, blocks=3, tile_bytes=8192)
    comm.sync()
    for x in xs:
        torch.testing.assert_close(x, torch.full_like(x, 10.0 * n * n))
    comm.close()


@pytest.mark.parametrize("path", PATHS)
def test_larger_than_l2(path):
    # 8 ranks x 64 MiB: every tile crosses HBM
    from stragglar_b200 import ops
    n, count = 8, 16 * 1024 * 1024
    comm = ops.LocalComm(n, emulate=True)
    prog = sc.compile_program("stragglar", n)
    xs = _inputs(n, count, torch.float32)
    comm.run(prog, xs, path=path, blocks=16, timed=True)
    ms = comm.sync()
    for x in xs:
        bad, worst = ops.verify_uniform_sum(x, list(range(n)), atol=1e-5)
        assert bad == 0, (bad, worst)
    assert ms[0] > 0
    comm.close()


def test_wait_runs_out_without_hanging():
    """A rank that arrives after the deadline: every block gives up, the status
    says so, the context stays usable and the next collective works."""
    from stragglar_b200 import ops
    n, count = 4, 10_000
    comm = ops.LocalComm(n, emulate=True)
    prog = sc.compile_program("stragglar", n)
    xs = _inputs(n, count, torch.float32)
    comm.run(prog, xs, blocks=2, tile_bytes=4096, delay_ms=[0, 0, 0, 400.0], timeout_s=0.05)
    comm.sync(check=False)
    assert comm.last_status != 0 and comm.last_status < 0x1000
    assert "timeout" in sc.status_string(comm.last_status) or "aborted" in sc.status_string(comm.last_status)
    torch.cuda.synchronize()
    # after the failure is cleared the communicator works again (fresh inputs, later epoch)
    ys = _inputs(n, count, torch.float32)
    want = torch.stack([y.double() for y in ys]).sum(0)
    comm.run(prog, ys, blocks=2, tile_bytes=4096)
    comm.sync()
    for y in ys:
        torch.testing.assert_close(y.double(), want, **TOL[torch.float32])
    comm.close()


def test_helper_kernels():
    from stragglar_b200 import ops
    x = torch.empty(1000, device="cuda:0")
    ops.fill_uniform(x, seed=7)
    torch.cuda.synchronize()
    assert -1.0 <= x.min().item() and x.max().item() < 1.0 and abs(x.mean().item()) < 0.1
    assert x[5].item() == pytest.approx(ops.host_uniform(7, 5))
    y = torch.empty(1000, device="cuda:0", dtype=torch.bfloat16)
    ops.scale_cast(y, x, 0.5)
    torch.cuda.synchronize()
    torch.testing.assert_close(y, (x * 0.5).bfloat16())
    ops.scale_cast(x, x, 2.0)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record(); ops.delay(5.0); t1.record(); torch.cuda.synchronize()
    assert 4.9 <= t0.elapsed_time(t1) < 7.0


@pytest.mark.parametrize("path", PATHS)
def test_round_trace(path):
    """Per-round statistics: every round of a rank's table shows up, starts before it ends, rounds end in order
    on the straggler (its matchings are serial), and a run without tracing leaves the record untouched."""
    from stragglar_b200 import ops
    n, count = 4, 60_000
    comm = ops.LocalComm(n, emulate=True)
    prog = sc.compile_program("stragglar", n)
    xs = _inputs(n, count, torch.float32)
    want = torch.stack([x.double() for x in xs]).sum(0)
    comm.run(prog, xs, path=path, blocks=2, tile_bytes=4096, timeout_s=5.0, trace_rounds=True)
    comm.sync()
    for x in xs:
        torch.testing.assert_close(x.double(), want, **TOL[torch.float32])
    tr = comm.round_trace()
    assert len(tr) == n
    for r in range(n):
        want_rounds = set()
        for t in prog.phases:
            want_rounds |= {int(k) for k in t.ranks[r].ops["round"]}
        assert set(tr[r]) == want_rounds, (r, sorted(tr[r]), sorted(want_rounds))
        for k, (start, end, wait) in tr[r].items():
            assert 0 < start <= end and wait < 5_000_000_000
    ends = [tr[n - 1][k][1] for k in sorted(tr[n - 1])]
    assert ends == sorted(ends)
    before = comm.round_trace()
    comm.run(prog, xs, path=path, blocks=2, tile_bytes=4096, timeout_s=5.0)
    comm.sync()
    assert comm.round_trace() == before
    comm.close()


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("alg,n,slack", [("stragglar", 8, 0), ("stragglar", 8, 3), ("stragglar", 6, 0), ("ring", 4, 0),
                                         ("stragglar_a2a", 4, 0)])
def test_round_gating(alg, n, slack, path, monkeypatch):
    """Rounds one after the other (STRAGGLAR_GATE): same sums, twice in a row on the same control words, and with
    the full barrier (slack 0) the traced rounds do not overlap on any rank."""
    monkeypatch.setenv("STRAGGLAR_GATE_SLACK", str(slack))
    from stragglar_b200 import ops
    monkeypatch.setenv("STRAGGLAR_GATE", "all")
    monkeypatch.setenv("STRAGGLAR_GATE_MIN_BYTES", "0")      # gate the small test buffers too
    prog = sc.compile_program(alg, n)
    assert prog.main.gate_rounds
    comm = ops.LocalComm(n, emulate=True)
    for rep in range(2):
        xs = _inputs(n, 50_003, torch.float32)
        want = torch.stack([x.double() for x in xs]).sum(0)
        comm.run(prog, xs, path=path, blocks=2, tile_bytes=4096, timeout_s=5.0, trace_rounds=True)
        comm.sync()
        for x in xs:
            torch.testing.assert_close(x.double(), want, **TOL[torch.float32])
    tr = comm.round_trace()
    starts = {}
    ends = {}
    for r in range(n):
        for k, (s, e, _) in tr[r].items():
            starts[k] = min(starts.get(k, s), s)
            ends[k] = max(ends.get(k, e), e)
    rounds = sorted(starts)
    # GPUs' %globaltimer values agree here: all ranks are emulated on one device
    if slack == 0:
        assert all(ends[a] <= starts[b] for a, b in zip(rounds, rounds[1:])), (starts, ends)
    comm.close()


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("alg,n", [("stragglar", 8), ("ring", 4), ("rsag", 4), ("stragglar_a2a", 6), ("stragglar", 1)])
@pytest.mark.parametrize("wire,user", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                       (torch.float32, torch.bfloat16)])
def test_staged_mode_reads_and_writes_the_callers_tensors(alg, n, wire, user, path):
    """Staged mode: the kernel itself copies the caller's tensor into the buffer peers reach (converting to the wire
    dtype), runs the table and copies every finished tile back; no separate copy or cast kernels."""
    from stragglar_b200 import ops
    count = 70_001
    comm = ops.LocalComm(n, emulate=True)
    prog = sc.compile_program(alg, n)
    if len(prog.phases) != 1:
        pytest.skip("staged mode serves single-phase programs")
    users = _inputs(n, count, user)
    # what the wire carries: the inputs rounded to the wire dtype, summed in fp32
    want = torch.stack([u.to(wire).double() for u in users]).sum(0) * 0.5
    arena = [torch.full((count,), float("nan"), dtype=wire, device="cuda:0") for _ in range(n)]
    torch.cuda.synchronize()
    for rep in range(2):   # twice: the second run finds the flags of the first
        if rep:
            for u, v in zip(users, _inputs(n, count, user)):
                u.copy_(v)
            torch.cuda.synchronize()
        comm.run(prog, arena, path=path, blocks=3, tile_bytes=4096, scale=0.5, timeout_s=5.0, user_tensors=users)
        comm.sync()
        lo = torch.bfloat16 in (wire, user)
        tol = dict(atol=6e-2, rtol=2e-2) if lo else dict(atol=1e-5, rtol=1e-6)
        for u in users:
            torch.testing.assert_close(u.double(), want, **tol)
    comm.close()
