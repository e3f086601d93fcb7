"""The c10d backend on CPU tensors: ranks are processes, arenas are POSIX
shared memory, collectives walk the same tables as on the GPU.  Covers the
Store bootstrap, Work/Future plumbing, every collective DDP needs, the
straggler swap and DistributedDataParallel itself."""
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, errq):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        os.environ.setdefault("STRAGGLAR_TIMEOUT_MS", "20000")
        import stragglar_b200.parallel  # noqa: F401
        dist.init_process_group("stragglar", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def run_ranks(world, fn, *args):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            msgs.append("a rank did not finish")
    assert not msgs and all(p.exitcode == 0 for p in procs), "\n".join(msgs)


def _seeded(rank, n, dtype=torch.float32):
    g = torch.Generator().manual_seed(rank)
    return torch.empty(n).uniform_(-1, 1, generator=g).to(dtype)


def _collectives(rank, world):
    import stragglar_b200.parallel as sp
    n = 10_007
    x = _seeded(rank, n)
    want = torch.stack([_seeded(r, n).double() for r in range(world)]).sum(0)
    y = x.clone()
    work = dist.all_reduce(y, async_op=True)
    work.wait()
    assert work.is_completed() and work.get_future().done()
    torch.testing.assert_close(y.double(), want, atol=1e-5, rtol=1e-6)
    y = x.clone()
    dist.all_reduce(y, op=dist.ReduceOp.AVG)
    torch.testing.assert_close(y.double(), want / world, atol=1e-5, rtol=1e-6)
    # the other algorithms through the same backend
    for alg in ("ring", "stragglar_a2a", "direct", "rsag"):
        sp.set_algorithm(alg, device="cpu")
        y = x.clone()
        dist.all_reduce(y)
        torch.testing.assert_close(y.double(), want, atol=1e-5, rtol=1e-6)
    sp.set_algorithm("stragglar", device="cpu")
    # straggler swap: physical rank 1 plays the last logical rank
    sp.set_straggler(1, device="cpu")
    assert sp.get_straggler(device="cpu") == 1
    y = x.clone()
    dist.all_reduce(y)
    torch.testing.assert_close(y.double(), want, atol=1e-5, rtol=1e-6)
    # broadcast / all_gather / reduce_scatter / reduce / gather / scatter / all_to_all
    b = torch.full((33,), float(rank))
    dist.broadcast(b, src=world - 1)
    assert (b == world - 1).all()
    outs = [torch.empty(5) for _ in range(world)]
    dist.all_gather(outs, torch.full((5,), float(rank)))
    assert all((outs[r] == r).all() for r in range(world))
    big = torch.empty(world * 7)
    dist.all_gather_into_tensor(big, torch.full((7,), float(rank)))
    assert torch.equal(big, torch.arange(world).repeat_interleave(7).float())
    rs = torch.empty(11)
    dist.reduce_scatter_tensor(rs, torch.arange(world * 11).float() + rank)
    torch.testing.assert_close(rs, world * (torch.arange(11).float() + 11 * rank) + sum(range(world)))
    r0 = x.clone()
    dist.reduce(r0, dst=0)
    if rank == 0:
        torch.testing.assert_close(r0.double(), want, atol=1e-5, rtol=1e-6)
    glist = [torch.empty(3) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.full((3,), float(rank)), glist, dst=0)
    if rank == 0:
        assert all((glist[r] == r).all() for r in range(world))
    sc = torch.empty(4)
    dist.scatter(sc, [torch.full((4,), float(10 + r)) for r in range(world)] if rank == 1 else None, src=1)
    assert (sc == 10 + rank).all()
    a2a = torch.empty(world * 2)
    dist.all_to_all_single(a2a, torch.arange(world * 2).float() + 100 * rank)
    want_a2a = torch.cat([torch.arange(2).float() + 2 * rank + 100 * p for p in range(world)])
    assert torch.equal(a2a, want_a2a)
    # point to point
    if rank == 0:
        dist.send(torch.arange(9).float(), dst=world - 1)
    if rank == world - 1:
        got = torch.empty(9)
        dist.recv(got, src=0)
        assert torch.equal(got, torch.arange(9).float())
    # symmetric tensors are reduced in place without staging
    s = sp.empty_symmetric(n, device="cpu")
    s.copy_(x)
    dist.all_reduce(s)
    torch.testing.assert_close(s.double(), want, atol=1e-5, rtol=1e-6)
    # half precisions
    for dt, tol in ((torch.bfloat16, 6e-2), (torch.float16, 8e-3)):
        h = _seeded(rank, 2050, dt)
        wanth = torch.stack([_seeded(r, 2050, dt).double() for r in range(world)]).sum(0)
        dist.all_reduce(h)
        torch.testing.assert_close(h.double(), wanth, atol=tol, rtol=2e-2)
    mx = torch.full((4,), float(rank))
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)          # not a table operation: gathered and reduced locally
    assert (mx == world - 1).all()
    # coalesced forms, reached through the functional collectives (what FSDP-style code uses)
    import torch.distributed._functional_collectives as fc
    ins = [torch.arange(world * 3).float() + rank, torch.arange(world * 5).float() * 2 + rank]
    outs = [fc.wait_tensor(t) for t in fc.reduce_scatter_tensor_coalesced(ins, "sum", [0, 0], dist.group.WORLD)]
    torch.testing.assert_close(outs[0], world * (torch.arange(3).float() + 3 * rank) + sum(range(world)))
    torch.testing.assert_close(outs[1], world * 2 * (torch.arange(5).float() + 5 * rank) + sum(range(world)))
    gouts = [fc.wait_tensor(t) for t in fc.all_gather_into_tensor_coalesced(
        [torch.full((2,), float(rank)), torch.full((4,), float(rank + 10))], dist.group.WORLD)]
    assert torch.equal(gouts[0], torch.arange(world).repeat_interleave(2).float())
    assert torch.equal(gouts[1], (torch.arange(world) + 10).repeat_interleave(4).float())
    # the canary bytes on both sides of the heap + staging region are intact after all of the above
    assert sp.check_guards("cpu") and sp.check_status("cpu") == 0


@pytest.mark.parametrize("world", [2, 4])
def test_collectives(world):
    run_ranks(world, _collectives)


def _ddp(rank, world, hook="fused"):
    import stragglar_b200.parallel as sp
    from torch.nn.parallel import DistributedDataParallel as DDP
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    ref.load_state_dict(model.state_dict())
    ddp = DDP(model, bucket_cap_mb=0.001)
    ddp.register_comm_hook(None, sp.fused_avg_hook if hook == "fused" else sp.SymmetricBucketHook())
    xs = [torch.randn(8, 16, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
    ys = [torch.randn(8, 4, generator=torch.Generator().manual_seed(200 + r)) for r in range(world)]
    for _ in range(3 if hook != "fused" else 1):   # several steps: DDP rebuilds its buckets after the first
        ddp.zero_grad()
        loss = torch.nn.functional.mse_loss(ddp(xs[rank]), ys[rank])
        loss.backward()
    # reference: average of the per-rank gradients computed locally
    total = None
    for r in range(world):
        ref.zero_grad()
        torch.nn.functional.mse_loss(ref(xs[r]), ys[r]).backward()
        g = [p.grad.clone() for p in ref.parameters()]
        total = g if total is None else [a + b for a, b in zip(total, g)]
    for p, g in zip(model.parameters(), total):
        torch.testing.assert_close(p.grad, g / world, atol=1e-6, rtol=1e-5)


def test_distributed_data_parallel_on_the_backend():
    run_ranks(2, _ddp)


def test_ddp_with_buckets_reduced_in_the_symmetric_heap():
    run_ranks(2, _ddp, "symmetric")


def _late_rank_times_out(rank, world):
    # rank 1 never joins this collective: rank 0's wait runs out and raises instead of hanging
    import time
    dist.barrier()   # the arenas exist from here on
    if rank == 0:
        t0 = time.time()
        # the failure belongs to the Work: issuing the collective returns, wait() raises, is_success() is false
        work = dist.all_reduce(torch.ones(64), async_op=True)
        with pytest.raises(RuntimeError, match="collective failed|timed out"):
            work.wait()
        assert not work.is_success()
        assert time.time() - t0 < 5.0
    else:
        time.sleep(0.35)  # joins the final barrier while rank 0 is still giving up on the all-reduce
    # afterwards both ranks meet again in the worker's final barrier (its own control channel)


def test_missing_rank_raises_after_the_timeout():
    os.environ["STRAGGLAR_TIMEOUT_MS"] = "700"
    try:
        run_ranks(2, _late_rank_times_out)
    finally:
        del os.environ["STRAGGLAR_TIMEOUT_MS"]


def _grad_sync(rank, world):
    from stragglar_b200.parallel.grad_sync import FlatGradSync, allreduce_gradients_per_param
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3))
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(10 + rank))
    model(x).sum().backward()
    mine = [p.grad.clone() for p in model.parameters()]
    gathered = []
    for g in mine:
        parts = [torch.empty_like(g) for _ in range(world)]
        dist.all_gather(parts, g)
        gathered.append(torch.stack(parts).mean(0))
    sync = FlatGradSync(model)           # flat buffer in the symmetric heap, 1/world fused
    sync()
    for p, want in zip(model.parameters(), gathered):
        torch.testing.assert_close(p.grad, want, atol=1e-6, rtol=1e-5)
    for p, g in zip(model.parameters(), mine):
        p.grad.copy_(g)
    nbytes = allreduce_gradients_per_param(model)
    assert nbytes == sum(g.numel() * 4 for g in mine)
    for p, want in zip(model.parameters(), gathered):
        torch.testing.assert_close(p.grad, want, atol=1e-6, rtol=1e-5)


def test_manual_gradient_sync_flat_and_per_parameter():
    run_ranks(2, _grad_sync)


def _bigger_than_staging(rank, world):
    # 1 MiB of staging (arena 2 MiB): 3 MiB tensors go through the arena in pieces
    n = 786_432 + 5
    x = _seeded(rank, n)
    want = torch.stack([_seeded(r, n).double() for r in range(world)]).sum(0)
    y = x.clone()
    dist.all_reduce(y)
    torch.testing.assert_close(y.double(), want, atol=1e-5, rtol=1e-6)
    b = x.clone() if rank == 1 else torch.zeros(n)
    dist.broadcast(b, src=1)
    torch.testing.assert_close(b, _seeded(1, n))
    out = torch.empty(world * n)
    dist.all_gather_into_tensor(out, x)
    for r in range(world):
        torch.testing.assert_close(out[r * n:(r + 1) * n], _seeded(r, n))
    rs = torch.empty(n)
    dist.reduce_scatter_tensor(rs, torch.cat([_seeded(10 * q + rank, n) for q in range(world)]))
    want_rs = torch.stack([_seeded(10 * rank + p, n).double() for p in range(world)]).sum(0)
    torch.testing.assert_close(rs.double(), want_rs, atol=1e-5, rtol=1e-6)
    r0 = x.clone()
    dist.reduce(r0, dst=1)
    if rank == 1:
        torch.testing.assert_close(r0.double(), want, atol=1e-5, rtol=1e-6)
    if rank == 0:
        dist.send(x, dst=1)
    elif rank == 1:
        got = torch.empty(n)
        dist.recv(got, src=0)
        torch.testing.assert_close(got, _seeded(0, n))


def test_tensors_larger_than_the_staging_area():
    os.environ["STRAGGLAR_CPU_ARENA_MB"] = "2"
    try:
        run_ranks(2, _bigger_than_staging)
    finally:
        del os.environ["STRAGGLAR_CPU_ARENA_MB"]


def _subgroups(rank, world):
    # a group of three ranks has no StragglAR schedule: it is served by the ring
    g3 = dist.new_group([0, 1, 2], backend="stragglar")
    g2 = dist.new_group([1, 3], backend="stragglar")
    x = torch.full((1001,), float(rank + 1))
    if rank in (0, 1, 2):
        dist.all_reduce(x, group=g3)
        assert (x == 6).all()
    y = torch.full((77,), float(rank + 1))
    if rank in (1, 3):
        dist.all_reduce(y, group=g2)
        assert (y == 6).all()
        out = [torch.empty(3) for _ in range(2)]
        dist.all_gather(out, torch.full((3,), float(rank)), group=g2)
        assert out[0][0] == 1 and out[1][0] == 3
    z = torch.ones(10)
    dist.all_reduce(z)
    assert (z == world).all()


def test_subgroups_and_odd_sizes():
    run_ranks(4, _subgroups)


def _alone(port, errq):
    """Rank 0 of a two-rank group whose other rank never starts."""
    try:
        import glob
        from datetime import timedelta
        sys.path.insert(0, ROOT)
        import stragglar_b200.parallel  # noqa: F401
        store = dist.TCPStore("127.0.0.1", port, 2, is_master=True, timeout=timedelta(seconds=2), wait_for_workers=False)
        try:
            dist.init_process_group("stragglar", store=store, rank=0, world_size=2, timeout=timedelta(seconds=2))
            dist.all_reduce(torch.ones(8))       # the arenas are opened by the first collective at the latest
            errq.put("a group with a missing rank came up")
        except Exception as e:                   # the store gives up waiting for the peer's arena
            if "imeout" not in str(e) and "wait" not in str(e).lower():
                errq.put(f"unexpected error: {e!r}")
        left = glob.glob(f"/dev/shm/sar_{os.getpid()}_*")
        if left:
            errq.put(f"shared memory left behind: {left}")
    except Exception:
        errq.put(traceback.format_exc())


def test_rank_that_never_joins_fails_the_bootstrap_and_leaves_no_shared_memory():
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    p = ctx.Process(target=_alone, args=(_free_port(), errq))
    p.start()
    p.join(60)
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    if p.is_alive():
        p.kill()
        msgs.append("the lone rank hung")
    assert not msgs, "\n".join(msgs)


def _auto(rank, world):
    import stragglar_b200.parallel as sp
    dev = "cpu"
    sp.set_algorithm("auto", dev)
    assert sp.get_algorithm(dev) == "auto" and sp.get_straggler(dev) == -1
    # nobody declared late: one-shot reduce-scatter + all-gather for small messages, the ring for large ones
    assert sp.algorithm_for(1 << 20, dev) == "rsag" and sp.algorithm_for(1 << 30, dev) == "ring"
    x = _seeded(rank, 5000)
    want = sum(_seeded(r, 5000) for r in range(world))
    dist.all_reduce(x)
    torch.testing.assert_close(x, want, atol=1e-5, rtol=1e-6)
    # a declared straggler switches to the straggler-aware variant, whatever the size
    sp.set_straggler(1, dev)
    assert sp.algorithm_for(1 << 20, dev) == "stragglar_a2a" == sp.algorithm_for(1 << 30, dev)
    y = _seeded(rank, 5000)
    dist.all_reduce(y)
    torch.testing.assert_close(y, want, atol=1e-5, rtol=1e-6)
    # the monitor withdraws the declaration when the last rank to arrive keeps changing
    mon = sp.StragglerMonitor(window=4, threshold=0.75, device=dev)
    fake = iter([[5, 1, 5, 5], [1, 5, 5, 5], [5, 5, 1, 5], [5, 5, 5, 1]])
    real = sp.last_collective_ms
    try:
        for times in fake:
            sp.last_collective_ms = lambda *a, _t=times, **k: float(_t[rank])
            mon.step()
    finally:
        sp.last_collective_ms = real
    assert sp.get_straggler(dev) == -1 and mon.changes == 1
    assert sp.algorithm_for(1 << 20, dev) == "rsag"
    # a fixed algorithm is returned as configured; an unknown name is refused and changes nothing
    sp.set_algorithm("ring", dev)
    assert sp.algorithm_for(123, dev) == "ring"
    with pytest.raises(RuntimeError, match="unknown algorithm"):
        sp.set_algorithm("tree", dev)
    assert sp.get_algorithm(dev) == "ring"


def test_auto_algorithm_selection():
    run_ranks(4, _auto)


def _other_dtypes_and_ops(rank, world):
    # integer / fp64 / bool tensors and MIN, MAX, PRODUCT, bitwise ops take the gather-and-reduce path
    x = torch.arange(10, dtype=torch.int64) * (rank + 1)
    dist.all_reduce(x)
    assert torch.equal(x, torch.arange(10, dtype=torch.int64) * sum(range(1, world + 1)))
    y = torch.full((7,), float(rank), dtype=torch.float64)
    dist.all_reduce(y, op=dist.ReduceOp.MAX)
    assert torch.equal(y, torch.full((7,), float(world - 1), dtype=torch.float64))
    z = _seeded(rank, 300)
    dist.all_reduce(z, op=dist.ReduceOp.MIN)
    assert torch.equal(z, torch.stack([_seeded(r, 300) for r in range(world)]).amin(0))
    p = torch.full((5,), 2.0)
    dist.all_reduce(p, op=dist.ReduceOp.PRODUCT)
    assert torch.equal(p, torch.full((5,), 2.0 ** world))
    bits = torch.tensor([1 << rank, 0xff, rank], dtype=torch.int32)
    b_or, b_and, b_xor = bits.clone(), bits.clone(), bits.clone()
    dist.all_reduce(b_or, op=dist.ReduceOp.BOR)
    dist.all_reduce(b_and, op=dist.ReduceOp.BAND)
    dist.all_reduce(b_xor, op=dist.ReduceOp.BXOR)
    ranks = list(range(world))
    import functools
    import operator
    assert b_or.tolist() == [(1 << world) - 1, 0xff, functools.reduce(operator.or_, ranks)]
    assert b_and.tolist() == [0, 0xff, functools.reduce(operator.and_, ranks)]
    assert b_xor.tolist() == [(1 << world) - 1, 0xff if world % 2 else 0, functools.reduce(operator.xor, ranks)]
    flag = torch.tensor([rank == 1])
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    assert flag.item() is True
    m = torch.full((4,), rank + 1, dtype=torch.int32)
    dist.all_reduce(m, op=dist.ReduceOp.SUM)           # several in a row reuse the staging area safely
    dist.all_reduce(m, op=dist.ReduceOp.MAX)
    assert m.tolist() == [sum(range(1, world + 1))] * 4
    with pytest.raises(RuntimeError, match="floating-point"):
        dist.all_reduce(torch.ones(3, dtype=torch.int32), op=dist.ReduceOp.AVG)
    # reduce to a root: only the root's tensor changes
    t = torch.full((6,), rank + 1, dtype=torch.int64)
    dist.reduce(t, dst=1, op=dist.ReduceOp.MAX)
    assert t.tolist() == [world if rank == 1 else rank + 1] * 6


def test_integer_tensors_and_other_reduce_ops():
    run_ranks(4, _other_dtypes_and_ops)


def _ddp_unused(rank, world):
    # find_unused_parameters=True makes DDP all-reduce an int32 bitmap next to the gradients
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b, self.c = torch.nn.Linear(6, 6), torch.nn.Linear(6, 3), torch.nn.Linear(6, 3)
        def forward(self, x, use_c):
            h = torch.tanh(self.a(x))
            return self.c(h) if use_c else self.b(h)

    net = Net()
    ddp = torch.nn.parallel.DistributedDataParallel(net, find_unused_parameters=True)
    x = torch.randn(5, 6, generator=torch.Generator().manual_seed(20 + rank))
    ddp(x, False).sum().backward()
    ref = Net()
    ref.load_state_dict(net.state_dict())
    grads = []
    for r in range(world):
        ref.zero_grad()
        ref(torch.randn(5, 6, generator=torch.Generator().manual_seed(20 + r)), False).sum().backward()
        grads.append([p.grad.clone() if p.grad is not None else None for p in ref.parameters()])
    for i, p in enumerate(net.parameters()):
        want = [g[i] for g in grads]
        if want[0] is None:
            assert p.grad is None or torch.count_nonzero(p.grad) == 0
        else:
            torch.testing.assert_close(p.grad, torch.stack(want).mean(0), atol=1e-6, rtol=1e-5)


def test_ddp_with_unused_parameters():
    run_ranks(2, _ddp_unused)


def _mismatched_arguments(rank, world):
    # STRAGGLAR_CHECK_ARGS=1: a rank that passes another kind of tensor (or another size) than its peers is told so
    import stragglar_b200.parallel as sp
    sym = sp.empty_symmetric(256, device="cpu")
    sym.fill_(1.0)
    x = sym if rank == 0 else torch.ones(256)          # rank 0: symmetric heap, rank 1: an ordinary tensor
    with pytest.raises(RuntimeError, match="different arguments"):
        dist.all_reduce(x)
    y = torch.ones(128 if rank == 0 else 64)
    with pytest.raises(RuntimeError, match="different arguments"):
        dist.all_reduce(y)
    z = torch.full((512,), float(rank + 1))            # the same everywhere: goes through
    dist.all_reduce(z)
    assert float(z[0]) == 3.0


def test_argument_check_names_mismatched_ranks():
    os.environ["STRAGGLAR_CHECK_ARGS"] = "1"
    try:
        run_ranks(2, _mismatched_arguments)
    finally:
        del os.environ["STRAGGLAR_CHECK_ARGS"]
