"""The c10d backend and the single-process communicator on real GPUs: one
rank per device, peer memory over NVLink.  World size 1 runs on any GPU box;
the multi-rank tests need two or more devices."""
import os

import pytest
import torch
import torch.distributed as dist

from test_backend_cpu import run_ranks

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _seeded(rank, n, dtype=torch.float32, device="cpu"):
    g = torch.Generator().manual_seed(rank)
    return torch.empty(n).uniform_(-1, 1, generator=g).to(dtype).to(device)


def _cuda_collectives(rank, world):
    import stragglar_b200.parallel as sp
    from stragglar_b200 import ops
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    n = 1_000_003
    x = _seeded(rank, n, device=dev)
    want = torch.stack([_seeded(r, n).double() for r in range(world)]).sum(0).to(dev)
    for path_alg in ("stragglar", "ring", "stragglar_a2a", "direct", "rsag"):
        sp.set_algorithm(path_alg)
        y = x.clone()
        work = dist.all_reduce(y, async_op=True)
        work.wait()
        torch.testing.assert_close(y.double(), want, atol=2e-5, rtol=1e-6)
    sp.set_algorithm("stragglar")
    # fused average, a late straggler that is not the last rank, a symmetric tensor (in place)
    late = 0
    sp.set_straggler(late)
    s = sp.empty_symmetric(n, device=dev)
    s.copy_(x)
    if rank == late:
        ops.delay(3.0)
    dist.all_reduce(s, op=dist.ReduceOp.AVG)
    torch.testing.assert_close(s.double(), want / world, atol=2e-5, rtol=1e-6)
    sp.set_straggler(-1)
    # an ordinary tensor (not in the symmetric heap) costs exactly one kernel: copy-in, reduction and copy-out are fused
    y = x.clone()
    l0 = sp.launches(dev)
    dist.all_reduce(y)
    assert sp.launches(dev) - l0 == 1
    torch.testing.assert_close(y.double(), want, atol=2e-5, rtol=1e-6)
    # bf16 on the wire, fp32 at the caller: the casts and the average are in the same single kernel
    z = x.clone()
    l0 = sp.launches(dev)
    sp.all_reduce_ex(z, average=True, comm_dtype=torch.bfloat16).wait()
    assert sp.launches(dev) - l0 == 1
    torch.testing.assert_close(z.double(), want / world, atol=4e-2, rtol=2e-2)
    h = _seeded(rank, 4099, torch.bfloat16, dev)
    wh = torch.stack([_seeded(r, 4099, torch.bfloat16).double() for r in range(world)]).sum(0).to(dev)
    dist.all_reduce(h)
    torch.testing.assert_close(h.double(), wh, atol=6e-2, rtol=2e-2)
    # the data-movement collectives
    b = torch.full((1025,), float(rank), device=dev)
    dist.broadcast(b, src=world - 1)
    assert (b == world - 1).all()
    outs = [torch.empty(7, device=dev) for _ in range(world)]
    dist.all_gather(outs, torch.full((7,), float(rank), device=dev))
    assert all((outs[r] == r).all() for r in range(world))
    rs = torch.empty(11, device=dev)
    dist.reduce_scatter_tensor(rs, torch.arange(world * 11, device=dev).float() + rank)
    torch.testing.assert_close(rs, world * (torch.arange(11, device=dev).float() + 11 * rank) + sum(range(world)))
    a2a = torch.empty(world * 2, device=dev)
    dist.all_to_all_single(a2a, torch.arange(world * 2, device=dev).float() + 100 * rank)
    assert torch.equal(a2a.cpu(), torch.cat([torch.arange(2).float() + 2 * rank + 100 * p for p in range(world)]))
    if world > 1:
        if rank == 0:
            dist.send(torch.arange(9, device=dev).float(), dst=world - 1)
        if rank == world - 1:
            got = torch.empty(9, device=dev)
            dist.recv(got, src=0)
            assert torch.equal(got.cpu(), torch.arange(9).float())
    torch.cuda.synchronize()
    assert sp.check_status(dev) == 0
    assert sp.launches(dev) > 0
    assert sp.check_guards(dev)      # nothing wrote outside the heap and the staging area


def test_backend_world1_on_one_gpu():
    run_ranks(1, _cuda_collectives)


@pytest.mark.multigpu
def test_backend_on_all_gpus():
    world = min(torch.cuda.device_count(), 8)
    if world % 2:
        world -= 1
    run_ranks(world, _cuda_collectives)


def _ddp_cuda(rank, world, hook="fused"):
    import stragglar_b200.parallel as sp
    from torch.nn.parallel import DistributedDataParallel as DDP
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 8)).to(dev)
    ref = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 8)).to(dev)
    ref.load_state_dict(model.state_dict())
    ddp = DDP(model, device_ids=[rank], bucket_cap_mb=0.01)
    hooks = {"fused": sp.fused_avg_hook, "bf16": sp.bf16_fused_avg_hook}
    ddp.register_comm_hook(None, hooks.get(hook) or sp.SymmetricBucketHook())
    xs = [torch.randn(16, 64, generator=torch.Generator().manual_seed(100 + r)).to(dev) for r in range(world)]
    ys = [torch.randn(16, 8, generator=torch.Generator().manual_seed(200 + r)).to(dev) for r in range(world)]
    for _ in range(2):
        ddp.zero_grad()
        torch.nn.functional.mse_loss(ddp(xs[rank]), ys[rank]).backward()
    total = None
    for r in range(world):
        ref.zero_grad()
        torch.nn.functional.mse_loss(ref(xs[r]), ys[r]).backward()
        g = [p.grad.clone() for p in ref.parameters()]
        total = g if total is None else [a + b for a, b in zip(total, g)]
    tol = dict(atol=1e-5, rtol=1e-4) if hook != "bf16" else dict(atol=2e-2, rtol=2e-2)
    for p, g in zip(model.parameters(), total):
        torch.testing.assert_close(p.grad, g / world, **tol)
    assert sp.check_status(dev) == 0


@pytest.mark.multigpu
@pytest.mark.parametrize("hook", ["fused", "symmetric", "bf16"])
def test_ddp_with_fused_average_hook(hook):
    run_ranks(2, _ddp_cuda, hook)


@pytest.mark.multigpu
@pytest.mark.parametrize("path", ["simt", "tma"])
def test_single_process_communicator_over_nvlink(path):
    from stragglar_b200 import compiler as sc, ops
    n = min(torch.cuda.device_count(), 8)
    n -= n % 2
    comm = ops.LocalComm(n)
    count = 4 * 1024 * 1024 + 3
    for alg, delay in (("stragglar", None), ("ring", None), ("stragglar", [0.0] * (n - 1) + [2.0])):
        prog = sc.compile_program(alg, n)
        xs = [torch.empty(count, device=f"cuda:{r}") for r in range(n)]
        for r, x in enumerate(xs):
            with torch.cuda.device(r):
                ops.fill_uniform(x, r)
                torch.cuda.synchronize()
        comm.run(prog, xs, path=path, delay_ms=delay, timed=True)
        ms = comm.sync()
        for x in xs:
            bad, worst = ops.verify_uniform_sum(x, list(range(n)), atol=2e-5)
            assert bad == 0, (alg, bad, worst)
        if delay:
            assert max(ms) >= 2.0
    comm.close()


def _monitor(rank, world):
    import stragglar_b200.parallel as sp
    from stragglar_b200 import ops
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    x = sp.empty_symmetric(1 << 20, device=dev)
    x.fill_(1.0)
    mon = sp.StragglerMonitor(window=5, threshold=0.8, device=dev)
    late = 0   # not the default straggler (the last rank)
    for _ in range(6):
        dist.barrier()
        if rank == late:
            ops.delay(4.0)
        dist.all_reduce(x, op=dist.ReduceOp.AVG)
        mon.step()
    assert sp.get_straggler(dev) == late and mon.changes == 1
    # the re-labelled schedule still reduces correctly
    y = torch.full((4099,), float(rank + 1), device=dev)
    dist.all_reduce(y)
    assert float(y[0]) == sum(range(1, world + 1))
    assert sp.check_status(dev) == 0


@pytest.mark.multigpu
def test_straggler_monitor_relabels_the_schedule():
    run_ranks(min(torch.cuda.device_count(), 4) // 2 * 2, _monitor)


def _late_rank_cuda(rank, world):
    """Rank 1 comes 1.5 s late to one collective while every device-side wait is limited to 400 ms: on both ranks
    the Work raises, nothing hangs, and the next collective is correct.  Nobody leaves; the failure is made on the
    host (a sleep), never on the device."""
    import datetime
    import time
    import stragglar_b200.parallel as sp
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    x = torch.full((1 << 16,), float(rank + 1), device=dev)
    dist.all_reduce(x)                       # arenas exist, the ranks are aligned
    torch.cuda.synchronize()
    assert float(x[0]) == 3.0
    t0 = time.time()                         # the ranks are within milliseconds of one another here
    if rank == 1:
        time.sleep(1.5)
    y = torch.full((1 << 16,), float(rank + 1), device=dev)
    work = dist.all_reduce(y, async_op=True)
    with pytest.raises(RuntimeError, match="collective failed"):
        work.wait(datetime.timedelta(seconds=10))
    assert work.is_completed() and not work.is_success()
    time.sleep(max(0.0, t0 + 2.6 - time.time()))   # both ranks have given up (by 1.9 s) before anybody goes on
    z = torch.full((1 << 16,), float(rank + 1), device=dev)
    work = dist.all_reduce(z, async_op=True)
    work.wait(datetime.timedelta(seconds=10))
    assert work.is_success() and float(z[0]) == 3.0 and float(z[-1]) == 3.0
    assert sp.check_status(dev) == 0


@pytest.mark.multigpu
def test_late_rank_raises_through_the_work_object():
    os.environ["STRAGGLAR_TIMEOUT_MS"] = "400"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        run_ranks(2, _late_rank_cuda)
    finally:
        del os.environ["STRAGGLAR_TIMEOUT_MS"]


def _host_streamed(rank, world):
    """sp.HostStreamedAllReduce: pieces of a pinned host tensor are reduced as they land on the device."""
    import stragglar_b200.parallel as sp
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    n = 3_000_017
    host = _seeded(rank, n).pin_memory()
    want = torch.stack([_seeded(r, n).double() for r in range(world)]).sum(0) / world
    stream = sp.HostStreamedAllReduce(n, dtype=torch.float32, device=dev, pieces=5)
    for _ in range(2):
        out = stream(host, op=dist.ReduceOp.AVG)
        torch.cuda.synchronize()
        torch.testing.assert_close(out.double().cpu(), want, atol=2e-5, rtol=1e-6)
    assert sp.check_status(dev) == 0


@pytest.mark.multigpu
def test_host_streamed_allreduce():
    run_ranks(2, _host_streamed)
