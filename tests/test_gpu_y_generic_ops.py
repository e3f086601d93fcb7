"""Integer tensors and the reduce operations beyond SUM / AVG on CUDA tensors: the backend gathers the
contributions through its arenas and reduces them with ATen on its communication stream."""
import pytest
import torch
import torch.distributed as dist

from test_backend_cpu import run_ranks

pytestmark = pytest.mark.gpu


def _generic(rank, world):
    import stragglar_b200.parallel as sp
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    x = torch.arange(100_000, dtype=torch.int64, device=dev) * (rank + 1)
    dist.all_reduce(x)
    assert torch.equal(x, torch.arange(100_000, dtype=torch.int64, device=dev) * sum(range(1, world + 1)))
    y = torch.full((33,), float(rank), dtype=torch.float64, device=dev)
    dist.all_reduce(y, op=dist.ReduceOp.MAX)
    assert (y == world - 1).all()
    g = torch.Generator().manual_seed(rank)
    z = torch.empty(5000).uniform_(-1, 1, generator=g).to(dev)
    want = torch.stack([torch.empty(5000).uniform_(-1, 1, generator=torch.Generator().manual_seed(r)) for r in range(world)])
    dist.all_reduce(z, op=dist.ReduceOp.MIN)
    assert torch.equal(z.cpu(), want.amin(0))
    bits = torch.tensor([1 << rank, 0xff], dtype=torch.int32, device=dev)
    dist.all_reduce(bits, op=dist.ReduceOp.BOR)
    assert bits.tolist() == [(1 << world) - 1, 0xff]
    # interleaved with a table all-reduce on the same stream
    f = torch.full((4096,), float(rank + 1), device=dev)
    dist.all_reduce(f)
    c = torch.tensor([rank + 1], dtype=torch.int32, device=dev)
    dist.all_reduce(c, op=dist.ReduceOp.PRODUCT)
    assert (f == sum(range(1, world + 1))).all()
    import math
    assert c.item() == math.factorial(world)
    t = torch.full((6,), rank + 1, dtype=torch.int64, device=dev)
    dist.reduce(t, dst=world - 1, op=dist.ReduceOp.MAX)
    assert t.tolist() == [world if rank == world - 1 else rank + 1] * 6
    torch.cuda.synchronize()
    assert sp.check_status(dev) == 0


def test_generic_ops_world1_on_one_gpu():
    run_ranks(1, _generic)


@pytest.mark.multigpu
def test_generic_ops_on_all_gpus():
    world = min(torch.cuda.device_count(), 8)
    run_ranks(world - world % 2, _generic)
