"""Symmetric buffers of the single-process communicator and their NVLink multicast views.

The multicast tests need two or more devices that offer NVLink multicast objects and skip elsewhere.
"""
import os

import pytest
import torch

from stragglar_b200 import compiler as sc

pytestmark = pytest.mark.gpu


def _fill(xs):
    from stragglar_b200 import ops
    for r, x in enumerate(xs):
        with torch.cuda.device(x.device):
            ops.fill_uniform(x, seed=100 + r)
    for x in xs:
        torch.cuda.synchronize(x.device)


def test_plain_symmetric_buffers_emulated():
    from stragglar_b200 import ops
    comm = ops.LocalComm(4, emulate=True)
    xs = comm.alloc(50_001, torch.float32, multicast=False)
    assert len(xs) == 4 and all(x.numel() == 50_001 and x.device.index == 0 for x in xs)
    assert comm.multicast_groups(xs[0]) == 0 and not comm.multicast_supported()
    _fill(xs)
    want = torch.stack([x.double() for x in xs]).sum(0)
    comm.run(sc.compile_program("rsag", 4), xs, path="simt", blocks=2, tile_bytes=4096, timeout_s=5.0)
    comm.sync()
    for x in xs:
        torch.testing.assert_close(x.double(), want, atol=1e-5, rtol=1e-6)
    # "try" falls back to plain memory when the ranks share a device; "require" refuses
    ys = comm.alloc(1024, torch.bfloat16, multicast="try")
    assert ys[0].dtype == torch.bfloat16 and comm.multicast_groups(ys[0]) == 0
    with pytest.raises(RuntimeError, match="one device per rank"):
        comm.alloc(1024, multicast=True)
    with pytest.raises(ValueError):
        comm.free([torch.empty(4, device="cuda:0")])
    comm.free(ys)
    comm.free(xs)
    comm.close()


def test_symmetric_buffers_single_rank():
    from stragglar_b200 import ops
    comm = ops.LocalComm(1)
    (x,) = comm.alloc(300_000, torch.float32, multicast=False)
    _fill([x])
    want = x.double() * 0.5
    comm.run(sc.compile_program("stragglar", 1), [x], path="tma", scale=0.5, timeout_s=5.0)
    comm.sync()
    torch.testing.assert_close(x.double(), want, atol=1e-6, rtol=1e-6)
    comm.close()   # releases the allocation too


@pytest.mark.multigpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("alg", ["rsag", "stragglar_a2a", "stragglar"])
def test_multicast_allreduce_multi_gpu(alg, dtype):
    from stragglar_b200 import ops
    n = min(torch.cuda.device_count(), 8)
    n -= n % 2
    if n < 2:
        pytest.skip("needs two or more GPUs")
    comm = ops.LocalComm(n)
    if not comm.multicast_supported():
        pytest.skip("the devices do not offer multicast")
    xs = comm.alloc((8 << 20) + 12, dtype, multicast=True, sub_members=(1 << (n - 1)) - 1)
    assert comm.multicast_groups(xs[0]) & 1
    _fill(xs)
    want = torch.stack([x.double().cpu() for x in xs]).sum(0) / n
    comm.run(sc.compile_program(alg, n), xs, path="simt", scale=1.0 / n, timeout_s=10.0)
    comm.sync()
    tol = dict(atol=1e-5, rtol=1e-6) if dtype == torch.float32 else dict(atol=6e-2, rtol=2e-2)
    for x in xs:
        torch.testing.assert_close(x.double().cpu(), want, **tol)
    comm.close()
