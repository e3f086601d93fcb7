"""AllReduce micro-benchmark through the c10d backend.

    torchrun --nproc-per-node=8 --master-addr 127.0.0.1 examples/example.py

The counterpart of the reference's implementation/custom_backend/example.py:
the same 1 GiB fp32 tensor (rounded up to a multiple of 7 KiB), filled with the
rank, one warm-up AllReduce that is printed, ten timed ones, the average
latency per rank.  It works for any world size and any rank as the straggler
(``STRAGGLAR_STRAGGLER``), and CPU tensors go through gloo.
"""
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import stragglar_b200.parallel as sp  # noqa: E402  (registers the "stragglar" backend)

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("MASTER_PORT", "29500")
rank = int(os.environ.get("RANK", "0"))
world_size = int(os.environ.get("WORLD_SIZE", "1"))
local_rank = int(os.environ.get("LOCAL_RANK", "0"))

size = 1024 ** 3 // 4
size = math.ceil(size * 4 / (1024 * 7)) * 1024 * 7 // 4
os.environ.setdefault("STRAGGLAR_ARENA_MB", str(size * 4 // (1 << 20) + 384))

dist.init_process_group("cpu:gloo,cuda:stragglar", rank=rank, world_size=world_size)
print(size)

x = torch.full((size,), rank, dtype=torch.float)
if torch.cuda.is_available():
    torch.cuda.set_device(local_rank)
    y = sp.empty_symmetric(size, dtype=torch.float, device=f"cuda:{local_rank}")   # reduced in place, no staging
    y.copy_(x)
    print(f"Device ID of CUDA tensor: {y.get_device()} | size: {y.size()}")
    dist.all_reduce(y)
    print(f"cuda allreduce: {y}")

    total_time = 0
    for itr in range(10):
        y.fill_(rank)
        t1 = torch.cuda.Event(enable_timing=True)
        t2 = torch.cuda.Event(enable_timing=True)
        t1.record()
        dist.all_reduce(y)
        t2.record()
        torch.cuda.synchronize()
        total_time = total_time + t1.elapsed_time(t2)
    print(f"Rank: {rank} | Avg latency: {total_time / 10}")
    status = sp.check_status(f"cuda:{local_rank}")
    assert status == 0, status
    assert float(y[0]) == sum(range(world_size)), (float(y[0]), sum(range(world_size)))
dist.destroy_process_group()
