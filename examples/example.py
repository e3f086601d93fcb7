"""AllReduce micro-benchmark through the c10d backend.

    torchrun --nproc-per-node=8 --master-addr 127.0.0.1 examples/example.py [--bytes N] [--iters K] [--alg A]

What the reference's implementation/custom_backend/example.py measures, on this library: every rank holds a
1 GiB fp32 tensor (rounded up to a multiple of 7 KiB, as there) filled with its rank, one AllReduce is printed,
``--iters`` more are timed with CUDA events and the mean latency is printed per rank in the reference's wording
("Rank: r | Avg latency: ms").  Differences: any world size with a schedule works, any rank can be named the
straggler (``--straggler`` / ``STRAGGLAR_STRAGGLER``), the tensor lives in the backend's symmetric heap so the
collective runs in place, the result is checked, and CPU tensors are served by gloo.
"""
import argparse
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import stragglar_b200.parallel as sp  # noqa: E402  (registers the "stragglar" backend)


def padded_elements(nbytes: int, unit: int = 7 * 1024) -> int:
    """fp32 elements of the smallest multiple of ``unit`` bytes that holds ``nbytes``."""
    return math.ceil(nbytes / unit) * unit // 4


def timed_allreduce(buf: torch.Tensor, fill: float, iters: int) -> float:
    """Mean device time in ms of ``iters`` in-place AllReduces of ``buf`` (refilled before each)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for _ in range(iters):
        buf.fill_(fill)
        start.record()
        dist.all_reduce(buf)
        stop.record()
        stop.synchronize()
        total += start.elapsed_time(stop)
    return total / max(iters, 1)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--alg", default=None, help="stragglar (default) | stragglar_a2a | ring | rhd | direct | rsag | auto")
    ap.add_argument("--straggler", type=int, default=None)
    args = ap.parse_args()

    env = os.environ
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env.setdefault("MASTER_PORT", "29500")
    rank, world, local = int(env.get("RANK", "0")), int(env.get("WORLD_SIZE", "1")), int(env.get("LOCAL_RANK", "0"))
    count = padded_elements(args.bytes)
    env.setdefault("STRAGGLAR_ARENA_MB", str(count * 4 // (1 << 20) + 384))
    opts = {k: v for k, v in (("alg", args.alg), ("straggler", args.straggler)) if v is not None}
    if opts:
        sp.configure(**opts)
    dist.init_process_group("cpu:gloo,cuda:stragglar", rank=rank, world_size=world)
    print(count)

    if not torch.cuda.is_available():
        host = torch.full((count,), float(rank))
        dist.all_reduce(host)                      # gloo
        print(f"cpu allreduce: {host}")
        dist.destroy_process_group()
        return 0

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    buf = sp.empty_symmetric(count, dtype=torch.float32, device=dev)
    buf.fill_(float(rank))
    print(f"Device ID of CUDA tensor: {buf.get_device()} | size: {buf.size()}")
    dist.all_reduce(buf)
    print(f"cuda allreduce: {buf}")
    want = float(sum(range(world)))
    latency = timed_allreduce(buf, float(rank), args.iters)
    print(f"Rank: {rank} | Avg latency: {latency}")
    status = sp.check_status(dev)
    ok = status == 0 and bool((buf == want).all())
    if not ok:
        print(f"Rank: {rank} | FAILED: status {status}, first element {float(buf[0])}, expected {want}", file=sys.stderr)
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
