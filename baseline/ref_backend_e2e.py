"""End-to-end AllReduce step through the reference's own c10d backend ("dummy"), for the reference arm.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        baseline/ref_backend_e2e.py --steps 10 --warmup 3 --delay-ms 5

Runs only the unmodified reference (``baseline/_ref/dummy_collectives*.so``, built from
implementation/custom_backend) and stock PyTorch; nothing of this library is imported.  The flow is the
reference's example.py (a 1 GiB fp32 tensor rounded to a multiple of 7 KiB, ``dist.all_reduce``,
example.py:18-40) with the device placement of its dp.py (logical rank 6, its hard-wired straggler, runs on the
last device and vice versa, dp.py:68-80; the backend does the same swap in its constructor, dummy.cpp:157-168).
Every step copies the input from pinned host memory, holds the straggler back with ``torch.cuda._sleep``,
all-reduces and reads 4 KiB of the result back.  The backend enqueues its NCCL calls on streams of its own and
reports every Work as complete at once (dummy.cpp:137-151), so the step has to synchronise the device before
and after the collective to be correct; those synchronisations are part of what a user of that backend pays.

The backend supports exactly 8 ranks (its schedule is written out for 8, dummy.cpp:273-656) and fp32.
Rank 0 prints one JSON line.
"""
import argparse
import json
import math
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "_ref"))

STRAGGLER_RANK = 6   # fixed in the reference (dummy.cpp:157, dp.py:22)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--delay-ms", type=float, default=5.0)
    ap.add_argument("--bytes", type=int, default=0)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    import dummy_collectives  # noqa: F401  (registers the backend "dummy")

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if world != 8:
        if rank == 0:
            print(json.dumps({"unavailable": f"the reference backend is written for 8 ranks, not {world}"}))
        return 0
    dev_index = world - 1 if local == STRAGGLER_RANK else STRAGGLER_RANK if local == world - 1 else local
    dev = torch.device("cuda", dev_index)
    dist.init_process_group(backend="dummy", rank=rank, world_size=world, device_id=dev)
    torch.cuda.set_device(dev)

    nbytes = args.bytes or math.ceil((1 << 30) / (1024 * 7)) * 1024 * 7
    count = nbytes // 4
    host_in = torch.empty(count, dtype=torch.float32).pin_memory()
    host_in.uniform_(-1, 1)
    host_out = torch.empty(1024, dtype=torch.float32).pin_memory()
    x = torch.empty(count, dtype=torch.float32, device=dev)
    # cycles of torch.cuda._sleep for the delay: calibrate against events on this device
    cycles = 0
    if args.delay_ms > 0 and rank == STRAGGLER_RANK:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        probe = 10_000_000
        torch.cuda._sleep(probe)
        e0.record(); torch.cuda._sleep(probe); e1.record(); e1.synchronize()
        cycles = int(probe * args.delay_ms / e0.elapsed_time(e1))

    def step():
        x.copy_(host_in, non_blocking=True)
        if cycles:
            torch.cuda._sleep(cycles)
        torch.cuda.synchronize()        # the backend's streams do not wait for the caller's stream
        dist.all_reduce(x)
        torch.cuda.synchronize()        # nor does the caller's stream wait for the backend's
        host_out.copy_(x[:1024], non_blocking=True)

    for _ in range(max(args.warmup, 1)):
        step()
    torch.cuda.synchronize()
    # No barrier is available (the backend implements allreduce only); the last warm-up step has just aligned
    # the ranks.  Wall clock around fully synchronised steps, per rank; rank 0 reports its own.
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    if rank == 0:
        net = ms - max(args.delay_ms, 0.0)
        print(json.dumps({"ms_per_step": ms, "steps": args.steps, "value": world * nbytes / 1e9 / (net / 1e3),
                          "unit": "GB/s", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 4096,
                          "path": "pinned host -> device -> dist.all_reduce on the reference's 'dummy' backend -> 4 KiB back",
                          "timing": "host clock of rank 0 around synchronised steps (the backend has no barrier and its "
                                    "Work objects carry no events)"}), flush=True)
    os._exit(0)   # the backend's destructor destroys NCCL communicators without an order between ranks


if __name__ == "__main__":
    sys.exit(main())
