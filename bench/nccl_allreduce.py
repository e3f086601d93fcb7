"""Stock NCCL AllReduce baseline ("NCCL ring" in the comparisons), measured the
same way as the library's own benchmark: one process per GPU, per-rank CUDA
events after a barrier, maximum over ranks, optional device delay on the
straggler (same %globaltimer kernel), the delay taken off for the bandwidth
columns.

    torchrun --nproc-per-node=8 --master-addr 127.0.0.1 bench/nccl_allreduce.py \
        --sizes 1048576,67108864,1073741824 --delays=-1,5 --iters 20 --warmup 5

Prints CSV rows with the columns of ``bin/allreduce`` (algorithm = nccl).
A delay of -1 or 0 means no delay (NCCL has no pre-phase to hide).
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200 import ops  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="1073741824")
    ap.add_argument("--delays", default="-1")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--straggler", type=int, default=-1)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    dtype = getattr(torch, args.dtype)
    straggler = args.straggler if args.straggler >= 0 else world - 1
    if rank == 0:
        print("algorithm,buffer_size_bytes,iteration,delay,runtime_ms,BW(GB/s),n,dtype,path,time_us_max,algbw_GBps,"
              "busbw_GBps,roofline_frac,real_delay_ms", flush=True)
    for size in [int(s) for s in args.sizes.split(",")]:
        esize = torch.empty(0, dtype=dtype).element_size()
        x = torch.empty(size // esize, dtype=dtype, device=dev)
        for delay in [float(d) for d in args.delays.split(",")]:
            real_delay = 0.0
            if delay > 0:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ops.delay(0.001)
                best = 1e9
                for _ in range(3):
                    e0.record(); ops.delay(delay); e1.record(); e1.synchronize()
                    best = min(best, e0.elapsed_time(e1))
                t = torch.tensor([best if rank == straggler else 0.0], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                real_delay = float(t.item())
            for it in range(-args.warmup, args.iters):
                ops.fill_uniform(x, rank + 131 * (it + args.warmup))
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if delay > 0 and rank == straggler:
                    ops.delay(delay)
                dist.all_reduce(x)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
                if it < 0 or rank != 0:
                    continue
                net = ms - real_delay
                algbw = size / 1e9 / (net / 1e3)
                ref_bw = size / 2**30 * 1000.0 / (ms - max(delay, 0.0))
                roof = 2.0 * (world - 1) / world * size / 770e9 * 1e3
                print(f"nccl,{size},{it + 1},{delay:.3f},{ms:.3f},{ref_bw:.3f},{world},{args.dtype},nccl,{ms * 1e3:.1f},"
                      f"{algbw:.2f},{algbw * 2 * (world - 1) / world:.2f},{roof / net:.3f},{real_delay:.3f}", flush=True)
        del x
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
