"""``dist.all_reduce`` through a c10d backend, one process per GPU: stock NCCL (the "NCCL ring" baseline of the
comparisons) or this library's ``stragglar`` backend, measured the same way as ``bin/allreduce``: per-rank CUDA
events after a barrier, maximum over ranks, optional device delay on the straggler (same %globaltimer kernel), the
delay taken off for the bandwidth columns.

    torchrun --nproc-per-node=8 --master-addr 127.0.0.1 bench/backend_allreduce.py \
        --sizes 1048576,26214400,1073741824 --delays=-1,5 --iters 20 --warmup 5 \
        [--backend stragglar --alg auto|rsag|stragglar_a2a|stragglar|ring [--symmetric] [--comm-dtype bfloat16]]

With ``--backend stragglar`` the tensor is an ordinary CUDA tensor, as a DistributedDataParallel bucket is (one
kernel copies it in, reduces and copies it out), or, with ``--symmetric``, a tensor of the backend's symmetric heap
(reduced in place).  Prints CSV rows with the columns of ``bin/allreduce`` (algorithm = nccl, or the algorithm's name
with the kind of tensor).  A delay of -1 or 0 means no delay.
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
    ap.add_argument("--backend", default="nccl", choices=["nccl", "stragglar"])
    ap.add_argument("--alg", default="auto", help="stragglar backend: comma-separated algorithms")
    ap.add_argument("--symmetric", action="store_true", help="stragglar backend: tensors of the symmetric heap")
    ap.add_argument("--comm-dtype", default="", help="stragglar backend: dtype on the wire (all_reduce_ex)")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dtype = getattr(torch, args.dtype)
    straggler = args.straggler if args.straggler >= 0 else world - 1
    sizes = [int(s) for s in args.sizes.split(",")]
    sp = None
    if args.backend == "nccl":
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        algs = ["nccl"]
    else:
        import stragglar_b200.parallel as sp
        os.environ.setdefault("STRAGGLAR_STAGING_MB", str(min(max(sizes) // (1 << 20) + 1, 256)))
        os.environ.setdefault("STRAGGLAR_ARENA_MB", str((max(sizes) // (1 << 20) + 1) * (2 if args.symmetric else 0) + 320))
        sp.configure(alg=args.alg.split(",")[0], straggler=args.straggler)
        dist.init_process_group("stragglar", rank=rank, world_size=world)
        algs = args.alg.split(",")
    comm_dtype = getattr(torch, args.comm_dtype) if args.comm_dtype else None
    if rank == 0:
        print("algorithm,buffer_size_bytes,iteration,delay,runtime_ms,BW(GB/s),n,dtype,path,time_us_max,algbw_GBps,"
              "busbw_GBps,roofline_frac,real_delay_ms", flush=True)
    for size in sizes:
        esize = torch.empty(0, dtype=dtype).element_size()
        if sp is not None and args.symmetric:
            x = sp.empty_symmetric(size // esize, dtype=dtype, device=dev)
        else:
            x = torch.empty(size // esize, dtype=dtype, device=dev)
        for alg in algs:
            if sp is not None:
                sp.set_algorithm(alg, dev)
            label = alg if sp is None else alg + ("+symm" if args.symmetric else "+bucket") + (f"+{args.comm_dtype}" if comm_dtype else "")
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
                    if comm_dtype is not None and sp is not None:
                        sp.all_reduce_ex(x, average=False, comm_dtype=comm_dtype).wait()
                    else:
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
                    print(f"{label},{size},{it + 1},{delay:.3f},{ms:.3f},{ref_bw:.3f},{world},{args.dtype},{args.backend},{ms * 1e3:.1f},"
                          f"{algbw:.2f},{algbw * 2 * (world - 1) / world:.2f},{roof / net:.3f},{real_delay:.3f}", flush=True)
        del x
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
