"""The library's op tables executed the reference's way: every round as
grouped NCCL send/recv calls plus separate add kernels, issued from the host
(stragglar_b200.parallel.cpu_exec.SendRecvExecutor on CUDA tensors).  This is
the baseline for GPU counts the reference has no program for (e.g. 6), and it
shows what the persistent peer-memory kernel saves over host-driven rounds.

    torchrun --nproc-per-node=6 --master-addr 127.0.0.1 bench/sendrecv_allreduce.py \
        --alg stragglar --sizes 16777216,268435456 --delays=5 --iters 10

Prints CSV rows with the columns of ``bin/allreduce`` (path = nccl_sendrecv).
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200 import ops  # noqa: E402
from stragglar_b200.compiler import compile_program  # noqa: E402
from stragglar_b200.parallel.cpu_exec import SendRecvExecutor  # noqa: E402
from stragglar_b200.synth import synthesize  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--alg", default="stragglar")
    ap.add_argument("--sizes", default="268435456")
    ap.add_argument("--delays", default="5")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ex = SendRecvExecutor(tile_elems=1 << 15)
    if rank == 0:
        print("algorithm,buffer_size_bytes,iteration,delay,runtime_ms,BW(GB/s),n,dtype,path,time_us_max,algbw_GBps,"
              "busbw_GBps,roofline_frac,real_delay_ms", flush=True)
    for size in [int(s) for s in args.sizes.split(",")]:
        x = torch.empty(size // 4, device=dev)
        for delay in [float(d) for d in args.delays.split(",")]:
            prog = compile_program(args.alg, world, prephase=delay >= 0)
            want = None
            for it in range(-args.warmup, args.iters):
                ops.fill_uniform(x, rank)
                if delay < 0:
                    raise SystemExit("the send/recv baseline times the pre-phase too: use a delay >= 0")
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if delay > 0 and rank == world - 1:
                    ops.delay(delay)
                ex.all_reduce(prog, x)
                e1.record()
                torch.cuda.synchronize()
                bad, worst = ops.verify_uniform_sum(x, list(range(world)), atol=2e-5)
                assert bad == 0, (bad, worst)
                t = torch.tensor([e0.elapsed_time(e1)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
                if it < 0 or rank != 0:
                    continue
                net = ms - max(delay, 0.0)
                algbw = size / 1e9 / (net / 1e3)
                print(f"{args.alg},{size},{it + 1},{delay:.3f},{ms:.3f},{size / 2**30 * 1000 / net:.3f},{world},float32,"
                      f"nccl_sendrecv,{ms * 1e3:.1f},{algbw:.2f},{algbw * 2 * (world - 1) / world:.2f},nan,{max(delay, 0.0):.3f}",
                      flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
