"""End-to-end data-parallel training on the straggler-aware backend.

    torchrun --nproc-per-node=8 --master-addr 127.0.0.1 examples/train_ddp.py \
        --backend stragglar --straggler 7 --delay-ms 20 --steps 30

The counterpart of the reference's implementation/custom_backend/dp.py and
motivation/dp_llama.py, with three differences: (1) the model is a random-init
Llama-style decoder of the Llama-3.2-1B shape and the batches are token ids
drawn uniformly from the vocabulary (no network: no checkpoint, no Alpaca);
(2) gradients are synchronised by the real ``DistributedDataParallel`` wrapper
(25 MB buckets, overlapped with the backward pass) with a communication hook
that fuses the average into the collective, instead of one flat all_reduce
after the backward pass (dp.py:50-65); (3) the straggler is made on purpose:
rank ``--straggler`` is held back ``--delay-ms`` on the device at the start
of every step, and the schedule is re-labelled so that it plays the last rank.
``--backend nccl`` runs the same loop on stock NCCL for comparison.

Per step and rank it prints the reference's log line
(``Rank r | Step s | Forward Time ... | AR Time ...``, dp.py:283), which
``python -m stragglar_b200.detect`` reads; rank 0 also prints tokens/s.
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200.models import LlamaConfig, LlamaForCausalLM  # noqa: E402

from stragglar_b200.utils.logfmt import format_step  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="stragglar", choices=["stragglar", "nccl"])
    ap.add_argument("--alg", default="stragglar")
    ap.add_argument("--straggler", type=int, default=-1, help="rank that is late every step (default: the last)")
    ap.add_argument("--delay-ms", type=float, default=20.0)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--tiny", action="store_true", help="a 2-layer model for smoke tests")
    ap.add_argument("--lr", type=float, default=5e-5)
    ap.add_argument("--grad-sync", default="ddp", choices=["ddp", "flat", "per-param"],
                    help="ddp: DistributedDataParallel buckets overlapped with backward; flat: one all_reduce of "
                         "the flattened gradients after backward (the reference's dp.py); per-param: one all_reduce "
                         "per parameter (the reference's dp_llama.py)")
    ap.add_argument("--auto-straggler", action="store_true",
                    help="find the late rank at run time (StragglerMonitor) instead of trusting --straggler")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    straggler = args.straggler if args.straggler >= 0 else world - 1

    if args.backend == "stragglar":
        import stragglar_b200.parallel as sp
        from stragglar_b200 import ops
        sp.configure(alg=args.alg, straggler=straggler)
        dist.init_process_group("stragglar", rank=rank, world_size=world)
    else:
        from stragglar_b200 import ops
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    torch.manual_seed(1234)   # the same initial weights everywhere; DDP broadcasts them anyway
    cfg = LlamaConfig.tiny() if args.tiny else LlamaConfig.llama32_1b()
    model = LlamaForCausalLM(cfg).to(dev, dtype=getattr(torch, args.dtype))
    from stragglar_b200.parallel.grad_sync import FlatGradSync, allreduce_gradients_per_param
    flat_sync = None
    if args.grad_sync == "ddp":
        ddp = DDP(model, device_ids=[local], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
        if args.backend == "stragglar":
            ddp.register_comm_hook(None, sp.fused_avg_hook)
    else:
        ddp = model                       # gradients are averaged by hand after the backward pass
        for p in model.parameters():
            dist.broadcast(p.data, src=0)
        if args.grad_sync == "flat":
            flat_sync = FlatGradSync(model)
    opt = torch.optim.AdamW(ddp.parameters(), lr=args.lr)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: min(1.0, (s + 1) / 50))
    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    nparams = sum(p.numel() for p in model.parameters())
    grad_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    if rank == 0:
        print(f"model: {nparams / 1e9:.3f} B parameters, {grad_bytes / 2**20:.0f} MiB of gradients per step, "
              f"backend {args.backend}, straggler rank {straggler} (+{args.delay_ms} ms)", flush=True)

    monitor = None
    if args.backend == "stragglar" and args.auto_straggler:
        monitor = sp.StragglerMonitor(window=5, threshold=0.8, device=dev)
    tokens_per_step = world * args.micro_batch * args.seq_len
    times = []
    for step in range(args.warmup + args.steps):
        ids_host = torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq_len), generator=gen).pin_memory()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        dist.barrier()
        torch.cuda.synchronize()
        t_host = time.perf_counter()
        ev[0].record()
        if rank == straggler and args.delay_ms > 0 and world > 1:
            ops.delay(args.delay_ms)                       # the persistent straggler
        ids = ids_host.to(dev, non_blocking=True)
        torch.cuda.nvtx.range_push("Forward")
        loss = ddp(ids, labels=ids)
        torch.cuda.nvtx.range_pop()
        ev[1].record()
        torch.cuda.nvtx.range_push("Backward+AllReduce_Gradients")
        loss.backward()                                    # with DDP the bucket AllReduces overlap this
        torch.cuda.nvtx.range_pop()
        if args.grad_sync != "ddp":
            torch.cuda.nvtx.range_push("AllReduce_Gradients")
            flat_sync() if flat_sync is not None else allreduce_gradients_per_param(model)
            torch.cuda.nvtx.range_pop()
        ev[2].record()
        opt.step(); sched.step(); opt.zero_grad(set_to_none=False)
        ev[3].record()
        loss_val = loss.item()                             # device -> host read of the step's result
        torch.cuda.synchronize()
        iter_ms = ev[0].elapsed_time(ev[3])
        fwd, bwd = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
        # the gradient AllReduces overlap the backward pass, so "AR Time" is the backward time
        print(format_step(rank, step, fwd, bwd, loss_val, iter_ms, bwd, grad_bytes) + "\n", flush=True)
        t = torch.tensor([iter_ms], device=dev)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        if monitor is not None:
            monitor.step()
        if step >= args.warmup:
            times.append(max(float(a.item()) for a in allt))
    if args.backend == "stragglar":
        st = sp.check_status(dev)
        assert st == 0, f"device status {st}"
    if rank == 0 and times:
        ms = sum(times) / len(times)
        print(f"RESULT backend={args.backend} alg={args.alg} world={world} step_ms={ms:.2f} "
              f"tokens_per_s={tokens_per_step / (ms / 1e3):.0f} delay_ms={args.delay_ms} straggler={straggler}", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
