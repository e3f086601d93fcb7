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

``--model-dir DIR`` loads a checkpoint in the Hugging Face layout (written by ``examples/load_model.py`` or by
``save_pretrained``) instead of initialising at random; ``--data-dir DIR`` trains on the instruction dataset
prepared by ``examples/load_dataset.py`` (prompt format, 512-token padding, batch 4 and ``DistributedSampler`` as
in dp.py:87-119) instead of uniform random token ids; ``--cpu`` runs the whole loop on CPU tensors (the backend's
host executor, or gloo), which is how the script is tested without a GPU.

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
    ap.add_argument("--hook", default="symmetric", choices=["fused", "symmetric", "bf16"],
                    help="stragglar backend, ddp: symmetric = buckets reduced in buffers of the symmetric heap (the "
                         "fastest: 4 x B200, 136.0 ms per step against 144.1 for fused and 137.0 for NCCL); fused = "
                         "all_reduce of the bucket itself with the fused average (one staged kernel per bucket); bf16 = "
                         "fused, bfloat16 on the wire")
    ap.add_argument("--auto-straggler", action="store_true",
                    help="find the late rank at run time (StragglerMonitor) instead of trusting --straggler")
    ap.add_argument("--model-dir", default=None, help="checkpoint directory (config.json + safetensors)")
    ap.add_argument("--data-dir", default=None, help="dataset directory written by examples/load_dataset.py")
    ap.add_argument("--samples", type=int, default=8192, help="records of --data-dir to use")
    ap.add_argument("--max-length", type=int, default=512, help="tokens per example with --data-dir")
    ap.add_argument("--cpu", action="store_true", help="CPU tensors (backend stragglar or gloo); for tests")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    cuda = not args.cpu
    if cuda:
        from stragglar_b200.utils.affinity import bind_to_gpu
        bind_to_gpu(local)                 # host threads and pinned batches next to this rank's GPU
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    straggler = args.straggler if args.straggler >= 0 else world - 1

    if args.backend == "stragglar":
        import stragglar_b200.parallel as sp
        if (args.grad_sync == "flat" or args.hook == "symmetric") and not args.tiny and cuda:
            # the flat gradient buffer (2.4 GB of bf16 for the 1B shape, twice that in fp32) lives in the symmetric heap
            os.environ.setdefault("STRAGGLAR_ARENA_MB", "6144")
        sp.configure(alg=args.alg, straggler=straggler)
        dist.init_process_group("stragglar", rank=rank, world_size=world)
    elif cuda:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    if cuda:
        from stragglar_b200 import ops

    class Stamp:
        """A point in time on the device stream (CUDA event) or on the host (--cpu)."""
        def __init__(self):
            self.ev = torch.cuda.Event(enable_timing=True) if cuda else None
            self.t = 0.0
        def record(self):
            if cuda:
                self.ev.record()
            else:
                self.t = time.perf_counter()
        def ms_until(self, other):
            return self.ev.elapsed_time(other.ev) if cuda else (other.t - self.t) * 1e3

    def sync():
        if cuda:
            torch.cuda.synchronize()

    def nvtx_push(name):
        if cuda:
            torch.cuda.nvtx.range_push(name)

    def nvtx_pop():
        if cuda:
            torch.cuda.nvtx.range_pop()

    torch.manual_seed(1234)   # the same initial weights everywhere; DDP broadcasts them anyway
    if args.model_dir:
        model = LlamaForCausalLM.from_pretrained(args.model_dir).to(dev, dtype=getattr(torch, args.dtype))
        cfg = model.cfg
    else:
        cfg = LlamaConfig.tiny() if args.tiny else LlamaConfig.llama32_1b()
        model = LlamaForCausalLM(cfg).to(dev, dtype=getattr(torch, args.dtype))
    from stragglar_b200.parallel.grad_sync import FlatGradSync, allreduce_gradients_per_param
    flat_sync = None
    if args.grad_sync == "ddp":
        ddp = DDP(model, device_ids=[local] if cuda else None, bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
        if args.backend == "stragglar":
            ddp.register_comm_hook(None, {"fused": sp.fused_avg_hook, "bf16": sp.bf16_fused_avg_hook}.get(args.hook)
                                   or sp.SymmetricBucketHook())
    else:
        ddp = model                       # gradients are averaged by hand after the backward pass
        for p in model.parameters():
            dist.broadcast(p.data, src=0)
        if args.grad_sync == "flat":
            flat_sync = FlatGradSync(model)
    opt = torch.optim.AdamW(ddp.parameters(), lr=args.lr)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: min(1.0, (s + 1) / 50))
    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    batches = None
    seq_len = args.seq_len
    if args.data_dir:
        from torch.utils.data import DataLoader
        from torch.utils.data.distributed import DistributedSampler
        from stragglar_b200.utils.data import InstructionDataset, load_records, load_tokenizer
        tok = load_tokenizer(args.model_dir)
        assert tok.vocab_size <= cfg.vocab_size, f"tokenizer has {tok.vocab_size} tokens, the model {cfg.vocab_size}"
        ds = InstructionDataset(load_records(args.data_dir, args.samples), tok, args.max_length)
        sampler = DistributedSampler(ds, num_replicas=world, rank=rank, shuffle=True, seed=0)
        loader = DataLoader(ds, batch_size=args.micro_batch, sampler=sampler, drop_last=True, pin_memory=cuda)
        seq_len = args.max_length

        def batch_stream():
            epoch = 0
            while True:
                sampler.set_epoch(epoch)
                yield from loader
                epoch += 1
        batches = batch_stream()
    nparams = sum(p.numel() for p in model.parameters())
    grad_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    if rank == 0:
        print(f"model: {nparams / 1e9:.3f} B parameters, {grad_bytes / 2**20:.0f} MiB of gradients per step, "
              f"backend {args.backend}, straggler rank {straggler} (+{args.delay_ms} ms)", flush=True)

    monitor = None
    if args.backend == "stragglar" and args.auto_straggler:
        monitor = sp.StragglerMonitor(window=5, threshold=0.8, device=dev)
    tokens_per_step = world * args.micro_batch * seq_len
    times, exposed = [], []
    nvtx_push("Epoch 0")                                   # the ranges of the reference's loop (dp.py:157,162,286,293)
    for step in range(args.warmup + args.steps):
        nvtx_push(f"Step {step}")
        if batches is not None:
            batch = next(batches)
            ids_host, labels_host = batch["input_ids"], batch["labels"]
        else:
            ids_host = torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq_len), generator=gen)
            labels_host = ids_host
        if cuda:
            ids_host, labels_host = ids_host.pin_memory(), labels_host.pin_memory()
        ev = [Stamp() for _ in range(5)]
        dist.barrier()
        sync()
        ev[0].record()
        if rank == straggler and args.delay_ms > 0 and world > 1:
            if cuda:
                ops.delay(args.delay_ms)                   # the persistent straggler, held back on the device
            else:
                time.sleep(args.delay_ms / 1e3)
        ids = ids_host.to(dev, non_blocking=True)
        labels = ids if labels_host is ids_host else labels_host.to(dev, non_blocking=True)
        nvtx_push("Forward")
        loss = ddp(ids, labels=labels)
        nvtx_pop()
        ev[1].record()
        nvtx_push("Backward+AllReduce_Gradients")
        loss.backward()                                    # with DDP the bucket AllReduces overlap this
        nvtx_pop()
        ev[4].record()
        if args.grad_sync != "ddp":
            nvtx_push("AllReduce_Gradients")
            flat_sync() if flat_sync is not None else allreduce_gradients_per_param(model, nvtx=True)
            nvtx_pop()
        ev[2].record()
        opt.step(); sched.step(); opt.zero_grad(set_to_none=False)
        ev[3].record()
        loss_val = loss.item()                             # device -> host read of the step's result
        sync()
        nvtx_pop()                                         # Step
        iter_ms = ev[0].ms_until(ev[3])
        fwd, bwd = ev[0].ms_until(ev[1]), ev[1].ms_until(ev[4])
        # flat / per-param: the AllReduce follows the backward pass and is timed on its own (exposed communication);
        # ddp: the bucket AllReduces overlap the backward pass, so "AR Time" is the backward time
        ar = ev[4].ms_until(ev[2]) if args.grad_sync != "ddp" else bwd
        print(format_step(rank, step, fwd, bwd, loss_val, iter_ms, ar, grad_bytes) + "\n", flush=True)
        t = torch.tensor([iter_ms, ar], device=dev)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        if monitor is not None:
            monitor.step()
        if step >= args.warmup:
            times.append(max(float(a[0].item()) for a in allt))
            exposed.append(max(float(a[1].item()) for a in allt))
    nvtx_pop()                                             # Epoch
    if args.backend == "stragglar":
        st = sp.check_status(dev)
        assert st == 0, f"device status {st}"
    if rank == 0 and times:
        ms = sum(times) / len(times)
        ar_ms = sum(exposed) / len(exposed)
        what = "exposed_allreduce_ms" if args.grad_sync != "ddp" else "backward_with_overlapped_allreduce_ms"
        print(f"RESULT backend={args.backend} alg={args.alg} grad_sync={args.grad_sync} world={world} step_ms={ms:.2f} "
              f"tokens_per_s={tokens_per_step / (ms / 1e3):.0f} {what}={ar_ms:.2f} steps={len(times)} "
              f"delay_ms={args.delay_ms} straggler={straggler}", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
