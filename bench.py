#!/usr/bin/env python
"""Headline benchmark: straggler-aware AllReduce on the GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

One process per GPU.  A step is: the straggler (the last rank) is held back by
``--delay-ms`` on the device, then all ranks AllReduce a ``--bytes`` buffer
(default 1 GiB rounded up to a multiple of 7 KiB, the size the reference's
micro-benchmark uses, implementation/custom_backend/example.py:18-19) of
``--dtype`` with ``--alg`` through this library's c10d backend.

Printed (rank 0, one JSON line): ``value`` = aggregate AllReduce throughput
N * bytes / (time per step - delay) in GB/s, i.e. the reference's
"BW = bytes / (ms - sleep)" (stragglar/allreduce_8GPU.cu:1054-1059) summed over
the N buffers.  Two measurements: the device-timed one (buffers resident in the
backend's symmetric heap, CUDA events, max over ranks) and ``e2e`` (every step
copies the input from pinned host memory, reduces it through
``dist.all_reduce`` and reads part of the result back).  ``--impl reference``
runs the unmodified reference program instead (4 or 8 GPUs only).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GIB = 1 << 30


def default_bytes() -> int:
    return math.ceil(GIB / (1024 * 7)) * 1024 * 7


def bench_bytes(requested: int, n: int, esize: int = 4) -> int:
    """Bytes per GPU that both arms use: the request (default: 1 GiB rounded up to a multiple of 7 KiB), cut to a whole
    number of elements per StragglAR chunk (n - 1 chunks), which the reference program needs
    (stragglar/allreduce_8GPU.cu:877) and this library does not mind."""
    nbytes = requested or default_bytes()
    unit = esize * max(n - 1, 1)
    return nbytes - nbytes % unit


def bench_config(alg: str, n: int, nbytes: int, delay_ms: float, straggler: int) -> dict:
    """The `config` entry of the JSON line; the same for both arms (what differs between them is said under `notes`)."""
    return {"model": f"allreduce {alg}", "bytes_per_gpu": nbytes, "delay_ms": delay_ms, "straggler_rank": straggler,
            "global_batch": None, "seq_len": None, "parallelism": f"dp{n}", "l2": "buffer per GPU larger than L2"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 7:
                    self.rows.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self) -> dict:
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.rows[0][1]),
                "power_w_max": max(float(r[2]) for r in self.rows if r[2].replace(".", "").isdigit()) if self.rows else None,
                "reasons": sorted(reasons), "samples": len(self.rows)}


def reference_backend_e2e(args) -> dict:
    """The end-to-end step through the reference's own c10d backend (baseline/ref_backend_e2e.py), run as eight
    processes of its own (the backend is written for exactly 8 ranks).  STRAGGLAR_REF_E2E=0 skips it."""
    script = os.path.join(ROOT, "baseline", "ref_backend_e2e.py")
    port = 20000 + (os.getpid() % 20000)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "8", "--master-addr", "127.0.0.1",
           "--master-port", str(port), script, "--steps", str(max(3, min(args.steps, 10))), "--warmup", "3",
           "--delay-ms", str(args.delay_ms)]
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_PORT", "MASTER_ADDR", "GROUP_RANK", "ROLE_RANK",
                        "LOCAL_WORLD_SIZE", "ROLE_WORLD_SIZE", "TORCHELASTIC_RUN_ID")}
    try:
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference backend did not finish its end-to-end steps within 300 s"}
    for line in reversed(p.stdout.splitlines()):
        line = line.strip()
        if line.startswith("{") and "ms_per_step" in line:
            try:
                return json.loads(line)
            except ValueError:
                pass
    return {"unavailable": f"the reference backend run exited {p.returncode}: {(p.stderr or p.stdout)[-200:]!r}"}


def run_reference(args) -> int:
    """The reference arm: the unmodified stragglar/allreduce_{4,8}GPU.cu
    program, built with nvcc as its README says, run by rank 0 on all N GPUs
    (it is a single-process program); the other ranks only wait."""
    rank = int(os.environ.get("RANK", "0"))
    n = args.gpus
    exe = os.path.join(ROOT, "baseline", "_ref", f"allreduce{n}")
    out = {"impl": "reference"}
    if n not in (4, 8):
        out["unavailable"] = f"the reference ships AllReduce programs for 4 and 8 GPUs only (README.md:26-30), not {n}"
    elif not os.path.exists(exe):
        out["unavailable"] = f"{os.path.relpath(exe, ROOT)} is not built (see baseline/README.md)"
    if "unavailable" in out:
        if rank == 0:
            print(json.dumps(out), flush=True)
        return 0
    done = os.path.join(ROOT, f".ref_done_{os.environ.get('MASTER_PORT', '0')}")
    if rank != 0:
        # rank 0 drives all GPUs from one process; stay off them
        t0 = time.time()
        while not os.path.exists(done) and time.time() - t0 < 3600:
            time.sleep(0.5)
        return 0
    try:
        nbytes = bench_bytes(args.bytes, n)
        with ClockSampler(0) as cs:
            t0 = time.time()
            # the program runs one iteration more than asked and discards the first (stragglar/allreduce_8GPU.cu:1009,1053)
            p = subprocess.run([exe, str(nbytes), args.alg, str(args.steps), str(args.delay_ms)], capture_output=True,
                               text=True, timeout=1800)
            wall = time.time() - t0
        rows = [l.split(",") for l in p.stdout.splitlines() if l.startswith(args.alg + ",")]
        if p.returncode != 0 or not rows:
            out["unavailable"] = f"reference program exited {p.returncode}: {(p.stderr or p.stdout)[-200:]!r}"
            print(json.dumps(out), flush=True)
            return 0
        e2e = {"unavailable": "the reference program fills its buffers on the device and reads nothing back: it has "
                              "no host path to time (stragglar/allreduce_8GPU.cu:1010-1020)"}
        if n == 8 and args.alg == "stragglar" and not args.no_e2e and os.environ.get("STRAGGLAR_REF_E2E", "1") != "0":
            e2e = reference_backend_e2e(args)
        ms = statistics.mean(float(r[4]) for r in rows)
        delay = max(args.delay_ms, 0.0)
        value = n * nbytes / 1e9 / ((ms - delay) / 1e3)
        out.update({"metric": "allreduce_aggregate_GBps", "value": value, "unit": "GB/s", "n_gpus": n, "steps": len(rows),
                    "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                    "dtype": "fp32", "data": "synthetic: constant fill (rank r holds r+1), as the reference program does",
                    "clocks": cs.summary(), "wall_s": wall,
                    "e2e": e2e,
                    "config": bench_config(args.alg, n, nbytes, args.delay_ms, n - 1),
                    "notes": {"timing": "device 0 events only (the reference's own clock), nominal delay subtracted",
                              "warmup": "the program's own: 10 send/recv exchanges and one discarded extra iteration, "
                                        "whatever --warmup says (stragglar/allreduce_8GPU.cu:992-1006,1053)",
                              "processes": f"1 process x {n} GPUs, NCCL send/recv"}})
        print(json.dumps(out), flush=True)
    finally:
        open(done, "w").close()
        time.sleep(3.0)    # the waiting ranks poll twice a second
        try:
            os.remove(done)
        except OSError:
            pass
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bytes", type=int, default=0)
    ap.add_argument("--alg", default="stragglar")
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16", "float16"])
    ap.add_argument("--delay-ms", type=float, default=5.0, help="device delay of the straggler per step (0: none)")
    ap.add_argument("--straggler", type=int, default=-1, help="physical rank that is late (default: the last)")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    import stragglar_b200.parallel as sp
    from stragglar_b200 import ops
    from stragglar_b200.compiler import compile_program, status_string

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run "
                  f"--nproc-per-node {args.gpus}", file=sys.stderr)
        return 2
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    # host threads and pinned buffers on the CPUs next to this rank's GPU (matters for the end-to-end copies)
    from stragglar_b200.utils.affinity import bind_to_gpu
    bound = bind_to_gpu(local)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dtype = getattr(torch, args.dtype)
    esize = torch.empty(0, dtype=dtype).element_size()
    nbytes = bench_bytes(args.bytes, world, esize)
    count = nbytes // esize
    straggler = args.straggler if args.straggler >= 0 else world - 1
    delay_ms = args.delay_ms if world > 1 else 0.0

    os.environ.setdefault("STRAGGLAR_STAGING_MB", "64")
    os.environ.setdefault("STRAGGLAR_ARENA_MB", str(2 * int(nbytes / (1 << 20)) + 64 + 64 + 16))
    sp.configure(alg=args.alg, straggler=straggler)
    dist.init_process_group("stragglar", rank=rank, world_size=world)
    x = sp.empty_symmetric(count, dtype=dtype, device=dev)           # resident, reduced in place
    seeds = list(range(world))

    def device_step():
        if rank == straggler and delay_ms > 0:
            ops.delay(delay_ms)
        # AVG: the 1/world_size is fused into the kernel, and repeating the step in
        # place keeps the seeded values bounded (the mean of N equal vectors)
        dist.all_reduce(x, op=dist.ReduceOp.AVG)

    # warm-up; the first step is verified against the seeded inputs
    tol = {torch.float32: 2e-5, torch.bfloat16: 0.07, torch.float16: 0.01}[dtype]
    ops.fill_uniform(x, seeds[rank])
    device_step()
    torch.cuda.synchronize()
    st = sp.check_status(dev)
    if st:
        raise RuntimeError("collective failed: " + status_string(st))
    bad, worst = ops.verify_uniform_sum(x, seeds, scale=1.0 / world, atol=tol,
                                        rtol=1e-2 if dtype != torch.float32 else 1e-6)
    if bad:
        raise RuntimeError(f"rank {rank}: {bad} wrong elements after AllReduce (max abs error {worst})")
    for _ in range(args.warmup - 1):
        device_step()

    # the delay as this device serves it
    real_delay = 0.0
    if delay_ms > 0:
        if rank == straggler:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            best = 1e9
            for _ in range(3):
                e0.record(); ops.delay(delay_ms); e1.record(); e1.synchronize()
                best = min(best, e0.elapsed_time(e1))
            real_delay = best
        t = torch.tensor([real_delay], device=dev)
        dist.broadcast(t, src=straggler)
        real_delay = float(t.item())

    def timed(step_fn, steps):
        dist.barrier()
        torch.cuda.synchronize()
        l0 = sp.launches(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        launches = sp.launches(dev) - l0
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        allms = [torch.zeros_like(ms) for _ in range(world)]
        dist.all_gather(allms, ms)
        return max(float(m.item()) for m in allms) / steps, launches

    # clocks are sampled from here to the end of the end-to-end region (nvidia-smi answers in
    # ~100 ms, the device-timed region alone may be shorter than that)
    cs = ClockSampler(local)
    cs.__enter__()
    ms_step, launches = timed(device_step, args.steps)
    st = sp.check_status(dev)
    if st:
        raise RuntimeError("collective failed: " + status_string(st))
    if rank == straggler and delay_ms > 0:
        launches += args.steps   # the delay kernels
    net_ms = ms_step - real_delay
    value = world * nbytes / 1e9 / (net_ms / 1e3)

    # end to end: pinned host input -> device -> all_reduce (public API) -> part of the result back on the host
    e2e = None
    if not args.no_e2e:
        host_in = torch.empty(count, dtype=dtype).pin_memory()
        host_in.uniform_(-1, 1)
        back = 4096 // esize
        host_out = torch.empty(back, dtype=dtype).pin_memory()

        # The library's own way to reduce data that comes from the host every step: the copy is streamed through the
        # collective piece by piece (sp.HostStreamedAllReduce), so the delay and the AllReduce hide behind the copy.
        streamed = sp.HostStreamedAllReduce(count, dtype=dtype, device=dev, pieces=8) if world > 1 else None

        def e2e_step():
            if streamed is None:
                x.copy_(host_in, non_blocking=True)          # this step's input, from pinned host memory
                dist.all_reduce(x, op=dist.ReduceOp.AVG)
                res = x
            else:
                hold = (lambda: ops.delay(delay_ms)) if (rank == straggler and delay_ms > 0) else None
                res = streamed(host_in, op=dist.ReduceOp.AVG, before_collective=hold)
            host_out.copy_(res[:back], non_blocking=True)    # part of the result back on the host

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        e2e_steps = max(3, min(args.steps, 10))
        ms_e2e, _ = timed(e2e_step, e2e_steps)
        e2e = {"value": world * nbytes / 1e9 / ((ms_e2e - real_delay) / 1e3), "unit": "GB/s",
               "ms_per_step": ms_e2e, "steps": e2e_steps, "h2d_bytes_per_step": nbytes,
               "d2h_bytes_per_step": back * esize, "host_cpus_bound": len(bound) if bound else None,
               "path": "pinned host -> symmetric device tensor in 8 pieces, each reduced by dist.all_reduce(op=AVG) as it "
                       "lands (sp.HostStreamedAllReduce) -> 4 KiB of the result back"}

    # the NVSwitch-native variant of the same collective, device-timed the same way
    variants = {}
    if args.alg == "stragglar" and world > 2:
        sp.set_algorithm("stragglar_a2a", dev)
        ops.fill_uniform(x, seeds[rank])
        device_step()
        torch.cuda.synchronize()
        bad, worst = ops.verify_uniform_sum(x, seeds, scale=1.0 / world, atol=tol,
                                            rtol=1e-2 if dtype != torch.float32 else 1e-6)
        if bad:
            raise RuntimeError(f"rank {rank}: stragglar_a2a: {bad} wrong elements (max abs error {worst})")
        for _ in range(2):
            device_step()
        ms_v, _ = timed(device_step, args.steps)
        variants["stragglar_a2a"] = {"value": world * nbytes / 1e9 / ((ms_v - real_delay) / 1e3), "unit": "GB/s",
                                     "ms_per_step": ms_v, "time_us_net": (ms_v - real_delay) * 1e3}
        sp.set_algorithm(args.alg, dev)
        st = sp.check_status(dev)
        if st:
            raise RuntimeError("collective failed: " + status_string(st))

    cs.__exit__(None, None, None)
    prog_post = compile_program(args.alg, world, prephase=(delay_ms == 0), straggler=straggler)
    link_bytes = prog_post.link_bytes(nbytes)
    roof_ms = link_bytes / 770e9 * 1e3 if world > 1 else 2 * nbytes / 6532.5e9 * 1e3
    clocks = cs.summary()
    if rank == 0:
        out = {
            "metric": "allreduce_aggregate_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"float32": "fp32", "bfloat16": "bf16", "float16": "fp16"}[args.dtype],
            "data": "synthetic: uniform[-1,1) seeded per rank, averaged in place every step (first step verified)",
            "config": bench_config(args.alg, world, nbytes, args.delay_ms if world > 1 else 0.0, straggler),
            "notes": {"processes": f"{world} ranks, one per GPU, own peer-memory kernels over NVLink",
                      "timing": "CUDA events on every rank, max over ranks, measured delay subtracted"},
            "time_us_net": net_ms * 1e3, "real_delay_ms": real_delay,
            "algbw_GBps": nbytes / 1e9 / (net_ms / 1e3),
            "busbw_GBps": nbytes / 1e9 / (net_ms / 1e3) * 2 * (world - 1) / world,
            "roofline_frac_of_measured": roof_ms / net_ms if net_ms > 0 else None,
            "roofline_frac_of_nominal": ((roof_ms * 770.0 / 900.0) / net_ms if world > 1 else (roof_ms * 6532.5 / 7700.0) / net_ms)
                                        if net_ms > 0 else None,
            "roofline": ("busiest rank's bytes per direction / 770 GB/s measured peer copy (nominal: 900 GB/s per direction)"
                         if world > 1 else "read+write of the buffer / 6532.5 GB/s measured copy (nominal: 7.7 TB/s)"),
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "impl": "ours", "variants": variants,
        }
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
