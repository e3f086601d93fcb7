"""PyTorch integration: the ``stragglar`` c10d backend, symmetric tensors,
DistributedDataParallel communication hooks and the CPU/gloo table executor.

Importing this package registers the backend:

    import stragglar_b200.parallel as sp
    dist.init_process_group("stragglar")            # or "cpu:gloo,cuda:stragglar"
    dist.all_reduce(x)                              # StragglAR AllReduce, straggler = last rank
    sp.set_straggler(2)                             # physical rank 2 is the late one from now on
    buf = sp.empty_symmetric(n, dtype=torch.float32, device="cuda")   # reduced in place, no staging

Options can be given per process group (``sp.configure(alg="ring", blocks=32)``
before ``init_process_group``) or through ``STRAGGLAR_*`` environment
variables (ALG, STRAGGLER, PATH, BLOCKS, THREADS, TILE_BYTES, TIMEOUT_MS,
ARENA_MB, STAGING_MB, CPU_ARENA_MB).
"""
from __future__ import annotations

from typing import Optional

_options: dict = {}
_registered = False


def _ext():
    from . import _build_ext
    return _build_ext.load()


def configure(**options) -> None:
    """Options of process groups created afterwards: alg ('stragglar' | 'stragglar_a2a' | 'ring' | 'rhd' |
    'direct' | 'rsag' | 'auto': the straggler-aware variant while a straggler is declared, else rsag or ring by
    size), straggler (physical rank; -1: the last rank, or nobody for 'auto'), path ('tma' | 'simt' | 'simta'),
    blocks, threads, tile_bytes, timeout_s, arena_bytes, staging_bytes, schedule_text, check_args (also
    STRAGGLAR_CHECK_ARGS=1: every AllReduce first compares through the Store what the ranks passed -- size, dtypes,
    symmetric offset or ordinary tensor -- and raises on a mismatch; a debugging aid, one Store round trip per call).  Lowering switches are read
    from the environment when a program is first built: STRAGGLAR_GATE, STRAGGLAR_COPY, STRAGGLAR_LANES,
    STRAGGLAR_LANE1_EIGHTHS."""
    _options.update(options)


def _create(store, rank, size, timeout):
    return _ext().create_backend(store, rank, size, timeout, dict(_options))


def register() -> None:
    """Register the backend name ``stragglar`` with torch.distributed
    (cf. the reference's self-registering "dummy" backend,
    implementation/custom_backend/include/dummy.hpp:106-111)."""
    global _registered
    if _registered:
        return
    import torch.distributed as dist
    dist.Backend.register_backend("stragglar", _create, devices=["cpu", "cuda"])
    _registered = True


def backend_of(device="cuda", group=None):
    """The stragglar Backend object serving ``device`` in ``group``."""
    import torch
    import torch.distributed as dist
    pg = group if group is not None else dist.distributed_c10d._get_default_group()
    return pg._get_backend(torch.device(device))


def set_straggler(rank: int, device="cuda", group=None) -> None:
    """Name the physical rank that is persistently late.  The schedule is
    re-labelled so that this rank plays logical rank n-1; no device remapping
    is needed (the reference swaps CUDA devices instead:
    implementation/custom_backend/dp.py:71-77).  Call it on every rank."""
    _ext().set_straggler(backend_of(device, group), rank)


def set_algorithm(alg: str, device="cuda", group=None) -> None:
    _ext().set_algorithm(backend_of(device, group), alg)


def get_straggler(device="cuda", group=None) -> int:
    return _ext().get_straggler(backend_of(device, group))


def get_algorithm(device="cuda", group=None) -> str:
    return _ext().get_algorithm(backend_of(device, group))


def algorithm_for(nbytes: int, device="cuda", group=None) -> str:
    """The algorithm an AllReduce of ``nbytes`` runs with: the configured one, or what ``"auto"`` picks --
    ``stragglar_a2a`` while a straggler is declared (``set_straggler(r)``, ``r >= 0``), otherwise the one-shot
    reduce-scatter + all-gather below 512 MiB and the ring above."""
    return _ext().algorithm_for(backend_of(device, group), int(nbytes))


def empty_symmetric(numel: int, dtype=None, device="cuda", group=None):
    """A 1-D tensor in the backend's symmetric heap.  Collective: every rank
    must call it with the same sizes in the same order.

    Collectives on such a tensor (or on equal slices of it) run in place: peers read and write the tensor itself.
    Every rank of a collective must then pass its tensor of the same allocation at the same offset; a rank that
    passes an ordinary tensor instead takes the staged path while its peers reach into its heap, and the result
    is wrong (or the collective times out).  The same holds the other way round."""
    import torch
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    dtype = dtype or torch.float32
    return _ext().alloc_symmetric(backend_of(dev, group), int(numel), dtype, dev.type == "cuda",
                                  dev.index if dev.type == "cuda" else -1)


def all_reduce_ex(tensor, average: bool = False, comm_dtype=None, group=None):
    """AllReduce with an explicit dtype on the wire; returns a Work.  For an ordinary CUDA tensor the casts to and
    from ``comm_dtype`` (and the division by world_size of ``average``) happen inside the one kernel that also copies
    the tensor into the peer-reachable staging area and back."""
    return _ext().allreduce_ex(backend_of(tensor.device, group), tensor, average, comm_dtype)


class HostStreamedAllReduce:
    """AllReduce of data that arrives from pinned host memory every step, with the host-to-device copy streamed
    through the collective: the tensor is cut into ``pieces``; piece k is reduced (in place, in a tensor of the
    symmetric heap) as soon as it has landed on the device while piece k+1 is still being copied on a stream of
    its own, so the collective -- and whatever holds the ranks back before it, e.g. a late rank -- hides behind
    the copy instead of following it.

        stream = sp.HostStreamedAllReduce(numel, dtype=torch.float32, device="cuda")   # collective: allocates
        out = stream(host_tensor, op=dist.ReduceOp.AVG)      # the device tensor that holds the result

    Everything is enqueued asynchronously; the caller's current stream is ordered after the last piece.
    """

    def __init__(self, numel: int, dtype=None, device="cuda", pieces: int = 8, group=None):
        import torch
        self.group = group
        self.out = empty_symmetric(numel, dtype=dtype, device=device, group=group)
        n = max(1, min(pieces, numel // 4096 or 1))
        step = -(-numel // n)
        step = -(-step // 64) * 64                      # pieces start on 256-byte boundaries
        self.bounds = [(b, min(b + step, numel)) for b in range(0, numel, step)]
        self.copy_stream = torch.cuda.Stream(self.out.device)
        self.events = [torch.cuda.Event() for _ in self.bounds]

    def __call__(self, host_tensor, op=None, before_collective=None):
        """``before_collective``: called once on the current stream before the first piece is reduced (a hook for
        whatever precedes the collective on this rank); the copies do not wait for it."""
        import torch
        import torch.distributed as dist
        op = dist.ReduceOp.SUM if op is None else op
        cur = torch.cuda.current_stream(self.out.device)
        self.copy_stream.wait_stream(cur)                # the previous result has been consumed
        if before_collective is not None:
            before_collective()
        for (b, e), ev in zip(self.bounds, self.events):
            with torch.cuda.stream(self.copy_stream):
                self.out[b:e].copy_(host_tensor[b:e], non_blocking=True)
                ev.record(self.copy_stream)
            cur.wait_event(ev)
            dist.all_reduce(self.out[b:e], op=op, group=self.group)
        return self.out


def check_status(device="cuda", group=None) -> int:
    """Wait for the communication stream and return the device status word
    (0 = ok; see ``stragglar_b200.compiler.status_string``)."""
    import torch
    return _ext().check_status(backend_of(device, group), torch.device(device).type == "cuda")


def check_guards(device="cuda", group=None) -> bool:
    """True while the canary bytes on both sides of this rank's data region (symmetric heap and staging area)
    are intact, i.e. no kernel or copy of the backend has written outside the region."""
    import torch
    return bool(_ext().check_guards(backend_of(device, group), torch.device(device).type == "cuda"))


def launches(device="cuda", group=None) -> int:
    """Number of this library's kernels the backend has launched so far."""
    return _ext().launches(backend_of(device, group))


def last_collective_ms(device="cuda", group=None) -> float:
    """Device time this rank spent inside its last collective kernel
    (arrival to exit, from %globaltimer stamps written by the kernel)."""
    a, b = _ext().last_trace(backend_of(device, group))
    return max(0.0, (b - a) / 1e6)


class StragglerMonitor:
    """Finds the persistent straggler at run time and re-labels the schedule.

    Call :meth:`step` once per training step on every rank (after the
    gradient AllReduces).  Every rank contributes the time it spent inside its
    last collective; the rank with the smallest time arrived last -- the rule of
    the reference's offline analysis (motivation/log_proc.ipynb), applied over
    a sliding window by :class:`stragglar_b200.detect.OnlineDetector`.  When a
    rank has been the straggler in ``threshold`` of the last ``window`` steps
    and differs from the current choice, ``set_straggler`` is applied on all
    ranks at the same step (every rank sees the same gathered times).  With
    ``alg="auto"`` the monitor also withdraws the declaration once no rank is
    the straggler in at least half of the window, which sends the group back
    to the straggler-free algorithms."""

    def __init__(self, window: int = 20, threshold: float = 0.8, device="cuda", group=None):
        import torch.distributed as dist
        from ..detect import OnlineDetector
        self.device, self.group = device, group
        self.detector = OnlineDetector(dist.get_world_size(group), window=window, threshold=threshold)
        self.changes = 0

    def step(self):
        import torch
        import torch.distributed as dist
        world = dist.get_world_size(self.group)
        mine = torch.tensor([last_collective_ms(self.device, self.group)], device=self.device)
        allv = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allv, mine, group=self.group)
        self.detector.update([float(v.item()) for v in allv])
        rec = self.detector.recommendation()
        raw = get_straggler(self.device, self.group)
        auto = get_algorithm(self.device, self.group) == "auto"
        # -1 is "the last rank" for the StragglAR algorithms and "nobody" for "auto"
        cur = raw if (auto or raw >= 0) else world - 1
        if rec is not None and rec != cur:
            set_straggler(rec, self.device, self.group)
            self.changes += 1
        elif auto and raw >= 0 and self.detector.no_straggler():
            set_straggler(-1, self.device, self.group)     # nobody is persistently late any more
            self.changes += 1
        return rec


# ------------------------------------------------------------------ DDP hooks
def fused_avg_hook(state, bucket):
    """DDP communication hook: AllReduce the gradient bucket with the division
    by world_size fused into the collective kernel (DDP's default path divides
    in a separate pass before the AllReduce; the reference divides the flat
    gradient after it, implementation/custom_backend/dp.py:59-60)."""
    import torch.distributed as dist
    group = state if state is not None else dist.group.WORLD
    buf = bucket.buffer()
    fut = dist.all_reduce(buf, op=dist.ReduceOp.AVG, group=group, async_op=True).get_future()
    return fut.then(lambda f: f.value()[0])


class SymmetricBucketHook:
    """DDP communication hook that reduces every gradient bucket in a buffer of the symmetric heap.

    DistributedDataParallel allocates its buckets itself, outside the heap that peers can reach, so a bucket handed
    to ``dist.all_reduce`` takes the staged path.  This hook keeps one symmetric buffer per bucket (allocated on the
    bucket's first use; a collective allocation, made in bucket order, which is the same on every rank), copies the
    bucket in, reduces in place with the fused average, and copies the result back: two local copies at memory speed
    around the fastest collective path.  The symmetric heap must hold all buckets (STRAGGLAR_ARENA_MB).

        ddp.register_comm_hook(None, sp.SymmetricBucketHook())
    """

    def __init__(self, group=None):
        self.group = group
        self._bufs = {}
        self.__name__ = self.__qualname__ = "symmetric_bucket_hook"   # DDP logs the hook's name

    def __call__(self, state, bucket):
        import torch.distributed as dist
        group = self.group if self.group is not None else (state if state is not None else dist.group.WORLD)
        buf = bucket.buffer()
        key = bucket.index()
        sym = self._bufs.get(key)
        if sym is None or sym.numel() != buf.numel() or sym.dtype != buf.dtype:
            # DDP rebuilds its buckets once after the first iteration: sizes change, on every rank alike
            sym = empty_symmetric(buf.numel(), dtype=buf.dtype, device=buf.device, group=group)
            self._bufs[key] = sym
        sym.copy_(buf)
        fut = dist.all_reduce(sym, op=dist.ReduceOp.AVG, group=group, async_op=True).get_future()

        def back(f):
            buf.copy_(sym)
            return buf
        return fut.then(back)


def bf16_fused_avg_hook(state, bucket):
    """DDP communication hook: gradients travel as bfloat16.  One kernel per bucket reads the fp32 bucket tile by
    tile, converts it to bfloat16 into the buffer the peers reach, reduces (fp32 accumulation, the division by
    world_size applied to the final sums) and writes every finished tile back to the bucket as fp32; there are no
    separate cast or copy launches."""
    import torch
    buf = bucket.buffer()
    work = all_reduce_ex(buf, average=True, comm_dtype=torch.bfloat16, group=state)
    return work.get_future().then(lambda f: f.value()[0])


register()
