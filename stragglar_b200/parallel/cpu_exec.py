"""Run a compiled collective over plain ``torch.distributed`` send/recv
(gloo for CPU tensors, NCCL for CUDA tensors).

Every rank is a process with its own buffer; nothing is shared.  The op tables
are pull based (the executing rank reads its peers), so each round is lowered
to messages: the peers an op reads send their part of the chunk, the executor
adds and stores, and a straggler matching sends the sum back.  Rounds are
executed one after the other, as in the reference's hand-written
ncclSend/ncclRecv schedules (stragglar/allreduce_4GPU.cu:299-368), which makes
this executor the message-passing oracle for the schedule compiler and the
CPU configuration of the benchmarks (4 ranks, 1 Mi fp32 elements, one rank
5 ms late, checked against an fp64 sum).  On CUDA tensors with the NCCL
backend it is the baseline "what the reference's approach costs": the same
tables executed as grouped ncclSend/ncclRecv plus separate add kernels, for
any rank count (the reference has such code for 4 and 8 GPUs only).
"""
from __future__ import annotations

import time
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..compiler import COPY, F_LOCAL, F_SCALE, PUSH, REDUCE_PUSH, Program, Table


def _chunk_bounds(count: int, esize: int, num_chunks: int) -> List[Tuple[int, int]]:
    vw = max(1, 16 // esize)
    nvec = count // vw
    q, rem = divmod(nvec, num_chunks)
    out = []
    for c in range(num_chunks):
        b = (q * c + min(c, rem)) * vw
        e = (q * (c + 1) + min(c + 1, rem)) * vw if c < num_chunks - 1 else count
        out.append((b, e))
    return out


def _op_range(bounds, op, tile_elems: int) -> Tuple[int, int]:
    """Element range an op covers: part ``part`` of ``parts`` of the chunk's tiles."""
    b, e = bounds[int(op["chunk"])]
    tiles = -(-(e - b) // tile_elems)
    part, parts = int(op["part"]), int(op["parts"])
    t0, t1 = tiles * part // parts, tiles * (part + 1) // parts
    return min(e, b + t0 * tile_elems), min(e, b + t1 * tile_elems)


class SendRecvExecutor:
    """Executes :class:`Program` objects on the default (or a given) process
    group with point-to-point messages."""

    def __init__(self, group=None, tile_elems: int = 4096):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.tile_elems = tile_elems
        self.rounds_executed = 0

    def _exchange(self, ops: List) -> None:
        if not ops:
            return
        for req in dist.batch_isend_irecv(ops):
            req.wait()

    def _run_table(self, t: Table, buf: torch.Tensor, scale: float) -> None:
        me = self.rank
        if not t.takes_part(me):
            return
        bounds = _chunk_bounds(buf.numel(), buf.element_size(), t.num_chunks)
        rounds = sorted({int(o["round"]) for r in t.ranks for o in r.ops})
        for rnd in rounds:
            # every rank walks (executor, op) in the same order, so the messages between a pair
            # of ranks are issued in the same order on both sides (NCCL matches by order, not tag)
            first: List = []
            recv_bufs: Dict[Tuple[int, int], torch.Tensor] = {}
            mine = []
            landed: List = []
            per_rank_ops = [[o for o in t.ranks[ex].ops if int(o["round"]) == rnd] for ex in range(self.world)]
            for ex in range(self.world):
                for k, op in enumerate(per_rank_ops[ex]):
                    lo, hi = _op_range(bounds, op, self.tile_elems)
                    if hi <= lo:
                        continue
                    if int(op["kind"]) == PUSH:
                        # a copy executed by its source: one message from the executor to every destination
                        for q in range(int(op["nsrc"])):
                            dst = int(op["src"][q])
                            if ex == me:
                                first.append(dist.P2POp(dist.isend, buf[lo:hi].clone(), dst, self.group))
                            elif dst == me:
                                rb = torch.empty(hi - lo, dtype=buf.dtype, device=buf.device)
                                first.append(dist.P2POp(dist.irecv, rb, ex, self.group))
                                landed.append((rb, lo, hi))
                        continue
                    for q in range(int(op["nsrc"])):
                        src = int(op["src"][q])
                        if ex == me:
                            rb = torch.empty(hi - lo, dtype=buf.dtype, device=buf.device)
                            recv_bufs[(k, q)] = rb
                            first.append(dist.P2POp(dist.irecv, rb, src, self.group))
                        elif src == me:
                            first.append(dist.P2POp(dist.isend, buf[lo:hi].clone(), ex, self.group))
                    if ex == me:
                        mine.append((k, op, lo, hi))
            self._exchange(first)
            for rb, lo, hi in landed:      # chunks that peers pushed into this rank's slots
                buf[lo:hi] = rb
            second: List = []
            for ex in range(self.world):
                for k, op in enumerate(per_rank_ops[ex]):
                    kind = int(op["kind"])
                    lo, hi = _op_range(bounds, op, self.tile_elems)
                    if hi <= lo:
                        continue
                    if kind == PUSH:
                        continue
                    if ex == me:
                        flags = int(op["flags"])
                        if kind == COPY:
                            buf[lo:hi] = recv_bufs[(k, 0)]
                            continue
                        acc = buf[lo:hi].float() if (kind == REDUCE_PUSH or flags & F_LOCAL) else torch.zeros(
                            hi - lo, device=buf.device)
                        for q in range(int(op["nsrc"])):
                            acc = acc + recv_bufs[(k, q)].float()
                        if flags & F_SCALE:
                            acc = acc * scale
                        buf[lo:hi] = acc.to(buf.dtype)
                        if kind == REDUCE_PUSH:
                            second.append(dist.P2POp(dist.isend, buf[lo:hi].clone(), int(op["src"][0]), self.group))
                    elif kind == REDUCE_PUSH and int(op["src"][0]) == me:
                        # the sum of a straggler matching executed by a peer comes back into this rank's slot
                        second.append(dist.P2POp(dist.irecv, buf[lo:hi], ex, self.group))
            self._exchange(second)
            self.rounds_executed += 1

    def all_reduce(self, program: Program, buf: torch.Tensor, scale: float = 1.0, delay_s: float = 0.0) -> torch.Tensor:
        """In-place collective on a contiguous 1-D tensor.  ``delay_s`` makes
        this rank late (an injected straggler delay on the host)."""
        if program.n != self.world:
            raise ValueError(f"program is for {program.n} ranks, group has {self.world}")
        if not (buf.dim() == 1 and buf.is_contiguous()):
            raise ValueError("a contiguous 1-D tensor is expected")
        if delay_s > 0:
            time.sleep(delay_s)
        for t in program.phases:
            self._run_table(t, buf, scale)
        return buf


GlooExecutor = SendRecvExecutor
