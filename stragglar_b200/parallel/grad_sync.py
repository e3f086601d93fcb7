"""Gradient synchronisation without the DistributedDataParallel wrapper.

The reference's training scripts average gradients by hand:
``flat`` -- flatten all gradients into one buffer, one all_reduce, divide, copy
back (implementation/custom_backend/dp.py:28-65); ``per_param`` -- one
all_reduce and one division per parameter (motivation/dp_llama.py:109-117).
Both are offered here for comparison runs.  On the ``stragglar`` backend the
division is fused into the collective (ReduceOp.AVG), the flat buffer can live
in the backend's symmetric heap (no staging), and nothing is dropped when the
element count is not a multiple of n-1 (the reference's unpadded flat buffer
loses the last ``numel mod 7`` gradient elements, dp.py:32-33).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _grads(model) -> List[torch.Tensor]:
    return [p.grad for p in model.parameters() if p.requires_grad and p.grad is not None]


class FlatGradSync:
    """One AllReduce per step over a persistent flat buffer."""

    def __init__(self, model, group=None, symmetric: bool = True):
        self.model, self.group = model, group
        params = [p for p in model.parameters() if p.requires_grad]
        self.numel = sum(p.numel() for p in params)
        first = params[0]
        self.buffer: Optional[torch.Tensor] = None
        if symmetric and dist.get_backend(group) == "stragglar":
            from . import empty_symmetric
            try:
                self.buffer = empty_symmetric(self.numel, dtype=first.dtype, device=first.device, group=group)
            except RuntimeError as e:   # heap too small (STRAGGLAR_ARENA_MB): an ordinary tensor is staged instead
                import warnings
                warnings.warn(f"flat gradient buffer not placed in the symmetric heap: {e}")
        if self.buffer is None:
            self.buffer = torch.empty(self.numel, dtype=first.dtype, device=first.device)

    def __call__(self) -> None:
        grads = _grads(self.model)
        if not grads:
            return
        off = 0
        for g in grads:
            self.buffer[off:off + g.numel()].copy_(g.reshape(-1))
            off += g.numel()
        flat = self.buffer[:off]
        if dist.get_backend(self.group) in ("stragglar", "nccl"):
            dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=self.group)
        else:
            dist.all_reduce(flat, group=self.group)
            flat /= dist.get_world_size(self.group)
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()


def allreduce_gradients_per_param(model, group=None, nvtx: bool = False) -> int:
    """One AllReduce per parameter; returns the bytes reduced.  ``nvtx``: an ``allreduce:<parameter name>`` range
    around every call, as the reference's script has (motivation/dp_llama.py:109-114)."""
    total = 0
    world = dist.get_world_size(group)
    named = [(n, p.grad) for n, p in model.named_parameters() if p.requires_grad and p.grad is not None]
    for name, g in named:
        if nvtx and g.is_cuda:
            torch.cuda.nvtx.range_push(f"allreduce:{name}")
        if dist.get_backend(group) in ("stragglar", "nccl"):
            dist.all_reduce(g, op=dist.ReduceOp.AVG, group=group)
        else:
            dist.all_reduce(g, group=group)
            g /= world
        if nvtx and g.is_cuda:
            torch.cuda.nvtx.range_pop()
        total += g.numel() * g.element_size()
    return total
