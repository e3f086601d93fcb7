"""The per-step training log line of the reference scripts
(implementation/custom_backend/dp.py:283, motivation/dp_llama.py:137):

    Rank r | Step s | Forward Time: f ms | Backward Time: b ms  | Loss: l | Iteration Time: i ms | AR Time: a ms | AR Buffer Size: k KB

``format_step`` writes it, ``parse_step`` reads it back; stragglar_b200.detect
uses the same pattern on whole log files.
"""
from __future__ import annotations

import re
from typing import Dict, Optional

RANK_COLORS = ["\033[91m", "\033[92m", "\033[93m", "\033[94m", "\033[95m", "\033[96m"]
RESET = "\033[0m"

_PAT = re.compile(r"Rank (\d+) \| Step (\d+) \| Forward Time: ([\d.]+) ms \| Backward Time: ([\d.]+) ms\s+\| "
                  r"Loss: ([-\d.naninf]+) \| Iteration Time: ([\d.]+) ms \| AR Time: ([\d.]+) ms \| "
                  r"AR Buffer Size: ([\d.]+) KB")


def format_step(rank: int, step: int, forward_ms: float, backward_ms: float, loss: float, iteration_ms: float,
                ar_ms: float, ar_bytes: int, color: bool = True) -> str:
    body = (f"Rank {rank} | Step {step} | Forward Time: {forward_ms:.2f} ms | Backward Time: {backward_ms:.2f} ms  | "
            f"Loss: {loss:.4f} | Iteration Time: {iteration_ms:.2f} ms | AR Time: {ar_ms:.2f} ms | "
            f"AR Buffer Size: {ar_bytes / 1024:.2f} KB")
    return f"{RANK_COLORS[rank % len(RANK_COLORS)]}{body}{RESET}" if color else body


def parse_step(line: str) -> Optional[Dict[str, float]]:
    m = _PAT.search(line)
    if not m:
        return None
    keys = ("rank", "step", "forward_ms", "backward_ms", "loss", "iteration_ms", "ar_ms", "ar_kb")
    vals = m.groups()
    return {k: (int(v) if k in ("rank", "step") else float(v)) for k, v in zip(keys, vals)}
