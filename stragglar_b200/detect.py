"""Find the persistent straggler from per-rank AllReduce times.

In synchronous data-parallel training the GPU that arrives last at the
gradient AllReduce waits least inside it, so the rank with the *smallest*
AllReduce time in a step is that step's straggler, and the gap to the
second-smallest time is the straggler's delay.  This is the analysis of the
reference notebook (motivation/log_proc.ipynb, cells 2-4) as a library and a
command line tool:

    python -m stragglar_b200.detect train.log [--skip 1]

It reads lines of the form written by the training scripts
(``Rank r | Step s | ... | AR Time: t ms | ...``; several records glued on one
line are split first, as the notebook does).  :class:`OnlineDetector` applies
the same rule to a stream of per-step arrival measurements and recommends
when to re-label the straggler.
"""
from __future__ import annotations

import argparse
import re
import sys
from collections import Counter, defaultdict
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

_LINE = re.compile(r"Rank (\d+) \| Step (\d+) .*? AR Time: ([\d.]+) ms")


def split_glued(lines: Iterable[str]) -> List[str]:
    """Put every ``Rank ...`` record on a line of its own."""
    out: List[str] = []
    for line in lines:
        if line.count("Rank") > 1:
            out.extend("Rank " + part.strip() + "\n" for part in line.split("Rank")[1:])
        else:
            out.append(line)
    return out


def parse_ar_times(lines: Iterable[str]) -> Dict[int, Dict[int, float]]:
    """step -> rank -> AllReduce time in ms."""
    table: Dict[int, Dict[int, float]] = defaultdict(dict)
    for line in split_glued(lines):
        m = _LINE.search(line)
        if m:
            table[int(m.group(2))][int(m.group(1))] = float(m.group(3))
    return dict(sorted(table.items()))


@dataclass
class StragglerReport:
    straggler: Optional[int]
    share: Dict[int, float]            # rank -> % of steps in which it had the smallest AR time
    delays_ms: List[float]             # per step: second-smallest minus smallest AR time
    steps: int

    @property
    def mean_delay_ms(self) -> float:
        return sum(self.delays_ms) / len(self.delays_ms) if self.delays_ms else 0.0

    @property
    def median_delay_ms(self) -> float:
        if not self.delays_ms:
            return 0.0
        s = sorted(self.delays_ms)
        k = len(s) // 2
        return s[k] if len(s) % 2 else 0.5 * (s[k - 1] + s[k])

    @property
    def max_delay_ms(self) -> float:
        return max(self.delays_ms, default=0.0)

    def cdf(self) -> List[Tuple[float, float]]:
        s = sorted(self.delays_ms)
        return [(d, (i + 1) / len(s)) for i, d in enumerate(s)]


def analyse(table: Dict[int, Dict[int, float]], skip_delay_steps: int = 1) -> StragglerReport:
    """``share`` counts every step (as the notebook does); ``delays_ms`` leaves
    out the first ``skip_delay_steps`` steps, which contain start-up cost."""
    wins: Counter = Counter()
    delays: List[float] = []
    steps = 0
    for i, (step, per_rank) in enumerate(table.items()):
        if len(per_rank) < 2:
            continue
        steps += 1
        order = sorted(per_rank.items(), key=lambda kv: (kv[1], kv[0]))
        wins[order[0][0]] += 1
        if i >= skip_delay_steps:
            delays.append(order[1][1] - order[0][1])
    share = {r: 100.0 * c / steps for r, c in wins.most_common()} if steps else {}
    straggler = wins.most_common(1)[0][0] if wins else None
    return StragglerReport(straggler, share, delays, steps)


class OnlineDetector:
    """Sliding-window version: feed per-step AllReduce times (or arrival
    stamps with ``arrival=True``, where the *largest* value is the last to
    arrive); :meth:`recommendation` names a rank once it was the straggler in
    at least ``threshold`` of the last ``window`` steps."""

    def __init__(self, world_size: int, window: int = 20, threshold: float = 0.8, arrival: bool = False):
        self.world_size, self.window, self.threshold, self.arrival = world_size, window, threshold, arrival
        self.history: List[int] = []

    def update(self, per_rank: Sequence[float]) -> int:
        if len(per_rank) != self.world_size:
            raise ValueError("one value per rank expected")
        pick = max if self.arrival else min
        r = pick(range(self.world_size), key=lambda i: (per_rank[i], -i if self.arrival else i))
        self.history.append(r)
        del self.history[:-self.window]
        return r

    def recommendation(self) -> Optional[int]:
        if len(self.history) < self.window:
            return None
        r, c = Counter(self.history).most_common(1)[0]
        return r if c >= self.threshold * len(self.history) else None

    def no_straggler(self, release: float = 0.5) -> bool:
        """True once the window is full and no rank was the straggler in ``release`` of it: the last-to-arrive
        rank keeps changing, i.e. nobody is persistently late.  (Lower than ``threshold`` on purpose: between the
        two fractions the current choice stands.)"""
        if len(self.history) < self.window:
            return False
        return Counter(self.history).most_common(1)[0][1] < release * len(self.history)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="find the persistent straggler in a training log")
    ap.add_argument("log")
    ap.add_argument("--skip", type=int, default=1, help="steps left out of the delay statistics")
    ap.add_argument("--cdf", metavar="FILE", help="write the empirical CDF of the straggler delay (delay_ms,fraction) "
                                                  "as CSV; FILE.png is drawn too when matplotlib is installed")
    args = ap.parse_args(argv)
    with open(args.log) as f:
        rep = analyse(parse_ar_times(f), args.skip)
    print("Percentage of time each rank has the smallest number:")
    for r, pct in rep.share.items():
        print(f"Rank {r}    {pct:.1f}")
    print(f"straggler: rank {rep.straggler}; delay mean {rep.mean_delay_ms:.1f} ms, "
          f"median {rep.median_delay_ms:.1f} ms, max {rep.max_delay_ms:.1f} ms over {len(rep.delays_ms)} steps")
    if args.cdf:
        pts = rep.cdf()
        with open(args.cdf, "w") as f:
            f.write("delay_ms,fraction\n")
            for x, y in pts:
                f.write(f"{x:.4f},{y:.6f}\n")
        try:   # the plot of the reference's notebook (motivation/log_proc.ipynb, last cell)
            import matplotlib
            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
            plt.figure(figsize=(5, 3.2))
            plt.step([p[0] for p in pts], [p[1] for p in pts], where="post")
            plt.xlabel("straggler delay (ms)"); plt.ylabel("CDF"); plt.grid(alpha=0.3); plt.tight_layout()
            plt.savefig(args.cdf + ".png", dpi=150)
        except ImportError:
            pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
