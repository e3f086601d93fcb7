"""Schedule synthesizer for an even number of GPUs that is not a power of two.

``python -m stragglar_b200.synth.nonpow2 <n>`` prints the schedule in the text
format of the reference tool (stragglar/synthesizer_nonpow2.py:216-222,246-249).
Unlike the reference module, :func:`synthesize` is importable (no global ``n``,
cf. stragglar/synthesizer_nonpow2.py:196) and odd ``n`` is refused with a clear
error instead of an assertion deep in the matcher.

Round r (L = ceil(log2 n)): the straggler matching and the seeding move are the
same as in the power-of-two case.  The idle GPUs are then paired by a
maximum-weight matching on a graph whose edge weight is the number of useful
directions (1 or 2) between two GPUs:

* r < L: only edges from a GPU that holds something to an empty GPU with rank
  above 2(L-1);
* L <= r < n-1: an edge carries the *lowest* chunk one side has and the other
  lacks, and edges that would hand a GPU meeting the straggler within L-1
  rounds a chunk that is too new are pruned;
* r >= n-1: the *highest* such chunk is forwarded instead.
"""
from __future__ import annotations

import math
import sys
import time
from typing import List, Optional

import numpy as np

from ..schedule import (HoldState, Matching, OneWayMatching, Schedule, StragglerMatching,
                        TwoWayMatching, check_round_degrees)
from .matching import Edge, max_weight_matching


def _offer(st: HoldState, giver: int, taker: int, lowest: bool) -> Optional[int]:
    """Lowest (or highest) chunk ``giver`` holds and ``taker`` lacks."""
    diff = st.mask[giver] & ~st.mask[taker]
    if not diff:
        return None
    return (diff & -diff).bit_length() - 1 if lowest else diff.bit_length() - 1


def _usefulness(st: HoldState, a: int, b: int, lowest: bool) -> int:
    return (_offer(st, a, b, lowest) is not None) + (_offer(st, b, a, lowest) is not None)


def _edges(st: HoldState, idle: List[int], r: int) -> List[Edge]:
    n = st.n
    L = math.ceil(math.log2(n))
    edges: List[Edge] = []
    if r < L:
        for a in idle:
            if not st.mask[a]:
                continue
            for b in idle:
                if b != a and b > 2 * (L - 1) and not st.mask[b]:
                    edges.append((a, b, 1))
        return edges
    for i, a in enumerate(idle):
        for b in idle[i + 1:]:
            if r < n - 1:
                # a GPU d rounds before its own straggler matching may only be
                # handed chunks up to r + d - L
                da, db = a - r, b - r
                tb, ta = st.top(b), st.top(a)
                if tb is not None and 0 < da < L and tb > r + da - L:
                    continue
                if ta is not None and 0 < db < L and ta > r + db - L:
                    continue
            wgt = _usefulness(st, a, b, lowest=r < n - 1)
            if wgt:
                edges.append((a, b, wgt))
    return edges


def synthesize(n: int, on_round=None, use_networkx: bool = True) -> Schedule:
    """Build the StragglAR schedule for an even ``n`` that is not a power of 2."""
    if n < 6 or n & (n - 1) == 0:
        raise ValueError("n must not be a power of 2 (use synth.pow2)")
    if n % 2:
        raise ValueError("odd GPU counts are not supported: every round pairs up the idle GPUs")
    L = math.ceil(math.log2(n))
    st = HoldState(n)
    sched = Schedule(n)
    r = 0
    while not st.done():
        rnd: List[Matching] = []
        busy = set()
        if r < n - 1:
            m = StragglerMatching(r, n - 1, r)
            st.apply(m)
            rnd.append(m)
            busy |= {r, n - 1}
        if 0 < r < L:
            m = OneWayMatching(r - 1, r - 1 + L, r - 1)
            st.apply(m)
            rnd.append(m)
            busy |= {r - 1, r - 1 + L}
        idle = [g for g in range(n) if g not in busy]
        lowest = r < n - 1
        for a, b in max_weight_matching(idle, _edges(st, idle, r), use_networkx):
            ca, cb = _offer(st, a, b, lowest), _offer(st, b, a, lowest)
            if ca is not None and cb is not None:
                m = TwoWayMatching(a, b, ca, cb)
            elif ca is not None:
                m = OneWayMatching(a, b, ca)
            elif cb is not None:
                m = OneWayMatching(b, a, cb)
            else:
                continue
            st.apply(m)
            rnd.append(m)
        check_round_degrees([m for m in rnd if not isinstance(m, StragglerMatching)])
        sched.rounds.append(rnd)
        if on_round is not None:
            on_round(r, rnd, st)
        r += 1
        if r > 4 * n + 8:
            raise RuntimeError("synthesizer does not converge")
    return sched


def main(argv=None) -> int:
    argv = sys.argv if argv is None else argv
    if len(argv) != 2:
        print("Usage: python synthesizer_nonpow2.py <n>")
        return 1
    n = int(argv[1])
    assert n > 0, "n must be positive"
    assert n & (n - 1) != 0, "n must not be a power of 2"

    def show(r, rnd, st):
        print("Round", r, flush=True)
        print(len(rnd), [str(m) for m in rnd], flush=True)
        for g in range(n):
            print("GPU", g, "chunks", st.as_array(g), flush=True)
        print("Active chunks", st.active_chunks(), flush=True)
        print("-" * 46, flush=True)

    t0 = time.time()
    sched = synthesize(n, on_round=show)
    print("Time taken:", time.time() - t0)
    print("Actual number of rounds", len(sched))
    print("Optimal number of rounds", n - 2 + math.ceil(np.log2(n)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
