"""Schedule synthesizer for a power-of-two number of GPUs.

``python -m stragglar_b200.synth.pow2 <n>`` prints the schedule in the text
format of the reference tool (stragglar/synthesizer_pow2.py:241-247,272-275)
and produces the same rounds for every n the reference handles (n >= 8).  It
also handles n = 2 and n = 4, where the reference aborts because no GPU is
idle in some round (stragglar/synthesizer_pow2.py:137).

How a round r is built (n GPUs, L = log2 n, straggler = rank n-1, chunk i is
"finished" once rank i has added its partial to the straggler's):

1. r < n-1: rank r and the straggler reduce chunk r.
2. 0 < r < L: rank r-1 seeds rank r-1+L with chunk r-1, so that high ranks
   start collecting early.
3. The GPUs that are still idle are paired greedily and each pair forwards
   the newest chunk of each side that the other side lacks.  The pairing
   works on the "window" of the L most recently finished chunks: holders of
   the oldest chunk in the window are paired with holders of the younger
   ones, except that GPUs about to meet the straggler in the next L-1 rounds
   are served first with the oldest chunk they miss.
"""
from __future__ import annotations

import math
import sys
import time
from typing import Dict, List, Sequence, Tuple

import numpy as np

from ..schedule import (HoldState, Matching, OneWayMatching, Schedule, StragglerMatching,
                        TwoWayMatching, check_round_degrees)


def _window_holders(st: HoldState, r: int, L: int) -> Dict[int, List[int]]:
    """chunk -> ranks (ascending) that hold it, for the chunks of the window
    that ends at round r.  Before round n-1 the straggler and rank r (busy with
    each other) are left out; from round n-1 on the straggler is free and is
    listed as a holder of the last chunk only, since that is all it still has
    to hand out."""
    n = st.n
    lo, hi = min(r - L, n - 2), min(r, n - 1)
    holders: Dict[int, List[int]] = {c: [] for c in range(lo, hi)}
    for g in range(n):
        if r < n - 1 and g in (n - 1, r):
            continue
        if r >= n - 1 and g == n - 1:
            holders[n - 2].append(g)
            continue
        for c in range(lo, hi):
            if st.holds(g, c):
                holders[c].append(g)
    return holders


def _zip_oldest_with_rest(holders: Dict[int, List[int]], hi: int) -> List[Tuple[int, int]]:
    oldest = min(holders)
    givers = holders[oldest]
    takers: List[int] = []
    for c in range(oldest + 1, hi):
        takers.extend(holders.get(c, ()))
    if set(givers) & set(takers):
        raise AssertionError("a GPU appears on both sides of the pairing")
    if len(givers) != len(takers):
        raise AssertionError("pairing sides differ in length")
    return list(zip(givers, takers))


def _pair_idle(st: HoldState, idle: Sequence[int], r: int) -> List[Tuple[int, int]]:
    n = st.n
    L = math.ceil(math.log2(n))
    if not idle:
        return []  # n = 2, n = 4: a round where everybody is already busy
    if len(idle) % 2:
        raise AssertionError("odd number of idle GPUs")
    if r < L:
        # start-up: every idle GPU that holds something feeds one that holds
        # nothing among the ranks above 2(L-1)
        givers = [g for g in idle if st.mask[g]]
        takers = [g for g in idle if g > 2 * (L - 1) and not st.mask[g]]
        return list(zip(givers, takers))
    holders = _window_holders(st, r, L)
    if r >= n - 1:
        return _zip_oldest_with_rest(holders, min(r, n - 1))
    pairs: List[Tuple[int, int]] = []
    soon = range(r + 1, min(r + L, n - 1))  # next partners of the straggler
    for g in soon:
        for c in range(r - L, r):
            if st.holds(g, c):
                holders[c].remove(g)
                if not holders[c]:
                    del holders[c]
                break
    for g in soon:
        for c in range(r - L, r):
            if not st.holds(g, c):
                partner = holders[c].pop(0)
                if not holders[c]:
                    del holders[c]
                pairs.append((g, partner))
                break
    pairs.extend(_zip_oldest_with_rest(holders, r))
    return pairs


def _forwarding(st: HoldState, a: int, b: int):
    """What a pair forwards: each side offers its newest chunk; a side sends
    only if the other lacks that chunk."""
    ca, cb = st.top(a), st.top(b)
    a_gives = ca is not None and not st.holds(b, ca)
    b_gives = cb is not None and not st.holds(a, cb)
    if ca is None or cb is None:
        # the side with nothing cannot give; the other one gives its newest
        a_gives, b_gives = ca is not None, cb is not None
    if a_gives and b_gives:
        return TwoWayMatching(a, b, ca, cb)
    if a_gives:
        return OneWayMatching(a, b, ca)
    if b_gives:
        return OneWayMatching(b, a, cb)
    return None


def synthesize(n: int, on_round=None) -> Schedule:
    """Build the StragglAR schedule for a power-of-two ``n`` (n >= 2).
    ``on_round(r, matchings, state)`` is called after each round."""
    if n < 2 or n & (n - 1):
        raise ValueError("n must be a power of 2 and at least 2")
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
        for a, b in _pair_idle(st, idle, r):
            m = _forwarding(st, a, b)
            if m is not None:
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
        print("Usage: python synthesizer_pow2.py <n>")
        return 1
    n = int(argv[1])
    assert n > 0, "n must be positive"
    assert n & (n - 1) == 0, "n must be a power of 2"
    t0 = time.time()
    if n == 1:
        sched = Schedule(1)
    else:
        def show(r, rnd, st):
            print("Round", r, flush=True)
            print(len(rnd), [str(m) for m in rnd], flush=True)
            for g in range(n):
                print("GPU", g, "chunks", st.as_array(g), flush=True)
            print("Active chunks", st.active_chunks(), flush=True)
            print("-" * 46, flush=True)
        sched = synthesize(n, on_round=show)
    print("Time taken:", time.time() - t0)
    print("Actual number of rounds", len(sched))
    print("Optimal number of rounds", n - 2 + np.log2(n))
    return 0


if __name__ == "__main__":
    sys.exit(main())
