"""Schedule IR for straggler-aware AllReduce.

A schedule is a list of rounds; a round is a list of matchings between GPUs.
The buffer is cut into ``n - 1`` chunks.  A GPU "holds" chunk ``c`` once it
owns the fully reduced value of that chunk.  Three matching kinds exist, with
the same meaning and the same printed form as the reference synthesizers
(stragglar/synthesizer_pow2.py:45-84):

* ``StragglerMatching(rank, straggler, chunk)`` -- both sides exchange their
  partial value of ``chunk`` and add; both hold it afterwards.
* ``OneWayMatching(src, dst, chunk)`` -- ``src`` forwards a finished chunk.
* ``TwoWayMatching(a, b, chunk_a, chunk_b)`` -- ``a`` forwards ``chunk_a`` to
  ``b`` while ``b`` forwards ``chunk_b`` to ``a``.

Unlike the reference classes, these are immutable records: holding state is
tracked separately in :class:`HoldState`, so a schedule can be replayed,
validated, permuted and re-printed any number of times.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple, Union

import numpy as np

RULE = "-" * 46


@dataclass(frozen=True)
class StragglerMatching:
    rank: int
    straggler: int
    chunk: int

    def __str__(self) -> str:
        return f"StragglerMatching: {self.rank} <-> {self.straggler}, chunk_id: {self.chunk}"

    def moves(self) -> Tuple[Tuple[int, int, int], ...]:
        return ((self.rank, self.straggler, self.chunk), (self.straggler, self.rank, self.chunk))


@dataclass(frozen=True)
class OneWayMatching:
    src: int
    dst: int
    chunk: int

    def __str__(self) -> str:
        return f"OneWayMatching: {self.src} -> {self.dst}, chunk_id: {self.chunk}"

    def moves(self) -> Tuple[Tuple[int, int, int], ...]:
        return ((self.src, self.dst, self.chunk),)


@dataclass(frozen=True)
class TwoWayMatching:
    a: int
    b: int
    chunk_a: int
    chunk_b: int

    def __str__(self) -> str:
        return (f"TwoWayMatching: {self.a} -> {self.b}, chunk_id: {self.chunk_a}; "
                f"{self.b} -> {self.a}, chunk_id: {self.chunk_b}")

    def moves(self) -> Tuple[Tuple[int, int, int], ...]:
        return ((self.a, self.b, self.chunk_a), (self.b, self.a, self.chunk_b))


Matching = Union[StragglerMatching, OneWayMatching, TwoWayMatching]


class ScheduleError(ValueError):
    """A schedule breaks one of the structural rules."""


class HoldState:
    """Which finished chunks every GPU holds; one bitmask per GPU."""

    def __init__(self, n: int):
        self.n = n
        self.mask: List[int] = [0] * n

    @property
    def full(self) -> int:
        return (1 << (self.n - 1)) - 1

    def holds(self, gpu: int, chunk: int) -> bool:
        return bool(self.mask[gpu] >> chunk & 1)

    def count(self, gpu: int) -> int:
        return bin(self.mask[gpu]).count("1")

    def top(self, gpu: int):
        m = self.mask[gpu]
        return m.bit_length() - 1 if m else None

    def done(self) -> bool:
        return all(m == self.full for m in self.mask)

    def apply(self, m: Matching, check: bool = True) -> None:
        if isinstance(m, StragglerMatching):
            self.mask[m.rank] |= 1 << m.chunk
            self.mask[m.straggler] |= 1 << m.chunk
            return
        for src, dst, chunk in m.moves():
            if check and not self.holds(src, chunk):
                raise ScheduleError(f"{m}: GPU {src} forwards chunk {chunk} before holding it")
        for src, dst, chunk in m.moves():
            self.mask[dst] |= 1 << chunk

    def as_array(self, gpu: int) -> np.ndarray:
        return np.array([float(self.mask[gpu] >> c & 1) for c in range(self.n - 1)])

    def active_chunks(self) -> Dict[int, int]:
        """Chunks the straggler holds that some GPU still lacks -> number of
        non-straggler holders (the ``Active chunks`` line of the printout)."""
        out: Dict[int, int] = {}
        for c in range(self.n - 1):
            if not self.holds(self.n - 1, c):
                continue
            if all(self.holds(g, c) for g in range(self.n)):
                continue
            out[c] = sum(1 for g in range(self.n - 1) if self.holds(g, c))
        return out


def check_round_degrees(rnd: Sequence[Matching]) -> None:
    """Every GPU sends at most one and receives at most one chunk per round
    among the forwarding matchings (the rule of ``valid_round``,
    stragglar/synthesizer_pow2.py:86-103), and -- stricter than the reference --
    the two sides of a StragglerMatching are counted as well."""
    senders, receivers = set(), set()
    for m in rnd:
        for src, dst, _ in m.moves():
            if src in senders:
                raise ScheduleError(f"GPU {src} sends twice in one round ({m})")
            if dst in receivers:
                raise ScheduleError(f"GPU {dst} receives twice in one round ({m})")
            senders.add(src)
            receivers.add(dst)


@dataclass
class Schedule:
    n: int
    rounds: List[List[Matching]] = field(default_factory=list)

    # ------------------------------------------------------------------ facts
    @property
    def straggler(self) -> int:
        return self.n - 1

    @property
    def num_chunks(self) -> int:
        return self.n - 1

    def __len__(self) -> int:
        return len(self.rounds)

    def optimal_rounds(self) -> int:
        return self.n - 2 + math.ceil(math.log2(self.n)) if self.n > 1 else 0

    def chunks_sent_by(self, gpu: int) -> int:
        return sum(1 for rnd in self.rounds for m in rnd for s, _, _ in m.moves() if s == gpu)

    # ------------------------------------------------------------- validation
    def validate(self) -> "Schedule":
        """Replay on chunk bitmaps and check every structural rule: ranks and
        chunks in range, per-round send/receive degree <= 1, forwards only of
        held chunks, no transfer of a chunk the receiver already holds,
        StragglerMatching i pairs rank i with rank n-1 on chunk i exactly once,
        and everybody holds everything at the end."""
        n = self.n
        if n < 2:
            if self.rounds:
                raise ScheduleError("a 1-GPU schedule has no rounds")
            return self
        st = HoldState(n)
        seen_straggler = set()
        for r, rnd in enumerate(self.rounds):
            for m in rnd:
                for src, dst, chunk in m.moves():
                    if not (0 <= src < n and 0 <= dst < n and src != dst):
                        raise ScheduleError(f"round {r}: bad ranks in {m}")
                    if not 0 <= chunk < n - 1:
                        raise ScheduleError(f"round {r}: bad chunk in {m}")
                if isinstance(m, StragglerMatching):
                    if m.straggler != n - 1 or m.rank == n - 1:
                        raise ScheduleError(f"round {r}: {m} does not involve rank {n - 1}")
                    if m.chunk != m.rank:
                        raise ScheduleError(f"round {r}: {m} must reduce the rank's own chunk")
                    if m.chunk in seen_straggler:
                        raise ScheduleError(f"round {r}: chunk {m.chunk} reduced twice")
                    seen_straggler.add(m.chunk)
                else:
                    for src, dst, chunk in m.moves():
                        if st.holds(dst, chunk):
                            raise ScheduleError(f"round {r}: {m} re-sends chunk {chunk} to GPU {dst}")
            check_round_degrees(rnd)
            # forwards read the state *before* the round: apply after checking all
            snapshot = list(st.mask)
            for m in rnd:
                if not isinstance(m, StragglerMatching):
                    for src, _, chunk in m.moves():
                        if not snapshot[src] >> chunk & 1:
                            raise ScheduleError(
                                f"round {r}: {m}: GPU {src} does not hold chunk {chunk} yet")
            for m in rnd:
                st.apply(m, check=False)
        if not st.done():
            lacking = [g for g in range(n) if st.mask[g] != st.full]
            raise ScheduleError(f"GPUs {lacking} miss chunks after the last round")
        return self

    # -------------------------------------------------------------- printing
    def format(self, footer: bool = True, optimal_as_float: bool = None) -> str:
        """The text the reference synthesizers print (without the wall-clock
        ``Time taken`` line): per round the matchings, every GPU's chunk bitmap
        after the round, the active chunks and a 46-dash rule; then the two
        round-count lines (stragglar/synthesizer_pow2.py:241-247,272-275)."""
        n = self.n
        st = HoldState(n)
        out: List[str] = []
        for r, rnd in enumerate(self.rounds):
            for m in rnd:
                st.apply(m, check=False)
            out.append(f"Round {r}")
            out.append(f"{len(rnd)} {[str(m) for m in rnd]}")
            for g in range(n):
                out.append(f"GPU {g} chunks {st.as_array(g)}")
            out.append(f"Active chunks {st.active_chunks()}")
            out.append(RULE)
        if footer:
            pow2 = n & (n - 1) == 0
            if optimal_as_float is None:
                optimal_as_float = pow2
            out.append(f"Actual number of rounds {len(self.rounds)}")
            if optimal_as_float:
                out.append(f"Optimal number of rounds {n - 2 + np.log2(n)}")
            else:
                out.append(f"Optimal number of rounds {n - 2 + math.ceil(np.log2(n))}")
        return "\n".join(out) + "\n"

    def compact(self) -> str:
        """One line per round, e.g. ``R3: 3<->7 c3 | 4->0 c1;0->4 c0``."""
        lines = []
        for r, rnd in enumerate(self.rounds):
            parts = []
            for m in rnd:
                if isinstance(m, StragglerMatching):
                    parts.append(f"{m.rank}<->{m.straggler} c{m.chunk}")
                elif isinstance(m, OneWayMatching):
                    parts.append(f"{m.src}->{m.dst} c{m.chunk}")
                else:
                    parts.append(f"{m.a}->{m.b} c{m.chunk_a};{m.b}->{m.a} c{m.chunk_b}")
            lines.append(f"R{r}: " + " | ".join(parts))
        return "\n".join(lines)

    # --------------------------------------------------------------- parsing
    _RE_S = re.compile(r"StragglerMatching: (\d+) <-> (\d+), chunk_id: (\d+)")
    _RE_1 = re.compile(r"OneWayMatching: (\d+) -> (\d+), chunk_id: (\d+)")
    _RE_2 = re.compile(r"TwoWayMatching: (\d+) -> (\d+), chunk_id: (\d+); (\d+) -> (\d+), chunk_id: (\d+)")
    _RE_ANY = re.compile(r"(StragglerMatching|OneWayMatching|TwoWayMatching): [^'\]]*")

    @classmethod
    def parse(cls, text: str) -> "Schedule":
        """Read a schedule back from the printed format.  Only the ``Round``
        headers and the matching lists are used; the bitmap lines give ``n``."""
        rounds: List[List[Matching]] = []
        n = 0
        expect_list = False
        for line in text.splitlines():
            line = line.strip()
            if line.startswith("Round "):
                expect_list = True
                continue
            if expect_list:
                expect_list = False
                rnd: List[Matching] = []
                for mm in cls._RE_ANY.finditer(line):
                    s = mm.group(0)
                    if (g := cls._RE_S.fullmatch(s.strip())):
                        rnd.append(StragglerMatching(*map(int, g.groups())))
                    elif (g := cls._RE_1.fullmatch(s.strip())):
                        rnd.append(OneWayMatching(*map(int, g.groups())))
                    elif (g := cls._RE_2.fullmatch(s.strip())):
                        a, b, ca, b2, a2, cb = map(int, g.groups())
                        if (a, b) != (a2, b2):
                            raise ScheduleError(f"two-way matching names four GPUs: {s}")
                        rnd.append(TwoWayMatching(a, b, ca, cb))
                    else:
                        raise ScheduleError(f"cannot parse matching: {s!r}")
                rounds.append(rnd)
                continue
            if line.startswith("GPU "):
                n = max(n, int(line.split()[1]) + 1)
        if n == 0:
            n = 1 + max((max(a, b) for rnd in rounds for m in rnd for a, b, _ in m.moves()), default=0)
        return cls(n, rounds)

    # ----------------------------------------------------------- permutation
    def rank_map_for_straggler(self, physical_straggler: int) -> List[int]:
        """logical -> physical rank map that puts ``physical_straggler`` at
        logical rank n-1 by swapping it with physical rank n-1; every other
        rank keeps its place.  This is the swap the reference does by remapping
        devices (implementation/custom_backend/src/dummy.cpp:157-168); here it
        is a relabelling of the schedule, no device remap is needed."""
        n = self.n
        if not 0 <= physical_straggler < n:
            raise ScheduleError(f"straggler {physical_straggler} out of range for n={n}")
        perm = list(range(n))
        perm[n - 1], perm[physical_straggler] = physical_straggler, n - 1
        return perm
