"""Maximum-weight maximum-cardinality matching on a small undirected graph.

The non-power-of-two synthesizer pairs idle GPUs by solving this problem once
per round.  When ``networkx`` is importable its blossom implementation is used
with the node and edge insertion order given by the caller, which makes the
synthesizer reproduce the reference's rounds for the same networkx version
(stragglar/synthesizer_nonpow2.py:169).  Without networkx an exact bitmask
dynamic program is used for up to 22 idle GPUs and a greedy heaviest-edge
pairing above that; both give valid schedules, possibly with other
tie-breaks.
"""
from __future__ import annotations

from functools import lru_cache
from typing import Dict, Sequence, Set, Tuple

Edge = Tuple[int, int, int]  # (u, v, weight)


def _exact(nodes: Sequence[int], edges: Sequence[Edge]) -> Set[Tuple[int, int]]:
    idx = {g: i for i, g in enumerate(nodes)}
    w: Dict[Tuple[int, int], int] = {}
    for u, v, wt in edges:
        a, b = sorted((idx[u], idx[v]))
        w[(a, b)] = max(w.get((a, b), 0), wt)
    k = len(nodes)

    @lru_cache(maxsize=None)
    def best(mask: int) -> Tuple[int, int]:
        # (cardinality, weight) of the best matching inside ``mask``
        if mask == 0:
            return (0, 0)
        i = (mask & -mask).bit_length() - 1
        rest = mask & ~(1 << i)
        res = best(rest)  # leave i unmatched
        m = rest
        while m:
            j = (m & -m).bit_length() - 1
            m &= m - 1
            if (i, j) in w:
                c, wt = best(rest & ~(1 << j))
                cand = (c + 1, wt + w[(i, j)])
                if cand > res:
                    res = cand
        return res

    out: Set[Tuple[int, int]] = set()
    mask = (1 << k) - 1
    while mask:
        i = (mask & -mask).bit_length() - 1
        rest = mask & ~(1 << i)
        target = best(mask)
        if best(rest) == target:
            mask = rest
            continue
        m = rest
        while m:
            j = (m & -m).bit_length() - 1
            m &= m - 1
            if (i, j) in w:
                c, wt = best(rest & ~(1 << j))
                if (c + 1, wt + w[(i, j)]) == target:
                    out.add((nodes[i], nodes[j]))
                    mask = rest & ~(1 << j)
                    break
    return out


def _greedy(nodes: Sequence[int], edges: Sequence[Edge]) -> Set[Tuple[int, int]]:
    used: Set[int] = set()
    out: Set[Tuple[int, int]] = set()
    for u, v, _ in sorted(edges, key=lambda e: (-e[2], e[0], e[1])):
        if u not in used and v not in used:
            used |= {u, v}
            out.add((u, v))
    return out


def max_weight_matching(nodes: Sequence[int], edges: Sequence[Edge], use_networkx: bool = True):
    """Pairs ``(u, v)`` of a maximum-cardinality matching of largest weight."""
    if use_networkx:
        try:
            import networkx as nx
        except ImportError:  # pragma: no cover - networkx is optional
            nx = None
        if nx is not None:
            g = nx.Graph()
            for v in nodes:
                g.add_node(v)
            for u, v, wt in edges:
                g.add_edge(u, v, weight=wt)
            return nx.max_weight_matching(g, maxcardinality=True)
    if len(nodes) <= 22:
        return _exact(list(nodes), list(edges))
    return _greedy(list(nodes), list(edges))
