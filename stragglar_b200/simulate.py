"""Analytical alpha-beta cost model of StragglAR, recursive halving-doubling,
ring and direct AllReduce.

``python -m stragglar_b200.simulate`` prints the two speedup lines of the
reference model (stragglar/simulation.py:50-58; alpha = 3 us, 450 GiB/s,
1 GiB).  ``--b200`` evaluates the same formulas with this machine class's
constants (NVLink 5: 900 GB/s per direction nominal, 770 GB/s measured peer
copy).  The formulas (stragglar/simulation.py:10-38), with R the number of
StragglAR rounds for n GPUs:

  stragglar  R*a + R/(n-1) * S*b
  rhd        2*log2(n)*a + 2(n-1)/n * S*b            (power of two)
             2*ceil(log2 n)*a + 2*S*b*(1.5 - 1/2^floor(log2 n))   (otherwise;
             3-2 elimination of Rabenseifner & Traff)
  ring       2(n-1)*a + 2(n-1)/n * S*b
  direct     log2(n)*a + log2(n) * S*b

``--table`` prints absolute times per n, with the two algorithms this library adds for a switched box
(every GPU reaches every peer at the full port rate):

  stragglar_a2a  3*a + S*b            all matchings at once, then a direct all-gather: S per direction per GPU
  rsag           2*a + 2(n-1)/n * S*b   one-shot reduce-scatter + all-gather (the ring's bytes in two steps)
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass
from typing import Dict, Iterable, Optional

import numpy as np

GIB = 1024 ** 3

#: rounds the reference model assumes for even non-power-of-two n
#: (stragglar/simulation.py:7)
NONPOW2_ROUNDS = {192: 208, 96: 108, 48: 57, 24: 27, 12: 15, 6: 7}

POWERS_OF_TWO = [4, 8, 16, 32, 64, 128, 256]
IN_BETWEEN = [6, 12, 24, 48, 96, 192]


@dataclass(frozen=True)
class LinkModel:
    alpha_ms: float = 3 / 1000
    beta_ms_per_byte: float = 1000 / (450 * GIB)
    size_bytes: int = 1 * GIB

    @classmethod
    def reference(cls) -> "LinkModel":
        return cls()

    @classmethod
    def b200(cls, measured: bool = True, size_bytes: int = GIB, alpha_us: float = 2.0) -> "LinkModel":
        gbs = 770.0 if measured else 900.0
        return cls(alpha_us / 1000, 1000 / (gbs * 1e9), size_bytes)


def stragglar_rounds(n: int, table: Optional[Dict[int, int]] = None):
    """Round count used by the model: n-2+log2(n) for powers of two, the
    table entry otherwise."""
    table = NONPOW2_ROUNDS if table is None else table
    if n in table:
        return table[n]
    return n - 2 + np.log2(n)


def compute_costs(N: Iterable[int], model: LinkModel = LinkModel(), rounds: Optional[Dict[int, int]] = None):
    """Per-n cost in ms of (stragglar, rhd, ring, direct)."""
    a, b, s = model.alpha_ms, model.beta_ms_per_byte, model.size_bytes
    table = NONPOW2_ROUNDS if rounds is None else rounds
    stragglar, rhd, ring, direct = [], [], [], []
    for n in N:
        c = stragglar_rounds(n, table)
        stragglar.append(c * a + (c / (n - 1)) * s * b)
        if n in table:
            up, down = np.ceil(np.log2(n)), np.floor(np.log2(n))
            rhd.append((2 * up * a) + (2 * s * b) * (1.5 - (1 / (2 ** down))))
        else:
            rhd.append((2 * np.log2(n)) * a + ((2 * (n - 1)) / n) * s * b)
        ring.append((2 * (n - 1)) * a + ((2 * (n - 1)) / n) * s * b)
        direct.append(np.log2(n) * a + np.log2(n) * s * b)
    return stragglar, rhd, ring, direct


def compute_speedups(N: Iterable[int], model: LinkModel = LinkModel(), rounds: Optional[Dict[int, int]] = None):
    """Speedup over ring of (stragglar, rhd, direct, ring)."""
    stragglar, rhd, ring, direct = compute_costs(N, model, rounds)
    return ([r / x for r, x in zip(ring, stragglar)],
            [r / x for r, x in zip(ring, rhd)],
            [r / x for r, x in zip(ring, direct)],
            [1.0 for _ in ring])


def compute_costs_switched(N: Iterable[int], model: LinkModel = LinkModel()):
    """Per-n cost in ms of (stragglar_a2a, rsag): the algorithms that rely on a full-bandwidth switch."""
    a, b, s = model.alpha_ms, model.beta_ms_per_byte, model.size_bytes
    return [3 * a + s * b for _ in N], [2 * a + (2 * (n - 1) / n) * s * b for n in N]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--b200", action="store_true", help="use NVLink 5 constants instead of the reference's")
    ap.add_argument("--nominal", action="store_true", help="with --b200: 900 GB/s instead of the measured 770")
    ap.add_argument("--size", type=int, default=GIB, help="buffer bytes (default 1 GiB)")
    ap.add_argument("--table", action="store_true", help="absolute times in ms per n instead of the two speedup lines")
    args = ap.parse_args(argv)
    model = LinkModel.b200(not args.nominal, args.size) if args.b200 else LinkModel(size_bytes=args.size)
    if args.table:
        N = sorted(POWERS_OF_TWO + IN_BETWEEN)
        sar, rhd, ring, direct = compute_costs(N, model)
        a2a, rsag = compute_costs_switched(N, model)
        print(f"{'n':>4s} {'stragglar':>10s} {'a2a':>8s} {'ring':>8s} {'rhd':>8s} {'rsag':>8s} {'direct':>8s}   (ms)")
        for i, n in enumerate(N):
            print(f"{n:4d} {sar[i]:10.3f} {a2a[i]:8.3f} {ring[i]:8.3f} {rhd[i]:8.3f} {rsag[i]:8.3f} {direct[i]:8.3f}")
        return 0
    p = compute_speedups(POWERS_OF_TWO, model)
    q = compute_speedups(IN_BETWEEN, model)
    print("Speedups for powers of two:", *p)
    print("Speedups for non-power-of-two values:", *q)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
