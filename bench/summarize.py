"""Summarise benchmark CSVs (ours, the reference's, NCCL's) into one table:
median runtime per (algorithm, size, delay), algorithm and bus bandwidth with
the measured delay taken off, and the fraction of the NVLink roofline.

    python bench/summarize.py out/ours.csv out/ref.csv out/nccl.csv
"""
import statistics
import sys
from collections import defaultdict


def load(path):
    rows = []
    with open(path) as f:
        for line in f:
            p = line.strip().split(",")
            if len(p) < 6 or not p[1].isdigit():
                continue
            try:
                rows.append(dict(alg=p[0], bytes=int(p[1]), it=int(p[2]), delay=float(p[3]), ms=float(p[4]),
                                 path=p[8] if len(p) > 8 else "ref", real_delay=float(p[13]) if len(p) > 13 else max(float(p[3]), 0.0),
                                 n=int(p[6]) if len(p) > 6 else 0, frac=float(p[12]) if len(p) > 12 else float("nan"),
                                 kernel_us=float(p[14]) if len(p) > 14 else float("nan")))
            except ValueError:
                continue
    return rows


def main(paths):
    print(f"{'source':28s} {'alg':14s} {'MiB':>8s} {'delay':>6s} {'median ms':>10s} {'net ms':>8s} {'algbw GB/s':>11s} {'roofline':>9s} {'in-kernel us':>13s}")
    for path in paths:
        groups = defaultdict(list)
        for r in load(path):
            groups[(r["alg"], r["path"], r["bytes"], r["delay"])].append(r)
        for (alg, pth, nbytes, delay), rs in sorted(groups.items(), key=lambda kv: (kv[0][2], kv[0][0], kv[0][3])):
            ms = statistics.median(r["ms"] for r in rs)
            net = ms - rs[0]["real_delay"]
            frac = statistics.median(r["frac"] for r in rs)
            kus = statistics.median(r["kernel_us"] for r in rs)
            print(f"{path[-28:]:28s} {alg + '/' + pth:14s} {nbytes / 2**20:8.1f} {delay:6.1f} {ms:10.3f} {net:8.3f} "
                  f"{nbytes / 1e9 / (net / 1e3):11.1f} {frac:9.3f} {kus:13.1f}")


if __name__ == "__main__":
    main(sys.argv[1:])
