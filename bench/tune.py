"""Sweep the lowering knobs of the StragglAR variants on the GPUs of this box and rank the settings.

    python bench/tune.py [--sizes 67108864,268435456,1073741824] [--delay -1] [--iters 10] [--full] [--out DIR]

Runs ``bin/allreduce`` once per setting (all sizes in one process), reads its CSV and prints, per algorithm and
size, the settings ordered by the median time (max over ranks, device-timed, every iteration verified on the
device).  The settings are combinations of the environment switches the library reads:

* ``STRAGGLAR_BLOCKS``         thread blocks per rank
* ``STRAGGLAR_GATE``           rounds of ``stragglar`` one after the other instead of overlapping freely
* ``STRAGGLAR_LANE1_EIGHTHS``  share of the blocks of the forwarding lane (``stragglar_a2a``)
* ``STRAGGLAR_COPY`` / ``STRAGGLAR_LANES``  pulled or pushed copies, one or two lanes
* ``STRAGGLAR_PATH``           bulk-copy pipeline (tma), simt, simta
* ``STRAGGLAR_NVLS``           buffers bound to NVLink multicast objects (``--nvls``)

The default set is about 30 runs of a few seconds each; ``--full`` adds the cross products.
"""
import argparse
import os
import statistics
import subprocess
import sys
from collections import defaultdict

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "bin", "allreduce")


def settings(full: bool, nvls: bool):
    out = []
    for b in (32, 48, 64, 96, 128):
        out.append(("stragglar", {"STRAGGLAR_BLOCKS": b}))
        out.append(("stragglar", {"STRAGGLAR_BLOCKS": b, "STRAGGLAR_GATE": 1}))
    for b in (24, 32, 48, 64):
        out.append(("stragglar_a2a", {"STRAGGLAR_BLOCKS": b}))
        for e in (5, 6):
            out.append(("stragglar_a2a", {"STRAGGLAR_BLOCKS": b, "STRAGGLAR_LANE1_EIGHTHS": e}))
    out.append(("stragglar", {"STRAGGLAR_PATH": "simta", "STRAGGLAR_BLOCKS": 64}))
    out.append(("stragglar_a2a", {"STRAGGLAR_PATH": "simta", "STRAGGLAR_BLOCKS": 32}))
    if full:
        for b in (64, 128):
            for copy in ("pull", "push"):
                for lanes in (1, 2):
                    for gate in (0, 1):
                        out.append(("stragglar", {"STRAGGLAR_BLOCKS": b, "STRAGGLAR_COPY": copy, "STRAGGLAR_LANES": lanes,
                                                  "STRAGGLAR_GATE": gate}))
        for b in (32, 64):
            for copy in ("pull", "push"):
                for lanes in (1, 2):
                    out.append(("stragglar_a2a", {"STRAGGLAR_BLOCKS": b, "STRAGGLAR_COPY": copy, "STRAGGLAR_LANES": lanes}))
    if nvls:
        for path in ("simt", "simta"):
            for alg in ("rsag", "stragglar_a2a", "stragglar"):
                out.append((alg, {"STRAGGLAR_NVLS": 1, "STRAGGLAR_PATH": path}))
    return out


def label(env) -> str:
    return " ".join(f"{k.replace('STRAGGLAR_', '').lower()}={v}" for k, v in env.items()) or "defaults"


def run_one(alg, env, sizes, iters, delay, warmup, out_dir):
    e = dict(os.environ)
    e.update({k: str(v) for k, v in env.items()})
    e["STRAGGLAR_WARMUP"] = str(warmup)
    p = subprocess.run([EXE, sizes, alg, str(iters), str(delay)], capture_output=True, text=True, env=e, timeout=900)
    if out_dir:
        name = (alg + "_" + label(env)).replace(" ", "_").replace("=", "")
        with open(os.path.join(out_dir, name + ".csv"), "w") as f:
            f.write(p.stdout)
        if p.stderr.strip():
            with open(os.path.join(out_dir, name + ".err"), "w") as f:
                f.write(p.stderr)
    times = defaultdict(list)
    for line in p.stdout.splitlines():
        c = line.split(",")
        if len(c) >= 14 and c[0] == alg and c[1].isdigit():
            times[int(c[1])].append(float(c[4]) - float(c[13]))      # runtime minus the delay as served
    failed = p.returncode != 0 or "VERIFY FAILED" in p.stderr
    return {s: statistics.median(v) for s, v in times.items()}, failed, p.stderr.strip().splitlines()[-1:] if failed else []


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="67108864,268435456,1073741824")
    ap.add_argument("--delay", default="-1")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--full", action="store_true")
    ap.add_argument("--nvls", action="store_true")
    ap.add_argument("--out", default=None, help="directory for the raw CSVs")
    args = ap.parse_args()
    if not os.path.exists(EXE):
        print("bin/allreduce is not built: python -m stragglar_b200.build", file=sys.stderr)
        return 2
    if args.out:
        os.makedirs(args.out, exist_ok=True)
    results = defaultdict(list)   # (alg, size) -> [(ms, label)]
    for alg, env in settings(args.full, args.nvls):
        try:
            med, failed, why = run_one(alg, env, args.sizes, args.iters, args.delay, args.warmup, args.out)
        except subprocess.TimeoutExpired:
            med, failed, why = {}, True, ["timed out"]
        tag = label(env) + (" [FAILED: " + " ".join(why) + "]" if failed else "")
        for size, ms in med.items():
            results[(alg, size)].append((ms, tag))
        print(f"# {alg} {tag}: " + ", ".join(f"{s >> 20} MiB {ms:.3f} ms" for s, ms in sorted(med.items())), flush=True)
    print()
    for (alg, size), rows in sorted(results.items()):
        print(f"{alg}, {size >> 20} MiB (net ms, best first)")
        for ms, tag in sorted(rows):
            print(f"  {ms:8.3f}  {tag}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
