"""Peer-copy bandwidth between two GPUs of the box, the denominator of the NVLink rooflines.

Times ``dst.copy_(src)`` across devices (the driver's peer copy) with CUDA events, one direction alone and both
directions at once (two streams, one per source device; the slower of the two defines the rate), for a buffer
larger than L2.  Prints one JSON line per case.

    python bench/peer_bw.py [--mib 1024] [--iters 10] [--a 0] [--b 1]
"""
from __future__ import annotations

import argparse
import json
import sys


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--a", type=int, default=0)
    ap.add_argument("--b", type=int, default=1)
    args = ap.parse_args()
    import torch
    if torch.cuda.device_count() < 2:
        print(json.dumps({"unavailable": "needs two GPUs"}))
        return 0
    nbytes = args.mib << 20
    da, db = torch.device(f"cuda:{args.a}"), torch.device(f"cuda:{args.b}")
    xa, ya = torch.empty(nbytes, dtype=torch.uint8, device=da), torch.empty(nbytes, dtype=torch.uint8, device=da)
    xb, yb = torch.empty(nbytes, dtype=torch.uint8, device=db), torch.empty(nbytes, dtype=torch.uint8, device=db)
    sa, sb = torch.cuda.Stream(da), torch.cuda.Stream(db)

    def timed(both: bool):
        best = 1e9
        for it in range(args.iters + 3):
            torch.cuda.synchronize(da); torch.cuda.synchronize(db)
            ea0, ea1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            eb0, eb1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(sa):
                ea0.record(); yb.copy_(xa, non_blocking=True); ea1.record()     # a -> b, issued by a
            if both:
                with torch.cuda.stream(sb):
                    eb0.record(); ya.copy_(xb, non_blocking=True); eb1.record()  # b -> a, issued by b
            torch.cuda.synchronize(da); torch.cuda.synchronize(db)
            ms = ea0.elapsed_time(ea1)
            if both:
                ms = max(ms, eb0.elapsed_time(eb1))
            if it >= 3:
                best = min(best, ms)
        return best

    for both in (False, True):
        ms = timed(both)
        print(json.dumps({"case": "both directions at once" if both else "one direction", "bytes": nbytes,
                          "devices": [args.a, args.b], "ms_best": round(ms, 4),
                          "GBps_per_direction": round(nbytes / ms / 1e6, 1)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
