"""Prepare the instruction dataset of the end-to-end run.

    python examples/load_dataset.py [--out alpaca] [--samples 8192] [--download]

The counterpart of the reference's motivation/load_dataset.py, which downloads ``tatsu-lab/alpaca`` and saves it
to ``./alpaca``.  With ``--download`` (needs the ``datasets`` package and network access) this does the same and
also writes ``data.jsonl``; without it, or when the download fails, it writes ``--samples`` Alpaca-shaped records
from a seeded generator, so that the training script has a dataset on machines without a network.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200.utils.data import save_records, synthetic_records  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="alpaca")
    ap.add_argument("--samples", type=int, default=8192, help="records to synthesize (the reference trains on 8192)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--download", action="store_true", help="fetch tatsu-lab/alpaca with the `datasets` package")
    args = ap.parse_args()
    if args.download:
        try:
            from datasets import load_dataset
            ds = load_dataset("tatsu-lab/alpaca")["train"]
            ds.save_to_disk(args.out)
            path = save_records((dict(r) for r in ds), args.out)
            print(f"downloaded {len(ds)} records to {args.out} ({path})")
            return 0
        except Exception as e:   # no package, no network, no cache
            print(f"download failed ({type(e).__name__}: {e}); writing synthetic records instead", file=sys.stderr)
    path = save_records(synthetic_records(args.samples, args.seed), args.out)
    print(f"wrote {args.samples} synthetic records to {path}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
