"""Buffer sizes padded for StragglAR's n-1 chunks.

``python -m stragglar_b200.pad <num_gpus>`` prints, for nine sizes from
256 KiB to 1 GiB, the padded size whose per-GPU chunk is the smallest multiple
of 1 KiB *strictly larger* than ``size // (n-1)`` -- the same two lines as the
reference helper (stragglar/pad_buffers.py:19-53).  The collectives of this
library accept any size (chunks are cut unevenly on 16-byte boundaries), so
padding is only needed to run the reference's executables on identical byte
counts.
"""
from __future__ import annotations

import sys
from typing import List

KIB = 1024
BUFFER_SIZES = [256 * KIB, 1 << 20, 4 << 20, 16 << 20, 64 << 20, 128 << 20, 256 << 20, 512 << 20, 1 << 30]


def padded_size(nbytes: int, n: int, granule: int = KIB) -> int:
    """Padded buffer size for ``n`` GPUs (n >= 2)."""
    if n < 2:
        raise ValueError("padding is defined for at least 2 GPUs")
    chunk = nbytes // (n - 1)
    return (chunk // granule + 1) * granule * (n - 1)


def padded_sizes(n: int) -> List[int]:
    return [padded_size(b, n) for b in BUFFER_SIZES]


def main(argv=None) -> int:
    argv = sys.argv if argv is None else argv
    if len(argv) != 2:
        print("Need exactly one argument: <num_gpus>")
        return 1
    n = int(argv[1])
    print("Original buffer sizes: ", " ".join(str(x) for x in BUFFER_SIZES))
    print("Padded buffer sizes: ", " ".join(str(x) for x in padded_sizes(n)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
