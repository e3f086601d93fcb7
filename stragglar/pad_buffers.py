#!/usr/bin/env python
"""`python pad_buffers.py ...` -- the command line of the reference's stragglar/pad_buffers.py,
served by stragglar_b200.pad."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200.pad import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(sys.argv))
