#!/usr/bin/env python
"""`python synthesizer_nonpow2.py ...` -- the command line of the reference's stragglar/synthesizer_nonpow2.py,
served by stragglar_b200.synth.nonpow2."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200.synth.nonpow2 import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(sys.argv))
