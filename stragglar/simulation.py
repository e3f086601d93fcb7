#!/usr/bin/env python
"""`python simulation.py ...` -- the command line of the reference's stragglar/simulation.py,
served by stragglar_b200.simulate."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200.simulate import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
