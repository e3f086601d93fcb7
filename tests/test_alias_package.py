"""The short package name `stragglar` resolves to the modules of `stragglar_b200` (one module object each)."""
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_alias_modules_are_the_same_objects():
    import stragglar.schedule as a
    import stragglar.synth.pow2 as p
    import stragglar_b200.schedule as b
    import stragglar_b200.synth.pow2 as q
    assert a is b and p is q
    import stragglar
    assert len(stragglar.synthesize(8).rounds) == 9


def test_alias_runs_as_module():
    out = subprocess.run([sys.executable, "-m", "stragglar.synth.pow2", "8"], cwd=REPO, capture_output=True, text=True,
                         check=True).stdout
    ref = subprocess.run([sys.executable, "-m", "stragglar_b200.synth.pow2", "8"], cwd=REPO, capture_output=True,
                         text=True, check=True).stdout
    strip = lambda s: [l for l in s.splitlines() if not l.startswith("Time taken")]
    assert strip(out) == strip(ref) and "Actual number of rounds 9" in out


def test_unknown_alias_submodule_raises_import_error():
    import importlib

    import pytest
    with pytest.raises(ImportError):
        importlib.import_module("stragglar.no_such_module")
