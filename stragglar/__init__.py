"""``stragglar``: the short name of :mod:`stragglar_b200`.

``import stragglar.synth.pow2`` and ``python -m stragglar.synth.pow2 8`` reach the very same modules as
``stragglar_b200.synth.pow2``: a meta-path finder maps ``stragglar.X`` to ``stragglar_b200.X`` and hands out
the one module object, so nothing is imported twice (the c10d backend registers once whichever name is
used).  The files beside this one (``synthesizer_pow2.py``, ``synthesizer_nonpow2.py``, ``simulation.py``,
``pad_buffers.py``) keep the script names of the reference's ``stragglar/`` folder.
"""
import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys

_ALIAS = __name__
_REAL = "stragglar_b200"


def _real_name(fullname: str) -> str:
    return _REAL + fullname[len(_ALIAS):]


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Resolves ``stragglar.<x>`` to the module ``stragglar_b200.<x>``."""

    def __init__(self):
        self._real_specs = {}

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        try:
            real = importlib.util.find_spec(_real_name(fullname))
        except (ImportError, ValueError):
            return None
        if real is None:
            return None   # e.g. stragglar.simulation: a script of this folder, found by the path finder
        return importlib.machinery.ModuleSpec(fullname, self, origin=real.origin,
                                              is_package=real.submodule_search_locations is not None)

    def create_module(self, spec):
        module = importlib.import_module(_real_name(spec.name))
        self._real_specs[spec.name] = module.__spec__
        return module

    def exec_module(self, module):
        # already executed under its real name; the import machinery has just put the alias spec on it
        for alias, real in list(self._real_specs.items()):
            if real.name == module.__name__:
                module.__spec__ = real
                del self._real_specs[alias]

    def get_code(self, fullname):   # what `python -m stragglar.<x>` runs
        real = importlib.util.find_spec(_real_name(fullname))
        return real.loader.get_code(real.name)

    def get_source(self, fullname):
        real = importlib.util.find_spec(_real_name(fullname))
        return real.loader.get_source(real.name)

    def is_package(self, fullname):
        real = importlib.util.find_spec(_real_name(fullname))
        return real.submodule_search_locations is not None


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

from stragglar_b200 import __version__, synthesize  # noqa: E402,F401
