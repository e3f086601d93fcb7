"""Packaging of stragglar_b200.

    pip install --no-build-isolation -e .        # builds the native parts in-tree, then installs in place

The native parts (schedule compiler, CUDA kernels for sm_100a, benchmark programs, c10d extension) are built by
``stragglar_b200/build.py`` into ``stragglar_b200/lib``, ``stragglar_b200/_C*.so`` and ``bin/`` -- nvcc is
needed, a GPU is not.  The counterpart of the reference's implementation/custom_backend/setup.py, which builds its
backend extension for sm_80 with torch's CUDAExtension.
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    """Runs the in-tree native build before the Python files are collected."""

    def run(self):
        if os.environ.get("STRAGGLAR_SKIP_NATIVE_BUILD", "0") != "1":
            sys.path.insert(0, ROOT)
            from stragglar_b200 import build
            build.build_all()
        super().run()


def version() -> str:
    with open(os.path.join(ROOT, "stragglar_b200", "__init__.py")) as f:
        for line in f:
            if line.startswith("__version__"):
                return line.split("=")[1].strip().strip('"')
    return "0"


setup(
    name="stragglar_b200",
    version=version(),
    description="Straggler-aware AllReduce for one NVSwitch box of B200 GPUs: compiled schedules, persistent peer-memory kernels, c10d backend",
    packages=find_packages(include=["stragglar_b200", "stragglar_b200.*", "stragglar"]),
    package_data={"stragglar_b200": ["lib/*.so", "_C*.so"]},
    python_requires=">=3.10",
    install_requires=["numpy", "torch"],
    extras_require={"nonpow2": ["networkx"], "test": ["pytest", "hypothesis"]},
    cmdclass={"build_py": BuildNative},
)
