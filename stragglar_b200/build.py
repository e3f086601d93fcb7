"""Builds the native parts in-tree: ``lib/libsar_core.so`` (schedule compiler
and host executor, host compiler only), ``lib/libsar_cuda.so`` (kernels and the
single-process communicator, nvcc for sm_100a), the ``allreduce`` and
``reducescatter`` benchmark programs under ``bin/`` and the c10d backend
extension ``_C``.  ``python -m stragglar_b200.build`` builds everything.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(ROOT, "csrc")
LIB = os.path.join(HERE, "lib")
BIN = os.path.join(ROOT, "bin")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-Wno-nonnull"]
CORE = [os.path.join(CSRC, "core", f) for f in ("plan.cpp", "host_exec.cpp", "c_api.cpp")]
CUDA = [os.path.join(CSRC, "kernels", "exec_table.cu"), os.path.join(CSRC, "runtime", "local_comm.cu"),
        os.path.join(CSRC, "kernels", "noalloc.cu"), os.path.join(CSRC, "runtime", "symm_alloc.cu")]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: str, deps: List[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def _all_sources() -> List[str]:
    out = []
    for base, _, files in os.walk(CSRC):
        out += [os.path.join(base, f) for f in files]
    return out


def _run(cmd: List[str]) -> None:
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_core(force: bool = False) -> str:
    from .compiler import build_core as f
    return f(force)


def build_cuda(force: bool = False) -> str:
    out = os.path.join(LIB, "libsar_cuda.so")
    if force or not _newer(out, _all_sources()):
        os.makedirs(LIB, exist_ok=True)
        _run([nvcc(), *NVCC_FLAGS, "-shared", *CUDA, *CORE, "-o", out])
    return out


def build_bench(force: bool = False) -> List[str]:
    os.makedirs(BIN, exist_ok=True)
    outs = []
    for name in ("allreduce", "reducescatter"):
        src = os.path.join(CSRC, "bench", name + ".cu")
        if not os.path.exists(src):
            continue
        out = os.path.join(BIN, name)
        if force or not _newer(out, _all_sources()):
            _run([nvcc(), *NVCC_FLAGS, src, *CUDA, *CORE, "-o", out])
        outs.append(out)
    return outs


def build_backend(force: bool = False):
    src = os.path.join(CSRC, "backend")
    if not os.path.isdir(src):
        return None
    from .parallel import _build_ext
    return _build_ext.build(force)


def build_all(force: bool = False) -> None:
    build_core(force)
    build_cuda(force)
    build_bench(force)
    build_backend(force)


if __name__ == "__main__":
    build_all("--force" in sys.argv)
