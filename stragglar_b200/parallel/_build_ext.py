"""Compiles the c10d backend extension ``stragglar_b200/_C*.so`` in-tree with
explicit compiler calls (nvcc for the kernels with
``-gencode arch=compute_100a,code=sm_100a``, g++ for the host code against
the installed torch headers).  Nothing is built at import time: ``load()``
only imports what ``build()`` produced."""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(ROOT, "csrc")
OBJ = os.path.join(ROOT, "build", "backend")
SO = os.path.join(PKG, "_C" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

HOST_SOURCES = [
    os.path.join(CSRC, "backend", "process_group_stragglar.cpp"),
    os.path.join(CSRC, "backend", "transport.cpp"),
    os.path.join(CSRC, "core", "plan.cpp"),
    os.path.join(CSRC, "core", "host_exec.cpp"),
    os.path.join(CSRC, "core", "c_api.cpp"),
]
CUDA_SOURCES = [os.path.join(CSRC, "kernels", "exec_table.cu")]


def _deps() -> List[str]:
    out = []
    for base, _, files in os.walk(CSRC):
        if os.path.basename(base) in ("bench", "runtime"):
            continue
        out += [os.path.join(base, f) for f in files]
    out.append(os.path.abspath(__file__))   # the source list lives here
    return out


def _stale(target: str, deps: List[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    from ..build import NVCC_FLAGS, nvcc

    if not force and not _stale(SO, _deps()):
        return SO
    os.makedirs(OBJ, exist_ok=True)
    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-DPYBIND11_COMPILER_TYPE=\"_gcc\"", "-DPYBIND11_STDLIB=\"_libstdcpp\"", "-DPYBIND11_BUILD_ABI=\"_cxxabi1018\""]
    # pybind ABI tags must match the ones torch was built with
    defs = defs[:3]
    for name in ("COMPILER_TYPE", "STDLIB", "BUILD_ABI"):
        val = getattr(torch._C, f"_PYBIND11_{name}", None)
        if val is not None:
            defs.append(f'-DPYBIND11_{name}="{val}"')
    jobs = []
    objs = []
    for src in HOST_SOURCES:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, _deps()):
            jobs.append(["g++", "-std=c++17", "-O2", "-fPIC", "-Wno-nonnull", *defs, *inc, "-c", src, "-o", obj])
    for src in CUDA_SOURCES:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, _deps()):
            jobs.append([nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj])

    def run(cmd):
        print("+", " ".join(cmd[:6]), "...", cmd[-3], flush=True)
        subprocess.check_call(cmd)

    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
    link = ["g++", "-shared", *objs, "-o", SO + ".tmp", f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-lc10", "-lc10_cuda",
            "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{cuda_lib}", "-lcudart", "-lrt", "-pthread"]
    run(link)
    os.replace(SO + ".tmp", SO)
    return SO


def load():
    """Import the built extension; raises with the build command when missing."""
    if "stragglar_b200._C" in sys.modules:
        return sys.modules["stragglar_b200._C"]
    if not os.path.exists(SO):
        raise ImportError(f"{SO} is missing: run `python -m stragglar_b200.build`")
    import torch  # noqa: F401  (libtorch must be loaded first)
    loader = importlib.machinery.ExtensionFileLoader("stragglar_b200._C", SO)
    spec = importlib.util.spec_from_loader("stragglar_b200._C", loader, origin=SO)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules["stragglar_b200._C"] = mod
    return mod
