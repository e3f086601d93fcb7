"""Report what the library will find on this machine.

    python -m stragglar_b200.utils.env_check

The counterpart of the reference's motivation/env_check.py (CUDA availability,
GPU names, torch version), extended with what this library depends on: the
peer-access matrix between the GPUs, the built native parts and the registered
c10d backend.
"""
from __future__ import annotations

import os
import sys


def report() -> dict:
    import torch
    info = {"torch": torch.__version__, "cuda_available": torch.cuda.is_available(),
            "cuda_version": torch.version.cuda, "gpus": [], "peer_access": [], "native": {}}
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            info["gpus"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}",
                                 "memory_gib": round(p.total_memory / 2**30, 1), "sms": p.multi_processor_count})
        info["peer_access"] = [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)]
                               for i in range(n)]
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    root = os.path.dirname(here)
    for name, path in (("libsar_core.so", os.path.join(here, "lib", "libsar_core.so")),
                       ("libsar_cuda.so", os.path.join(here, "lib", "libsar_cuda.so")),
                       ("bin/allreduce", os.path.join(root, "bin", "allreduce")),
                       ("bin/reducescatter", os.path.join(root, "bin", "reducescatter"))):
        info["native"][name] = os.path.exists(path)
    ext = [f for f in os.listdir(here) if f.startswith("_C") and f.endswith(".so")]
    info["native"]["c10d extension"] = bool(ext)
    try:
        import torch.distributed as dist
        import stragglar_b200.parallel  # noqa: F401
        info["backend_registered"] = "stragglar" in dist.Backend.backend_list
    except Exception as e:  # pragma: no cover - depends on the build state
        info["backend_registered"] = f"no ({e})"
    return info


def main() -> int:
    info = report()
    print(f"CUDA available: {info['cuda_available']}")
    print(f"PyTorch version: {info['torch']} (CUDA {info['cuda_version']})")
    print(f"Number of GPUs: {len(info['gpus'])}")
    for g in info["gpus"]:
        print(f"GPU {g['index']}: {g['name']} sm_{g['sm']} {g['memory_gib']} GiB {g['sms']} SMs")
    if info["peer_access"]:
        ok = all(all(row) for row in info["peer_access"])
        print("Peer access between all GPU pairs:", "yes" if ok else "NO (the collectives need it)")
    for k, v in info["native"].items():
        print(f"{k}: {'built' if v else 'missing (python -m stragglar_b200.build)'}")
    print(f"c10d backend 'stragglar' registered: {info['backend_registered']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
