"""Keep a rank's host threads and pinned buffers on the CPUs next to its GPU.

On a two-socket host a process that runs on the far socket allocates its pinned staging buffers there, and every
host-to-device copy then crosses the socket interconnect; with eight ranks copying at once that halves the rate
each of them sees.  :func:`bind_to_gpu` reads the GPU's CPU affinity from NVML (read-only: nothing about the GPU
is changed) and narrows the calling process to those CPUs, so that memory it pins afterwards is local.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence


def cpus_from_masks(masks: Sequence[int], bits_per_word: int = 64) -> List[int]:
    """CPU indices set in NVML's affinity bit masks (word i covers CPUs i*bits .. i*bits+bits-1)."""
    out = []
    for w, m in enumerate(masks):
        m = int(m)
        b = 0
        while m:
            if m & 1:
                out.append(w * bits_per_word + b)
            m >>= 1
            b += 1
    return out


def gpu_cpus(index: int, nvml=None) -> Optional[List[int]]:
    """CPUs NVML names as local to GPU ``index`` (its physical index among the visible devices), or None."""
    try:
        if nvml is None:
            import pynvml as nvml
        nvml.nvmlInit()
        try:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if ids and index < len(ids) and ids[index].isdigit():
                index = int(ids[index])
            h = nvml.nvmlDeviceGetHandleByIndex(index)
            words = (os.cpu_count() or 64) // 64 + 1
            return cpus_from_masks(nvml.nvmlDeviceGetCpuAffinity(h, words)) or None
        finally:
            nvml.nvmlShutdown()
    except Exception:
        return None


def bind_to_gpu(index: int, nvml=None) -> Optional[List[int]]:
    """Restrict this process to the CPUs local to GPU ``index``.  Returns the CPUs now in effect, or None when
    NVML gave no answer or none of its CPUs is available to the process (nothing is changed then)."""
    cpus = gpu_cpus(index, nvml)
    if not cpus or not hasattr(os, "sched_setaffinity"):
        return None
    allowed = sorted(set(cpus) & os.sched_getaffinity(0))
    if not allowed:
        return None
    try:
        os.sched_setaffinity(0, allowed)
    except OSError:
        return None
    return allowed
