"""Runs every helper kernel of ``libsar_cuda.so`` once or twice on one GPU and prints its device time.

The helpers are the kernels around the table executor: seeded fill, constant fill, pre-phase fill, fused
scale/cast (same-type vector form and converting form), on-device verification, segment copy, segment reduce,
the device delay, the cross-rank barrier and the signal/wait hand-shake (both with one rank, so nothing waits).
The buffers are larger than L2 so that DRAM figures mean something.  Used for timing and as the workload of
the Nsight Compute captures summarised under ``profiles/``:

    python bench/helper_kernels.py [--mib 256] [--reps 2]
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=256, help="size of the fp32 working buffers")
    ap.add_argument("--reps", type=int, default=2)
    a = ap.parse_args()
    import torch
    from stragglar_b200 import ops
    L = ops.cuda_lib()
    dev = torch.device("cuda:0")
    n = a.mib * (1 << 20) // 4
    f32 = torch.empty(n, dtype=torch.float32, device=dev)
    f32b = torch.empty(n, dtype=torch.float32, device=dev)
    f32c = torch.empty(n, dtype=torch.float32, device=dev)
    bf = torch.empty(n, dtype=torch.bfloat16, device=dev)
    res = torch.zeros(2, dtype=torch.int32, device=dev)
    ctrl = torch.zeros(128, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    seeds = (C.c_uint64 * 2)(3, 4)

    class Seg(C.Structure):
        _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("bytes", C.c_uint64)]

    seg = (Seg * 1)(Seg(f32.data_ptr(), f32c.data_ptr(), n * 4))
    srcs = (C.c_void_p * 2)(f32.data_ptr(), f32b.data_ptr())
    ctrls = (C.c_void_p * 1)(ctrl.data_ptr())
    L.sar_cuda_fill_uniform_sum.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.POINTER(C.c_uint64), C.c_int, C.c_void_p]
    L.sar_cuda_copy_segments.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    L.sar_cuda_reduce_segments.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_uint64, C.c_int, C.c_float, C.c_void_p]
    L.sar_cuda_barrier.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_uint32, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p]
    L.sar_cuda_signal_wait.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]

    # (name, bytes read + written, call)
    cases = [
        ("sar_fill_uniform_kernel<float>", 4 * n, lambda: L.sar_cuda_fill_uniform(f32.data_ptr(), n, 0, 3, st)),
        ("sar_fill_uniform_kernel<float> (2nd buffer)", 4 * n, lambda: L.sar_cuda_fill_uniform(f32b.data_ptr(), n, 0, 4, st)),
        ("sar_fill_const_kernel<bf16>", 2 * n, lambda: L.sar_cuda_fill_const(bf.data_ptr(), n, 1, 1.5, st)),
        ("sar_scale_cast_vec8_kernel<bf16,float>", 6 * n, lambda: L.sar_cuda_scale_cast(bf.data_ptr(), 1, f32.data_ptr(), 0, n, 0.125, st)),
        ("sar_reduce_segments_vec_kernel<float>", 12 * n, lambda: L.sar_cuda_reduce_segments(f32c.data_ptr(), srcs, 2, n, 0, 1.0, st)),
        ("sar_verify_kernel<float>", 4 * n, lambda: L.sar_cuda_verify_uniform_sum(f32c.data_ptr(), 0, n, 0, seeds, 2, 1.0, 1e-5, 0.0, res.data_ptr(), st)),
        ("sar_scale_vec_kernel<float>", 8 * n, lambda: L.sar_cuda_scale_cast(f32c.data_ptr(), 0, f32c.data_ptr(), 0, n, 0.5, st)),
        ("sar_copy_segments_kernel", 8 * n, lambda: L.sar_cuda_copy_segments(seg, 1, st)),
        ("sar_fill_uniform_sum_kernel<float>", 4 * n, lambda: L.sar_cuda_fill_uniform_sum(f32c.data_ptr(), 0, n, 0, seeds, 2, st)),
        ("sar_delay_kernel (50 us)", 0, lambda: L.sar_cuda_delay(50_000, st)),
        ("sar_barrier_kernel (one rank)", 0, lambda: L.sar_cuda_barrier(ctrls, 0, 1, 1, 1, 1_000_000, res.data_ptr(), st)),
        ("sar_signal_wait_kernel (set, then wait for the same word)", 0,
         lambda: L.sar_cuda_signal_wait(ctrl.data_ptr() + 64, 7, ctrl.data_ptr() + 64, 7, 1_000_000, ctrl.data_ptr() + 8, res.data_ptr(), st)),
    ]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bad = 0
    for name, nbytes, call in cases:
        best = 1e9
        for _ in range(a.reps):
            e0.record()
            rc = call()
            e1.record()
            torch.cuda.synchronize()
            if rc:
                print(f"{name}: CUDA error {rc}")
                bad += 1
                break
            best = min(best, e0.elapsed_time(e1))
        gbs = nbytes / best / 1e6 if nbytes else 0.0
        note = ""
        if name.startswith("sar_verify"):
            # the buffer holds uniform(3) + uniform(4) at this point (reduce_segments): no element may be off
            wrong = res.cpu().tolist()[0]
            note = f"  wrong elements: {wrong}"
            bad += 1 if wrong else 0
        print(f"{name:62s} {best * 1e3:9.1f} us" + (f"  {gbs:8.1f} GB/s (read+write)" if nbytes else "") + note)
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
