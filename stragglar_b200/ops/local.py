"""ctypes face of ``libsar_cuda.so``: the single-process communicator and the
helper kernels, operating on torch CUDA tensors.

The library must be present (``python -m stragglar_b200.build``); on a machine
with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

from ..compiler import Program, status_string

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libsar_cuda.so")
_lib = None

PATHS = {"simt": 0, "tma": 1, "simta": 2}


class RunOpts(C.Structure):
    _fields_ = [("path", C.c_int), ("blocks", C.c_int), ("threads", C.c_int), ("tile_bytes", C.c_uint32),
                ("timeout_s", C.c_double), ("scale", C.c_float), ("timed", C.c_int), ("trace_rounds", C.c_int),
                ("stages", C.c_int), ("store_window", C.c_int),
                ("user_in", C.POINTER(C.c_void_p)), ("user_out", C.POINTER(C.c_void_p)), ("user_dtype", C.c_int)]


def cuda_lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"{_LIB_PATH} is missing: run `python -m stragglar_b200.build`")
        L = C.CDLL(_LIB_PATH)
        L.sar_local_create.restype = C.c_void_p
        L.sar_local_create.argtypes = [C.c_int, C.POINTER(C.c_int), C.c_int, C.c_char_p, C.c_int]
        L.sar_local_destroy.argtypes = [C.c_void_p]
        L.sar_local_stream.restype, L.sar_local_stream.argtypes = C.c_void_p, [C.c_void_p, C.c_int]
        L.sar_local_run.restype = C.c_int
        L.sar_local_run.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_uint64, C.c_int,
                                    C.POINTER(RunOpts), C.POINTER(C.c_uint64), C.c_char_p, C.c_int]
        L.sar_local_sync.restype, L.sar_local_sync.argtypes = C.c_uint32, [C.c_void_p, C.POINTER(C.c_float)]
        L.sar_local_trace.restype, L.sar_local_trace.argtypes = C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]
        L.sar_local_round_trace.restype, L.sar_local_round_trace.argtypes = C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]
        L.sar_local_alloc.restype = C.c_int
        L.sar_local_alloc.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.POINTER(C.c_void_p), C.c_char_p, C.c_int]
        L.sar_local_free.restype, L.sar_local_free.argtypes = C.c_int, [C.c_void_p, C.c_void_p]
        L.sar_local_multicast_groups.restype, L.sar_local_multicast_groups.argtypes = C.c_int, [C.c_void_p, C.c_void_p]
        L.sar_local_multicast_supported.restype, L.sar_local_multicast_supported.argtypes = C.c_int, [C.c_void_p]
        L.sar_cuda_delay.argtypes = [C.c_uint64, C.c_void_p]
        L.sar_cuda_fill_uniform.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_uint64, C.c_void_p]
        L.sar_cuda_fill_const.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_float, C.c_void_p]
        L.sar_cuda_scale_cast.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_uint64, C.c_float, C.c_void_p]
        L.sar_cuda_verify_uniform_sum.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.POINTER(C.c_uint64),
                                                  C.c_int, C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_void_p]
        L.sar_cuda_max_emulated_blocks.argtypes = [C.c_int, C.c_int, C.c_int]
        L.sar_host_uniform.restype, L.sar_host_uniform.argtypes = C.c_float, [C.c_uint64, C.c_uint64]
        # the compiler entry points live in this library as well
        L.sar_program_build.restype = C.c_void_p
        _lib = L
    return _lib


def _dtype_code(t) -> int:
    import torch
    return {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[t.dtype]


def _check(err: int, what: str) -> None:
    if err:
        raise RuntimeError(f"{what}: CUDA error {err}")


def _stream_ptr(stream=None) -> int:
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return s.cuda_stream


def delay(ms: float, stream=None) -> None:
    """Keep the stream busy for ``ms`` milliseconds of device wall clock."""
    _check(cuda_lib().sar_cuda_delay(int(ms * 1e6), _stream_ptr(stream)), "delay")


def fill_uniform(t, seed: int, stream=None) -> None:
    """t[i] = uniform[-1, 1) from a counter hash of (seed, i); reproducible on the host with :func:`host_uniform`."""
    _check(cuda_lib().sar_cuda_fill_uniform(t.data_ptr(), t.numel(), _dtype_code(t), seed, _stream_ptr(stream)), "fill")


def fill_const(t, value: float, stream=None) -> None:
    _check(cuda_lib().sar_cuda_fill_const(t.data_ptr(), t.numel(), _dtype_code(t), value, _stream_ptr(stream)), "fill")


def host_uniform(seed: int, index: int) -> float:
    return cuda_lib().sar_host_uniform(seed, index)


def scale_cast(dst, src, scale: float = 1.0, stream=None) -> None:
    """dst[i] = dtype(dst)(src[i] * scale) in one pass."""
    if dst.numel() != src.numel():
        raise ValueError("size mismatch")
    _check(cuda_lib().sar_cuda_scale_cast(dst.data_ptr(), _dtype_code(dst), src.data_ptr(), _dtype_code(src),
                                          src.numel(), scale, _stream_ptr(stream)), "scale_cast")


def verify_uniform_sum(t, seeds: Sequence[int], scale: float = 1.0, atol: float = 1e-5, rtol: float = 0.0,
                       begin: int = 0, end: Optional[int] = None):
    """Compare ``t`` on the device with scale * sum_r uniform(seeds[r], i).
    Returns (number of bad elements, max abs error)."""
    import torch
    res = torch.zeros(2, dtype=torch.int32, device=t.device)
    arr = (C.c_uint64 * len(seeds))(*seeds)
    end = t.numel() if end is None else end
    with torch.cuda.device(t.device):
        _check(cuda_lib().sar_cuda_verify_uniform_sum(t.data_ptr(), begin, end, _dtype_code(t), arr, len(seeds), scale,
                                                      atol, rtol, res.data_ptr(), _stream_ptr()), "verify")
        bad, bits = res.cpu().tolist()
    import struct
    return bad, struct.unpack("f", struct.pack("I", bits & 0xffffffff))[0]


class LocalComm:
    """n ranks in this process: one per CUDA device, or (``emulate=True``) all
    on one device where a collective is a single cooperative launch."""

    def __init__(self, n: int, devices: Optional[Sequence[int]] = None, emulate: bool = False):
        L = cuda_lib()
        devices = list(devices) if devices is not None else ([0] * n if emulate else list(range(n)))
        err = C.create_string_buffer(256)
        self._h = L.sar_local_create(n, (C.c_int * len(devices))(*devices), int(emulate), err, 256)
        if not self._h:
            raise RuntimeError("communicator: " + err.value.decode())
        self.n, self.devices, self.emulate = n, devices, emulate

    def close(self):
        if self._h:
            cuda_lib().sar_local_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def run(self, program: Program, tensors, path: str = "simt", blocks: int = 0, threads: int = 0,
            tile_bytes: int = 0, scale: float = 1.0, delay_ms: Optional[Sequence[float]] = None,
            timeout_s: float = 10.0, timed: bool = False, trace_rounds: bool = False, stages: int = 0, store_window: int = 0,
            user_tensors=None) -> None:
        """Enqueue ``program`` in place on ``tensors`` (one per rank).  ``trace_rounds`` keeps per-round
        statistics of this run for :meth:`round_trace`.

        ``user_tensors`` (one per rank, any of the three dtypes, same numel) selects staged mode for a single-phase
        program: ``tensors`` then only serve as the buffers the ranks reach into; the kernel reads rank r's input
        from ``user_tensors[r]`` and writes the result back there, converting between the two dtypes."""
        if len(tensors) != self.n:
            raise ValueError(f"need {self.n} tensors")
        t0 = tensors[0]
        for t in tensors:
            if t.dtype != t0.dtype or t.numel() != t0.numel() or not t.is_contiguous() or not t.is_cuda:
                raise ValueError("tensors must be contiguous CUDA tensors of one dtype and size")
        if program._h is None:
            raise ValueError("program was freed")
        # program handles come from libsar_core.so; libsar_cuda.so is built from the same
        # sources and reads them through the same accessors
        uin = None
        udt = 0
        if user_tensors is not None:
            if len(user_tensors) != self.n or any(u.numel() != t0.numel() or not u.is_contiguous() for u in user_tensors):
                raise ValueError("user_tensors: one contiguous tensor of the same numel per rank")
            uin = (C.c_void_p * self.n)(*[u.data_ptr() for u in user_tensors])
            udt = _dtype_code(user_tensors[0])
        opts = RunOpts(PATHS[path], blocks, threads, tile_bytes, timeout_s, scale, int(timed), int(trace_rounds), stages,
                       store_window, uin, uin, udt)
        ptrs = (C.c_void_p * self.n)(*[t.data_ptr() for t in tensors])
        dl = (C.c_uint64 * self.n)(*[int(d * 1e6) for d in delay_ms]) if delay_ms is not None else None
        # The ranks run on streams of the communicator: make them wait for what the caller has queued on the
        # current torch stream of every device involved (fills, clones, reference sums), so that the collective
        # neither reads inputs that are not written yet nor overwrites tensors that are still being read.
        import torch
        for r in range(self.n):
            dev = tensors[r].device
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dev))
            torch.cuda.ExternalStream(cuda_lib().sar_local_stream(self._h, r), device=dev).wait_event(ev)
        err = C.create_string_buffer(256)
        rc = cuda_lib().sar_local_run(self._h, program._h, ptrs, t0.numel(), _dtype_code(t0), C.byref(opts), dl, err, 256)
        if rc:
            raise RuntimeError(f"launch failed ({rc}): {err.value.decode()}")

    def sync(self, check: bool = True) -> List[float]:
        """Wait for every rank; returns the per-rank device time in ms of the
        last timed run.  Raises on a device-side timeout unless ``check`` is
        false, in which case the status code is stored in ``last_status``."""
        ms = (C.c_float * self.n)()
        self.last_status = cuda_lib().sar_local_sync(self._h, ms)
        if check and self.last_status:
            raise RuntimeError("collective failed: " + (status_string(self.last_status) if self.last_status < 0x1000
                                                        else f"CUDA error {self.last_status - 0x1000}"))
        return list(ms)

    def trace(self):
        out = (C.c_uint64 * (2 * self.n))()
        _check(cuda_lib().sar_local_trace(self._h, out), "trace")
        return [(out[2 * r], out[2 * r + 1]) for r in range(self.n)]

    # ---- symmetric buffers, optionally bound to NVLink multicast (NVLS) objects
    MULTICAST_MODES = {False: 0, None: 0, "off": 0, True: 1, "require": 1, "try": 2}

    def multicast_supported(self) -> bool:
        """True when every device of the communicator offers NVLink multicast (one rank per device)."""
        return bool(cuda_lib().sar_local_multicast_supported(self._h))

    def alloc(self, numel: int, dtype=None, multicast="try", sub_members: int = 0):
        """One buffer of ``numel`` elements per rank, as torch tensors that alias the allocation.

        ``multicast``: ``False`` plain device memory; ``True`` virtual-memory allocations bound to a multicast
        object over all ranks and, when ``sub_members`` (a rank bitmask) is given, to a second one over those ranks
        -- an error where multicast is not available; ``"try"`` multicast when available, else plain.  On the simt
        path, collectives on these tensors (or on equal slices of them) send reductions over, and pushes to, all
        members of a group through the switch.  Free with :meth:`free` (or by closing the communicator); the
        tensors must not be used afterwards."""
        import torch
        dtype = dtype or torch.float32
        esize = torch.empty(0, dtype=dtype).element_size()
        ptrs = (C.c_void_p * self.n)()
        err = C.create_string_buffer(512)
        rc = cuda_lib().sar_local_alloc(self._h, numel * esize, self.MULTICAST_MODES[multicast], sub_members, ptrs, err, 512)
        if rc:
            raise RuntimeError("symmetric allocation failed: " + err.value.decode())

        class _Raw:   # what torch.as_tensor needs to alias device memory
            def __init__(self, ptr, nbytes):
                self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

        out = []
        for r in range(self.n):
            dev = self.devices[0] if self.emulate else self.devices[r]
            raw = torch.as_tensor(_Raw(ptrs[r], max(numel * esize, 1)), device=f"cuda:{dev}")
            out.append(raw[: numel * esize].view(dtype))
        return out

    def free(self, tensors) -> None:
        """Releases an allocation made by :meth:`alloc` (pass the list it returned)."""
        if cuda_lib().sar_local_free(self._h, C.c_void_p(tensors[0].data_ptr())):
            raise ValueError("not an allocation of this communicator")

    def multicast_groups(self, tensor) -> int:
        """Bit 0: the multicast group of all ranks serves ``tensor``'s allocation; bit 1: the sub-group does."""
        return cuda_lib().sar_local_multicast_groups(self._h, C.c_void_p(tensor.data_ptr()))

    MAX_ROUNDS = 64

    def round_trace(self):
        """Per rank, the rounds it worked on in the last run made with ``trace_rounds=True``:
        ``[{round: (start_ns, end_ns, wait_ns)}]`` -- %globaltimer stamps of the round's first item starting and
        its last item being announced, and the time its items spent waiting for operands (summed over items)."""
        m = self.MAX_ROUNDS
        out = (C.c_uint64 * (self.n * 3 * m))()
        _check(cuda_lib().sar_local_round_trace(self._h, out), "round_trace")
        res = []
        for r in range(self.n):
            base = r * 3 * m
            res.append({k: (out[base + k], out[base + m + k], out[base + 2 * m + k]) for k in range(m)
                        if out[base + k] != 0xFFFFFFFFFFFFFFFF})
        return res

    def max_emulated_blocks(self, dtype_code: int = 0, path: str = "simt", threads: int = 0) -> int:
        return cuda_lib().sar_cuda_max_emulated_blocks(dtype_code, PATHS[path], threads)
