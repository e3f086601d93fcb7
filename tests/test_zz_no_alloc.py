"""The allocation-free entry point, called through its exported C symbol.

Callers that may not call cudaMalloc (code living inside another framework's
memory budget, plugins in a context without headroom, tools that must not
disturb the host program's allocations) get `sar_emulated_allreduce_noalloc`:
the same table executor, with flags, control words, parameters and the device
copy of the op table in a static 1 MiB device array instead of allocated
memory.  Here its output is compared with the regular entry point's
(`LocalComm(emulate=True)`, simt path) on two calls in a row -- the second
call finds the first call's flags in the shared array and must clear them --
and oversized requests must be refused with a message.  This file is collected
last so that a failure here cannot hide the result of any other test.
"""
import ctypes as C

import pytest
import torch

from stragglar_b200 import compiler as sc

pytestmark = pytest.mark.gpu


def _entry():
    from stragglar_b200.ops import cuda_lib
    L = cuda_lib()
    f = L.sar_emulated_allreduce_noalloc
    f.restype = C.c_int
    f.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_uint64, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_void_p,
                  C.c_char_p, C.c_int]
    return f


def _inputs(n, count, dtype, salt):
    from stragglar_b200 import ops
    xs = [torch.empty(count, dtype=dtype, device="cuda:0") for _ in range(n)]
    for r, x in enumerate(xs):
        ops.fill_uniform(x, seed=100 * salt + r)
    torch.cuda.synchronize()
    return xs


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 6e-2)])
def test_matches_the_allocating_entry_point_twice_in_a_row(dtype, tol):
    from stragglar_b200 import ops
    f = _entry()
    n, count, scale = 8, 300_007, 0.125
    table = sc.compile_table("stragglar", n)
    comm = ops.LocalComm(n, emulate=True)
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    code = {torch.float32: 0, torch.bfloat16: 1}[dtype]
    for call in range(2):
        a = _inputs(n, count, dtype, salt=call)
        b = [x.clone() for x in a]
        want = torch.stack([x.double() for x in a]).sum(0) * scale
        comm.run(table._program, a, path="simt", blocks=4, scale=scale)
        comm.sync()
        err = C.create_string_buffer(256)
        ptrs = (C.c_void_p * n)(*[x.data_ptr() for x in b])
        rc = f(table._h, ptrs, count, code, scale, 4, status.data_ptr(), torch.cuda.current_stream().cuda_stream, err, 256)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for x, y in zip(a, b):
            torch.testing.assert_close(y.double(), x.double(), atol=tol, rtol=1e-2 if dtype != torch.float32 else 1e-6)
            torch.testing.assert_close(y.double(), want, atol=tol, rtol=1e-2 if dtype != torch.float32 else 1e-6)
    comm.close()


def test_requests_beyond_the_static_array_are_refused():
    f = _entry()
    err = C.create_string_buffer(256)
    # 16 ranks do not fit the array
    t16 = sc.compile_table("ring", 16)
    xs = [torch.zeros(64, device="cuda:0") for _ in range(16)]
    ptrs = (C.c_void_p * 16)(*[x.data_ptr() for x in xs])
    assert f(t16._h, ptrs, 64, 0, 1.0, 1, None, None, err, 256) == 2 and b"too many ranks" in err.value
    # a buffer that would need more flag words than the array holds (nothing is touched: the size check comes first)
    t2 = sc.compile_table("ring", 2)
    ptrs = (C.c_void_p * 2)(xs[0].data_ptr(), xs[1].data_ptr())
    assert f(t2._h, ptrs, 1 << 36, 0, 1.0, 1, None, None, err, 256) == 2 and b"too large" in err.value
    # misaligned buffer
    ptrs = (C.c_void_p * 2)(xs[0].data_ptr() + 4, xs[1].data_ptr())
    assert f(t2._h, ptrs, 32, 0, 1.0, 1, None, None, err, 256) == 1


def test_a_call_during_stream_capture_is_refused():
    """The entry point copies its parameters from host memory that only lives during the call, so it must not be
    recorded into a graph: while the stream is capturing it returns code 1 and enqueues nothing."""
    f = _entry()
    n = 2
    table = sc.compile_table("ring", n)
    xs = [torch.zeros(64, device="cuda:0") for _ in range(n)]
    ptrs = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    err = C.create_string_buffer(256)
    # first call outside capture: resolves the scratch array's address on this device
    assert f(table._h, ptrs, 64, 0, 1.0, 1, None, torch.cuda.current_stream().cuda_stream, err, 256) == 0
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        g.capture_begin()
        try:
            rc = f(table._h, ptrs, 64, 0, 1.0, 1, None, s.cuda_stream, err, 256)
        finally:
            g.capture_end()
    assert rc == 1 and b"not capturable" in err.value
    torch.cuda.synchronize()
