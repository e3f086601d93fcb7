"""Programs are freed and rebuilt on the host all the time; a new one may be
allocated at the address of a freed one.  The communicator's device-side table
cache must therefore never confuse two different tables."""
import gc

import pytest
import torch

from stragglar_b200 import compiler as sc

pytestmark = pytest.mark.gpu


def test_tables_of_freed_programs_are_not_reused():
    from stragglar_b200 import ops
    n, count = 4, 20_000
    comm = ops.LocalComm(n, emulate=True)
    for rep in range(6):
        for alg, pre in (("stragglar", False), ("ring", True), ("direct", False), ("stragglar_a2a", False), ("rhd", True)):
            prog = sc.compile_program(alg, n, pre)
            xs = [torch.empty(count, device="cuda:0") for _ in range(n)]
            for r, x in enumerate(xs):
                ops.fill_uniform(x, r)
            torch.cuda.synchronize()
            want = torch.stack([x.double() for x in xs]).sum(0)
            if not pre:
                from test_gpu_emulated import _prephase
                _prephase(xs, alg, n - 1)
            comm.run(prog, xs, blocks=2, tile_bytes=4096)
            comm.sync()
            for x in xs:
                torch.testing.assert_close(x.double(), want, atol=2e-5, rtol=1e-6)
            del prog
            gc.collect()
    comm.close()
