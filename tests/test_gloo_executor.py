"""The CPU configuration: 4 gloo ranks execute the StragglAR schedule that the
power-of-two synthesizer gives for n = 4 on 1,048,576 fp32 elements per rank
(uniform[-1, 1) seeded by rank), rank 3 arrives 5 ms late; the result is
checked against an fp64 sum and the round count against the analytical model."""
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, alg, count, straggler, q):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from stragglar_b200 import simulate
        from stragglar_b200.compiler import compile_program
        from stragglar_b200.parallel.cpu_exec import GlooExecutor
        from stragglar_b200.synth import synthesize
        sched = synthesize(world) if alg == "stragglar" and world & (world - 1) == 0 else None
        prog = compile_program(alg, world, prephase=True, straggler=straggler, schedule=sched)
        x = torch.empty(count).uniform_(-1, 1, generator=torch.Generator().manual_seed(rank))
        want = torch.stack([torch.empty(count).uniform_(-1, 1, generator=torch.Generator().manual_seed(r)).double()
                            for r in range(world)]).sum(0)
        ex = GlooExecutor()
        late = straggler if straggler is not None else world - 1
        ex.all_reduce(prog, x, delay_s=0.005 if rank == late else 0.0)
        err = (x.double() - want).abs().max().item()
        assert err <= 1e-5, err
        if alg == "stragglar" and sched is not None:
            # the pre-phase is one extra round on top of the schedule's n - 2 + log2(n)
            assert len(sched) == simulate.stragglar_rounds(world)
            assert ex.rounds_executed == len(sched) + (1 if world > 2 else 0)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def _run(world, alg, count, straggler=None):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ps = [ctx.Process(target=_worker, args=(r, world, port, alg, count, straggler, q)) for r in range(world)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(180)
    msgs = []
    while not q.empty():
        msgs.append(q.get())
    assert not msgs and all(p.exitcode == 0 for p in ps), "\n".join(msgs)


def test_n4_stragglar_one_mebi_elements_late_rank3():
    _run(4, "stragglar", 1_048_576)


@pytest.mark.parametrize("alg,world,straggler", [("ring", 4, None), ("stragglar", 6, 2), ("direct", 4, None),
                                                 ("rhd", 4, None), ("stragglar_a2a", 4, 1)])
def test_other_algorithms_over_gloo(alg, world, straggler):
    _run(world, alg, 20_011, straggler)
