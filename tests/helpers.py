"""Shared test helpers: seeded inputs, the fp64 oracle and chunk geometry."""
import numpy as np


def chunk_bounds(count: int, esize: int, num_chunks: int):
    """Element ranges of the chunks, as the library cuts them."""
    vw = 16 // esize
    nvec = count // vw
    q, rem = divmod(nvec, num_chunks)
    out = []
    for c in range(num_chunks):
        b = (q * c + min(c, rem)) * vw
        e = (q * (c + 1) + min(c + 1, rem)) * vw if c < num_chunks - 1 else count
        out.append((b, e))
    return out


def seeded_inputs(n: int, count: int, dtype=np.float32):
    """Rank r's buffer: uniform[-1, 1) from a generator seeded with r."""
    return [np.random.default_rng(r).uniform(-1.0, 1.0, count).astype(dtype) for r in range(n)]


def oracle_sum(bufs):
    return np.sum(np.stack([b.astype(np.float64) for b in bufs]), axis=0)


def emulate_prephase(bufs, alg: str, straggler: int):
    """Put the buffers in the state the DELAY = -1 mode assumes: the
    non-stragglers' sum is already in place (in chunk i of logical rank i for
    the StragglAR variants, everywhere for direct)."""
    n = len(bufs)
    if n < 2:
        return
    count = bufs[0].size
    non = [r for r in range(n) if r != straggler]
    part = np.sum(np.stack([bufs[r].astype(np.float64) for r in non]), axis=0).astype(bufs[0].dtype)
    if alg == "direct":
        for r in non:
            bufs[r][:] = part
        return
    l2p = list(range(n))
    l2p[n - 1], l2p[straggler] = straggler, n - 1
    for i, (b, e) in enumerate(chunk_bounds(count, bufs[0].itemsize, n - 1)):
        bufs[l2p[i]][b:e] = part[b:e]
