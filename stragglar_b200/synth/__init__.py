"""Schedule synthesizers: :mod:`pow2` for power-of-two GPU counts,
:mod:`nonpow2` for even counts that are not a power of two."""
from ..schedule import Schedule


def synthesize(n: int) -> Schedule:
    """StragglAR schedule for ``n`` GPUs with the straggler at rank n-1."""
    if n == 1:
        return Schedule(1)
    if n & (n - 1) == 0:
        from .pow2 import synthesize as f
    else:
        from .nonpow2 import synthesize as f
    return f(n)
