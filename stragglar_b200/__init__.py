"""stragglar_b200: straggler-aware AllReduce for one NVSwitch box of B200 GPUs.

Sub-packages and modules (imported on demand; importing this package loads neither torch nor CUDA):

* :mod:`.synth`     schedule synthesizers (power-of-two and even non-power-of-two GPU counts)
* :mod:`.schedule`  schedule IR, parser / printer / validator, straggler relabelling
* :mod:`.compiler`  schedule -> per-rank op tables (native), host executor, hazard checker
* :mod:`.simulate`  alpha-beta cost model    :mod:`.pad`  padded buffer sizes    :mod:`.detect`  straggler detection
* :mod:`.ops`       single-process CUDA communicator and helper kernels (ctypes)
* :mod:`.parallel`  c10d backend ``"stragglar"``, symmetric tensors, DDP hooks, send/recv executor
* :mod:`.models`    the Llama-style decoder of the end-to-end run
"""
__version__ = "0.1.0"

__all__ = ["synthesize", "__version__"]


def synthesize(n: int):
    """StragglAR schedule for ``n`` GPUs with the straggler at rank n-1 (see :func:`.synth.synthesize`)."""
    from .synth import synthesize as f
    return f(n)
