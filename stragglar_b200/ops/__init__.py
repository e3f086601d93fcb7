"""CUDA ops: the table-executing collective kernels and their helpers
(seeded fill, device delay, fused scale/cast, on-device verification)."""
from .local import LocalComm, cuda_lib, delay, fill_const, fill_uniform, host_uniform, scale_cast, verify_uniform_sum  # noqa: F401
