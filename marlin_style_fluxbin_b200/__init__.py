"""B200-native batch-1 packed-Linear decode path (W3 g128 planar GEMV, two-base binary-basis GEMV,
fused RMSNorm / RoPE, static-cache decode under CUDA graphs), behind the reference project's
Python plugin surface.  Device code lives in ``csrc/`` and is reached through the C ABI declared in
``include/fluxbin_b200.h``; there is no CPU or other fallback for the packed kernels.
"""
from .packing import TWO_BASE_PACKED_FORMAT, pack_two_bases, unpack_two_bases  # noqa: F401

__version__ = "0.1.0"
__all__ = ["TWO_BASE_PACKED_FORMAT", "pack_two_bases", "unpack_two_bases"]
