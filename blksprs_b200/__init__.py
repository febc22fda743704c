"""B200-native (sm_100a) block-sparse matmul, drop-in for ``blksprs.ops.matmul``.

Same data model and call signatures as the blksprs library for the matmul path:
``ops.matmul``, ``ops.transpose``, ``layouting.build_sparsity_layout_matmul*``,
``utils.enable/disable_validation``; the compute runs in a C-ABI CUDA library
(``include/blksprs_b200.h``) loaded through ctypes.
"""
from .utils.blksprs_tensor import BlksprsTensor
from . import layouting, ops, utils

__version__ = "0.1.0"

__all__ = ["BlksprsTensor", "layouting", "ops", "utils", "__version__"]
