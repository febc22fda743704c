"""Host-side helpers of the matmul path: compressed-tensor marker, validation switches, shape helpers."""
from . import validation
from .blksprs_tensor import BlksprsTensor
from .processing import apply_torch_linear, apply_torch_linear_cached
from .tools import do_shape_blocksparse, undo_shape_blocksparse
from .validation import disable_contiguous, disable_validation, enable_contiguous, enable_validation

__all__ = [
    "BlksprsTensor",
    "apply_torch_linear",
    "apply_torch_linear_cached",
    "disable_contiguous",
    "disable_validation",
    "do_shape_blocksparse",
    "enable_contiguous",
    "enable_validation",
    "undo_shape_blocksparse",
    "validation",
]
