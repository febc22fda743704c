"""Host-side helpers of the matmul path: compressed-tensor marker, validation switches, shape helpers."""
from . import validation
from .blksprs_tensor import BlksprsTensor
from .processing import apply_torch_linear, apply_torch_linear_cached
from .tools import clear_implicit_layout_caches, do_shape_blocksparse, set_implicit_layout_caches, \
    undo_shape_blocksparse
from .validation import disable_contiguous, disable_validation, enable_contiguous, enable_validation

__all__ = [
    "BlksprsTensor",
    "apply_torch_linear",
    "apply_torch_linear_cached",
    "clear_implicit_layout_caches",
    "disable_contiguous",
    "disable_validation",
    "do_shape_blocksparse",
    "enable_contiguous",
    "enable_validation",
    "set_implicit_layout_caches",
    "undo_shape_blocksparse",
    "validation",
]
