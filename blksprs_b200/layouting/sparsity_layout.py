"""Output-layout inference for the block-sparse matmul.

Same three helpers, signatures, messages and results as the reference
(blksprs/layouting/sparsity_layout.py:244-319); the layouts are combined by one
CUDA kernel of the native library instead of a float ``bmm`` / ``any``.
"""
import torch
from torch import Tensor

from .. import _cabi
from ..utils.validation import validate_device, validate_dimensions, validate_sparsity_block_size, \
    validate_sparsity_layout


def _check_matmul_layouts(sparsity_layout_x: Tensor, sparsity_layout_y: Tensor) -> None:
    validate_sparsity_layout(sparsity_layout_x, sparsity_layout_y)
    validate_device(sparsity_layout_x, sparsity_layout_y)
    if sparsity_layout_x.size(0) != sparsity_layout_y.size(0):
        raise ValueError("Batch dimensions of sparsity layouts must match")
    if sparsity_layout_x.size(-1) != sparsity_layout_y.size(-2):
        raise ValueError("Inner dimensions of sparsity layouts must match")


def _infer(sparsity_layout_x: Tensor, sparsity_layout_y: Tensor, mode: int) -> Tensor:
    _check_matmul_layouts(sparsity_layout_x, sparsity_layout_y)
    lx = sparsity_layout_x.contiguous()
    ly = sparsity_layout_y.contiguous()
    if lx.device.type != "cuda":
        raise RuntimeError("blksprs_b200 infers layouts on the GPU only")
    B, R, K = lx.shape
    C = ly.size(2)
    out = torch.empty((B, R, C), dtype=torch.bool, device=lx.device)
    with torch.cuda.device(lx.device):
        _cabi.check(_cabi.lib().bsp_layout_matmul(
            _cabi.ptr(lx), _cabi.LAYOUT_DTYPE_CODES[lx.dtype], _cabi.ptr(ly), _cabi.LAYOUT_DTYPE_CODES[ly.dtype],
            B, R, K, C, mode, _cabi.ptr(out), _cabi.stream_handle(lx.device)), "bsp_layout_matmul")
    return out


@torch.amp.custom_fwd(device_type="cuda")
def build_sparsity_layout_matmul(sparsity_layout_x: Tensor, sparsity_layout_y: Tensor) -> Tensor:
    """Exact structural product: block ``(i, j)`` is active iff some inner index ``k`` has both
    ``x(i, k)`` and ``y(k, j)`` active.

    Args:
        sparsity_layout_x (Tensor): layout ``(B, R, K)`` of the left operand.
        sparsity_layout_y (Tensor): layout ``(B, K, C)`` of the right operand.

    Returns:
        Tensor: bool layout ``(B, R, C)`` (a base ``torch.Tensor``).
    """
    return _infer(sparsity_layout_x, sparsity_layout_y, _cabi.LAYOUT_EXACT)


@torch.amp.custom_fwd(device_type="cuda")
def build_sparsity_layout_matmul_fast(sparsity_layout_x: Tensor, sparsity_layout_y: Tensor) -> Tensor:
    """Conservative approximation: ``(i, j)`` is active iff row ``i`` of x and column ``j`` of y each hold
    an active block (they need not share an inner index)."""
    return _infer(sparsity_layout_x, sparsity_layout_y, _cabi.LAYOUT_FAST)


@torch.amp.custom_fwd(device_type="cuda")
def build_sparsity_layout_matmul_outer(sparsity_layout_x: Tensor, sparsity_layout_y: Tensor) -> Tensor:
    """Outer approximation: ``(i, j)`` is active iff row ``i`` of x or column ``j`` of y holds an active block."""
    return _infer(sparsity_layout_x, sparsity_layout_y, _cabi.LAYOUT_OUTER)


def build_sparsity_layout_full(x: Tensor, sparsity_block_size: int) -> Tensor:
    """All-ones bool layout for a dense ``(B, rows, cols)`` tensor."""
    validate_dimensions(x)
    validate_device(x)
    validate_sparsity_block_size(sparsity_block_size, x)
    return torch.ones((x.size(0), x.size(1) // sparsity_block_size, x.size(2) // sparsity_block_size),
                      dtype=torch.bool, device=x.device)
