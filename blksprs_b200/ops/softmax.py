"""Row-wise block-sparse softmax (fp32), the op between the two matmuls of block-sparse attention.

``softmax``, ``softmax_regular`` and ``softmax_fused`` keep the reference's signatures and errors
(blksprs/ops/softmax.py:23-91, 373-436); all three run the same single kernel of the native library,
so the fused variant has no row-size limit to fall back from.  Inactive blocks do not take part in
the softmax (they are equivalent to ``-inf``).
"""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _cabi
from ..utils.blksprs_tensor import BlksprsTensor
from ..utils.tools import build_packed_indices, finalize_layout_cache, plain_dispatch, prepare_layout_cache
from ..utils.validation import ensure_contiguous, validate_contiguous, validate_device, validate_dimensions, \
    validate_dtype_float_32, validate_sparsity, validate_sparsity_block_size


def softmax_build_layout_cache(layout_cache: dict | None, sparsity_layout: Tensor) -> dict:
    """Reverse LUT of the layout, cached under the reference's "softmax" cache key."""
    layout_cache = prepare_layout_cache(layout_cache, "softmax", sparsity_layout)
    if "packed_indices" not in layout_cache:
        layout_cache["packed_indices"] = build_packed_indices(sparsity_layout)
    validate_contiguous(sparsity_layout, layout_cache["packed_indices"])
    return finalize_layout_cache(layout_cache)


class _BlockSparseSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, packed: Tensor, layout_shape, bs: int):
        B, R, C = layout_shape
        x = _cabi.aligned(x)
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _cabi.check(_cabi.lib().bsp_softmax_fwd(_cabi.ptr(x), x.size(0), _cabi.ptr(packed), B, R, C, bs,
                                                    _cabi.ptr(out), _cabi.stream_handle(x.device)), "bsp_softmax_fwd")
        ctx.save_for_backward(out, packed)
        ctx.layout_shape, ctx.sparsity_block_size = (B, R, C), bs
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    @plain_dispatch
    def backward(ctx, grad_output: Tensor):
        out, packed = ctx.saved_tensors
        B, R, C = ctx.layout_shape
        grad_output = _cabi.aligned(grad_output.contiguous().to(torch.float32))
        grad_x = torch.empty_like(out)
        with torch.cuda.device(out.device):
            _cabi.check(_cabi.lib().bsp_softmax_bwd(_cabi.ptr(grad_output), _cabi.ptr(out), out.size(0),
                                                    _cabi.ptr(packed), B, R, C, ctx.sparsity_block_size,
                                                    _cabi.ptr(grad_x), _cabi.stream_handle(out.device)),
                        "bsp_softmax_bwd")
        return grad_x, None, None, None


@torch.compiler.disable
@plain_dispatch
def _softmax_eager(x, sparsity_layout, sparsity_block_size, layout_cache):
    x = ensure_contiguous(x)
    validate_dimensions(x)
    validate_contiguous(x)
    validate_dtype_float_32(x)
    validate_device(x)
    validate_sparsity(sparsity_block_size, (x, sparsity_layout))
    validate_sparsity_block_size(sparsity_block_size, x)
    if x.size(0) == 0:
        return BlksprsTensor.wrap(x)
    layout_cache = softmax_build_layout_cache(layout_cache, sparsity_layout)
    out = _BlockSparseSoftmax.apply(x, layout_cache["packed_indices"], tuple(sparsity_layout.shape),
                                    sparsity_block_size)
    return BlksprsTensor.wrap(out)


@torch.amp.custom_fwd(device_type="cuda")
def softmax(x: BlksprsTensor, sparsity_layout: Tensor, sparsity_block_size: int,
            flag_fused: bool = True, layout_cache: dict | None = None) -> BlksprsTensor:
    """Computes a row-wise block-sparse softmax.

    Args:
        x (BlksprsTensor): The compressed input tensor (float32).
        sparsity_layout (Tensor): The sparsity layout of ``x``.
        sparsity_block_size (int): The size of the sparsity blocks.
        flag_fused (bool, optional): Kept for compatibility; both settings run the same kernel.
        layout_cache (dict, optional): Reusable layout metadata cache (default ``None``).

    Returns:
        BlksprsTensor: The row-wise softmax in compressed form.
    """
    return _softmax_eager(x, sparsity_layout, sparsity_block_size, layout_cache)


@torch.amp.custom_fwd(device_type="cuda")
def softmax_regular(x: BlksprsTensor, sparsity_layout: Tensor, sparsity_block_size: int,
                    layout_cache: dict | None = None) -> BlksprsTensor:
    """Row-wise softmax over the active blocks of each row (maximum and sum across all of them)."""
    return _softmax_eager(x, sparsity_layout, sparsity_block_size, layout_cache)


@torch.amp.custom_fwd(device_type="cuda")
def softmax_fused(x: BlksprsTensor, sparsity_layout: Tensor, sparsity_block_size: int,
                  layout_cache: dict | None = None) -> BlksprsTensor:
    """Row-wise softmax; same kernel as :func:`softmax` (no row-size limit applies here)."""
    return _softmax_eager(x, sparsity_layout, sparsity_block_size, layout_cache)
