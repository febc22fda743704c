"""Compressed transpose ``bs.ops.transpose`` (the op the reference's matmul backward is defined through).

Same signature, cache entries and results as blksprs/ops/transpose.py:13-99.
The reference makes two full copies (``x.transpose(-1,-2).contiguous()`` and a
block permutation, blksprs/ops/flow.py:64-111); here one kernel of the native
library transposes and permutes the blocks in a single pass.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _cabi
from ..utils.blksprs_tensor import BlksprsTensor
from ..utils.tools import as_base_tensor, build_layout_indices, build_packed_indices, count_active_blocks, \
    finalize_layout_cache, plain_dispatch, prepare_layout_cache
from ..utils.validation import ensure_contiguous, validate_contiguous, validate_device, validate_dimensions, \
    validate_dtype_supported, validate_sparsity, validate_sparsity_block_size

_SRC = "_b200_source_blocks"


def transpose_build_layout_cache(layout_cache: dict | None, sparsity_layout: Tensor) -> dict:
    """Builds or reuses the transpose metadata (blksprs/ops/transpose.py:63-88)."""
    layout_cache = prepare_layout_cache(layout_cache, "transpose", sparsity_layout)

    if "sparsity_layout_t" not in layout_cache:
        layout_t = as_base_tensor(sparsity_layout.transpose(-1, -2).contiguous())
        if layout_t.data_ptr() == sparsity_layout.data_ptr():
            layout_t = layout_t.clone()  # the derived layout never aliases its source
        layout_cache["sparsity_layout_t"] = layout_t
    if "n_sparse_blocks" not in layout_cache:
        layout_cache["n_sparse_blocks"] = count_active_blocks(sparsity_layout)
    if "layout_indices" not in layout_cache:
        layout_cache["layout_indices"] = build_layout_indices(layout_cache["sparsity_layout_t"],
                                                              layout_cache["n_sparse_blocks"])
    if "packed_indices" not in layout_cache:
        # reverse LUT of the source layout, viewed at transposed coordinates
        layout_cache["packed_indices"] = (build_packed_indices(sparsity_layout)
                                          .reshape(sparsity_layout.size()).transpose(-1, -2).contiguous().reshape(-1))
    if _SRC not in layout_cache:
        lut = layout_cache["layout_indices"]
        _, rows_t, cols_t = layout_cache["sparsity_layout_t"].shape
        flat = (lut[:, 0] * rows_t + lut[:, 1]) * cols_t + lut[:, 2]
        layout_cache[_SRC] = layout_cache["packed_indices"][flat].contiguous()

    validate_contiguous(layout_cache["sparsity_layout_t"], layout_cache["layout_indices"],
                        layout_cache["packed_indices"])
    return finalize_layout_cache(layout_cache)


def _transpose_blocks(x: Tensor, source_blocks: Tensor, n_out: int, bs: int) -> Tensor:
    out = torch.empty((n_out, bs, bs), dtype=x.dtype, device=x.device)
    if n_out:
        with torch.cuda.device(x.device):
            _cabi.check(_cabi.lib().bsp_transpose_blocks(
                _cabi.ptr(x), x.size(0), _cabi.ptr(out), n_out, _cabi.ptr(source_blocks), bs, x.element_size(),
                _cabi.stream_handle(x.device)), "bsp_transpose_blocks")
    return out


class _BlockSparseTranspose(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, source_blocks: Tensor, n_out: int, bs: int, layout_t: Tensor):
        ctx.layout_t = layout_t
        ctx.sparsity_block_size = bs
        return _transpose_blocks(x, source_blocks, n_out, bs)

    @staticmethod
    @torch.autograd.function.once_differentiable
    @plain_dispatch
    def backward(ctx, grad_output: Tensor):
        grad, _ = transpose(grad_output.contiguous(), ctx.layout_t, ctx.sparsity_block_size)
        return Tensor(grad), None, None, None, None


@torch.compiler.disable
@plain_dispatch
def _transpose_eager(x, sparsity_layout, sparsity_block_size, layout_cache):
    x = ensure_contiguous(x)

    validate_dimensions(x)
    validate_contiguous(x)
    validate_dtype_supported(x)
    validate_device(x)
    validate_sparsity(sparsity_block_size, (x, sparsity_layout))
    validate_sparsity_block_size(sparsity_block_size, x)

    layout_cache = transpose_build_layout_cache(layout_cache, sparsity_layout)
    out = _BlockSparseTranspose.apply(x, layout_cache[_SRC], layout_cache["n_sparse_blocks"],
                                      sparsity_block_size, layout_cache["sparsity_layout_t"])
    return BlksprsTensor.wrap(out), layout_cache["sparsity_layout_t"]


@torch.amp.custom_fwd(device_type="cuda")
def transpose(x: BlksprsTensor, sparsity_layout: Tensor,
              sparsity_block_size: int, layout_cache: dict | None = None) -> tuple[BlksprsTensor, Tensor]:
    """Transposes a block-sparse tensor in compressed form.

    Args:
        x (BlksprsTensor): The compressed input tensor.
        sparsity_layout (Tensor): The sparsity layout of ``x``.
        sparsity_block_size (int): The size of the sparsity blocks.
        layout_cache (dict, optional): Reusable layout metadata cache (default ``None``).

    Returns:
        tuple[BlksprsTensor, Tensor]: The transposed tensor in compressed form and its sparsity layout.
    """
    return _transpose_eager(x, sparsity_layout, sparsity_block_size, layout_cache)
