"""Dense <-> compressed conversion: ``to_sparse`` / ``to_dense`` and their aliases.

Same signatures, cache entries, autograd behaviour and results as the reference
(blksprs/ops/conversion.py:17-56, 158-305, 307-349, 429-621).  Each direction is one pass of a
copy kernel of the native library (``bsp_to_sparse`` / ``bsp_to_dense``); ``to_dense`` writes
the fill value and the blocks in the same pass instead of ``torch.full`` followed by a scatter.
"""
from __future__ import annotations

import struct

import torch
from torch import Tensor

from .. import _cabi
from ..utils.blksprs_tensor import BlksprsTensor
from ..utils.tools import build_layout_indices, build_packed_indices, \
    finalize_layout_cache, plain_dispatch, prepare_layout_cache
from ..utils.validation import ensure_contiguous, validate_contiguous, validate_device, validate_dimensions, \
    validate_dtype_supported, validate_sparsity, validate_sparsity_block_size, validate_sparsity_dense

_PACK = {torch.float16: "<e", torch.float32: "<f", torch.float64: "<d", torch.int8: "<b", torch.uint8: "<B",
         torch.int16: "<h", torch.int32: "<i", torch.int64: "<q", torch.bool: "<?"}


def _fill_bits(fill_value, dtype: torch.dtype) -> int:
    """Bit pattern of ``fill_value`` converted to ``dtype`` (as ``torch.full`` would convert it)."""
    if dtype == torch.bfloat16:
        raw = struct.pack("<f", float(torch.tensor(fill_value, dtype=torch.bfloat16).float()))
        return int.from_bytes(raw[2:], "little")
    value = torch.tensor(fill_value, dtype=dtype).item()
    return int.from_bytes(struct.pack(_PACK[dtype], value), "little")


def to_sparse_build_layout_cache(layout_cache: dict | None, sparsity_layout: Tensor) -> dict:
    layout_cache = prepare_layout_cache(layout_cache, "to_sparse", sparsity_layout)
    if "layout_indices" not in layout_cache:
        layout_cache["layout_indices"] = build_layout_indices(sparsity_layout, layout_cache.get("n_sparse_blocks"))
    if "n_sparse_blocks" not in layout_cache:
        layout_cache["n_sparse_blocks"] = layout_cache["layout_indices"].size(0)
    validate_contiguous(sparsity_layout, layout_cache["layout_indices"])
    return finalize_layout_cache(layout_cache)


def to_dense_build_layout_cache(layout_cache: dict | None, sparsity_layout: Tensor) -> dict:
    layout_cache = prepare_layout_cache(layout_cache, "to_dense", sparsity_layout)
    if "packed_indices" not in layout_cache:
        layout_cache["packed_indices"] = build_packed_indices(sparsity_layout)
    validate_contiguous(layout_cache["packed_indices"])
    return finalize_layout_cache(layout_cache)


def _gather_blocks(x: Tensor, layout_indices: Tensor, n_blocks: int, bs: int) -> Tensor:
    out = torch.empty((n_blocks, bs, bs), dtype=x.dtype, device=x.device)
    if n_blocks:
        with torch.cuda.device(x.device):
            _cabi.check(_cabi.lib().bsp_to_sparse(
                _cabi.ptr(x), x.size(0), x.size(1), x.size(2), _cabi.ptr(layout_indices), n_blocks, bs,
                x.element_size(), _cabi.ptr(out), _cabi.stream_handle(x.device)), "bsp_to_sparse")
    return out


def _scatter_blocks(x: Tensor, packed_indices: Tensor, layout_shape, bs: int, fill_value) -> Tensor:
    B, R, C = layout_shape
    out = torch.empty((B, R * bs, C * bs), dtype=x.dtype, device=x.device)
    if out.numel():
        with torch.cuda.device(x.device):
            _cabi.check(_cabi.lib().bsp_to_dense(
                _cabi.ptr(x), x.size(0), _cabi.ptr(packed_indices), B, R, C, bs, x.element_size(),
                _fill_bits(fill_value, x.dtype), _cabi.ptr(out), _cabi.stream_handle(x.device)), "bsp_to_dense")
    return out


class _ToSparse(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, sparsity_layout: Tensor, layout_indices: Tensor, bs: int, n_blocks: int):
        ctx.sparsity_layout, ctx.sparsity_block_size = sparsity_layout, bs
        return _gather_blocks(x, layout_indices, n_blocks, bs)

    @staticmethod
    @torch.autograd.function.once_differentiable
    @plain_dispatch
    def backward(ctx, grad_output: Tensor):
        # the scatter itself: the gradient's shape is the output's, so the op's input checks (and the
        # device reads they need) have nothing to find
        layout = ctx.sparsity_layout
        grad = _scatter_blocks(grad_output.contiguous(), build_packed_indices(layout), layout.shape,
                               ctx.sparsity_block_size, 0)
        return grad, None, None, None, None


class _ToDense(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, sparsity_layout: Tensor, packed_indices: Tensor, bs: int, fill_value):
        ctx.sparsity_layout, ctx.sparsity_block_size, ctx.n_blocks = sparsity_layout, bs, x.size(0)
        return _scatter_blocks(x, packed_indices, sparsity_layout.shape, bs, fill_value)

    @staticmethod
    @torch.autograd.function.once_differentiable
    @plain_dispatch
    def backward(ctx, grad_output: Tensor):
        # the gather itself; the number of blocks is the forward input's, no device read needed
        layout = ctx.sparsity_layout
        lut = build_layout_indices(layout, ctx.n_blocks)
        grad = _gather_blocks(grad_output.contiguous(), lut, ctx.n_blocks, ctx.sparsity_block_size)
        return grad, None, None, None, None


def _single_full_block(sparsity_layout: Tensor) -> bool:
    return sparsity_layout.size(1) == 1 and sparsity_layout.size(2) == 1 and bool(torch.all(sparsity_layout))


@torch.compiler.disable
@plain_dispatch
def _to_sparse_eager(x, sparsity_layout, sparsity_block_size, layout_cache):
    x = ensure_contiguous(x)
    validate_dimensions(x)
    validate_contiguous(x)
    validate_device(x)
    validate_dtype_supported(x)
    validate_sparsity_dense(sparsity_block_size, (x, sparsity_layout))
    validate_sparsity_block_size(sparsity_block_size, x)
    layout_cache = to_sparse_build_layout_cache(layout_cache, sparsity_layout)
    if _single_full_block(sparsity_layout):
        return BlksprsTensor.wrap(x)
    return BlksprsTensor.wrap(_ToSparse.apply(x, sparsity_layout, layout_cache["layout_indices"],
                                              sparsity_block_size, layout_cache["n_sparse_blocks"]))


@torch.compiler.disable
@plain_dispatch
def _to_dense_eager(x, sparsity_layout, sparsity_block_size, fill_value, layout_cache):
    x = ensure_contiguous(x)
    validate_dimensions(x)
    validate_contiguous(x, sparsity_layout)
    validate_device(x)
    validate_dtype_supported(x)
    validate_sparsity(sparsity_block_size, (x, sparsity_layout))
    validate_sparsity_block_size(sparsity_block_size, x)
    layout_cache = to_dense_build_layout_cache(layout_cache, sparsity_layout)
    if _single_full_block(sparsity_layout):
        return x.as_subclass(Tensor)
    out = _ToDense.apply(x, sparsity_layout, layout_cache["packed_indices"], sparsity_block_size, fill_value)
    return out.as_subclass(Tensor)


@torch.amp.custom_fwd(device_type="cuda")
def to_sparse(x: Tensor, sparsity_layout: Tensor,
              sparsity_block_size: int, layout_cache: dict | None = None) -> BlksprsTensor:
    """Converts a three-dimensional dense tensor to compressed block-sparse form.

    Args:
        x (Tensor): The dense input tensor.
        sparsity_layout (Tensor): The sparsity layout of ``x``.
        sparsity_block_size (int): The size of the sparsity blocks.
        layout_cache (dict, optional): Reusable layout metadata cache (default ``None``).

    Returns:
        BlksprsTensor: ``x`` in compressed form.
    """
    return _to_sparse_eager(x, sparsity_layout, sparsity_block_size, layout_cache)


@torch.amp.custom_fwd(device_type="cuda")
def to_dense(x: BlksprsTensor, sparsity_layout: Tensor,
             sparsity_block_size: int, fill_value: float = 0, layout_cache: dict | None = None) -> Tensor:
    """Converts a compressed block-sparse tensor to three-dimensional dense form.

    Args:
        x (BlksprsTensor): The compressed input tensor.
        sparsity_layout (Tensor): The sparsity layout of ``x``.
        sparsity_block_size (int): The size of the sparsity blocks.
        fill_value (float, optional): The value used for inactive blocks (default ``0``).
        layout_cache (dict, optional): Reusable layout metadata cache (default ``None``).

    Returns:
        Tensor: ``x`` in three-dimensional dense form.
    """
    return _to_dense_eager(x, sparsity_layout, sparsity_block_size, fill_value, layout_cache)


def to_blksprs(x: Tensor, sparsity_layout: Tensor, sparsity_block_size: int,
               layout_cache: dict | None = None) -> BlksprsTensor:
    """Alias of :func:`to_sparse`."""
    return to_sparse(x, sparsity_layout, sparsity_block_size, layout_cache=layout_cache)


def to_sparse_shaped(x: Tensor, sparsity_layout: Tensor, sparsity_block_size: int,
                     layout_cache: dict | None = None) -> BlksprsTensor:
    """Alias of :func:`to_sparse` for inputs that already are ``(B, rows, cols)``."""
    return to_sparse(x, sparsity_layout, sparsity_block_size, layout_cache=layout_cache)


def from_blksprs(x: BlksprsTensor, sparsity_layout: Tensor, sparsity_block_size: int,
                 fill_value: float = 0, layout_cache: dict | None = None) -> Tensor:
    """Alias of :func:`to_dense`."""
    return to_dense(x, sparsity_layout, sparsity_block_size, fill_value=fill_value, layout_cache=layout_cache)


def to_dense_shaped(x: BlksprsTensor, sparsity_layout: Tensor, sparsity_block_size: int,
                    fill_value: float = 0, layout_cache: dict | None = None) -> Tensor:
    """Alias of :func:`to_dense` returning the ``(B, rows, cols)`` tensor."""
    return to_dense(x, sparsity_layout, sparsity_block_size, fill_value=fill_value, layout_cache=layout_cache)
