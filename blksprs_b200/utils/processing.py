"""``apply_torch_linear`` / ``apply_torch_linear_cached``: a ``torch.nn.Linear`` applied to a compressed tensor.

Same signatures, validation errors, results and gradients as the reference helpers
(blksprs/utils/processing.py:26-202); the work is organised differently:

* The reference copies the transposed weight once per batch entry and multiplies batch by batch
  (processing.py:48-52, 137-148).  A linear layer treats every row alike, so the input layout
  ``(B, R, K)`` is read here as ``(1, B*R, K)`` — the compressed tensor is the same, block for
  block — and multiplied with ONE copy of the weight blocks, layout ``(1, K, N)``.  The cache
  entries ``sparsity_layout_w_t`` / ``w_t_bs`` therefore hold one batch entry, not ``B``.
* The weight gradient contracts over all ``B*R`` block rows.  To keep every SM busy the rows are
  cut into ``S`` chunks that are multiplied side by side (layouts ``(S, B*R/S, ·)``) and folded in
  fp32 by ``bsp_sum_chunks``; the reference's equivalent is the sum over the batch copies.
* The bias stays a vector: the tcgen05 kernel adds it to the accumulators in its epilogue (behind
  the mma.sync kernel ``bsp_bias_add`` adds it in place); its gradient is one column sum
  (``bsp_bias_grad``).  The reference builds a compressed copy of the bias per output block
  (processing.py:72-84).
"""
from __future__ import annotations

import torch
from torch import Tensor, nn

from .. import _cabi
from ..plan import Product
from .blksprs_tensor import BlksprsTensor
from .tools import build_layout_indices, build_packed_indices, cast_for_autocast, count_active_blocks, \
    finalize_layout_cache, plain_dispatch, prepare_layout_cache
from .validation import ensure_contiguous, validate_contiguous, validate_device, validate_dimensions, \
    validate_dtype_float, validate_sparsity, validate_sparsity_block_size, validation_enabled

_PLANS = "_b200_linear_plans"

# The chunked weight-gradient product should have at least this many output blocks.
_MIN_GRAD_W_BLOCKS = 2048


def _validate_linear_dtypes(x: Tensor, weight: Tensor, bias: Tensor | None) -> None:
    tensors = (x, weight) if bias is None else (x, weight, bias)
    if torch.is_autocast_enabled():
        for tensor in tensors:
            validate_dtype_float(tensor)
    else:
        validate_dtype_float(*tensors)


def _chunk_count(rows: int, weight_blocks: int) -> int:
    """Smallest divisor ``S`` of ``rows`` with ``S * weight_blocks >= _MIN_GRAD_W_BLOCKS`` (``rows`` itself if none)."""
    if rows <= 1 or weight_blocks <= 0 or weight_blocks >= _MIN_GRAD_W_BLOCKS:
        return 1
    want = -(-_MIN_GRAD_W_BLOCKS // weight_blocks)
    for s in range(want, rows + 1):
        if rows % s == 0:
            return s
    return rows


class _LinearPlans:
    """Plans of the three products of one (input layout, output layout, weight shape) combination."""

    def __init__(self, sparsity_layout: Tensor, sparsity_layout_output: Tensor, k_blocks: int, n_blocks: int):
        B, R, K = sparsity_layout.shape
        if K != k_blocks:
            raise ValueError("Inner dimensions of tensors must match")
        device = sparsity_layout.device
        self.rows, self.K, self.N = B * R, K, n_blocks
        self.layout_x = sparsity_layout.contiguous().reshape(1, self.rows, K)
        self.layout_o = sparsity_layout_output.contiguous().reshape(1, self.rows, n_blocks)
        self.layout_w = torch.ones((1, K, n_blocks), dtype=torch.bool, device=device)
        self.packed_x = build_packed_indices(self.layout_x)
        self.packed_w = build_packed_indices(self.layout_w)
        self.n_x = count_active_blocks(self.layout_x)
        self.n_o = count_active_blocks(self.layout_o)
        self.lut_o = build_layout_indices(self.layout_o, self.n_o)
        self.forward = Product(_cabi.OP_NN, self.lut_o, self.packed_x, self.packed_w, self.rows, K, n_blocks)
        self.grad_x: Product | None = None
        self.grad_w: Product | None = None
        self.packed_o: Tensor | None = None
        self.chunks = 1

    def backward_plans(self) -> None:
        if self.grad_x is not None:
            return
        self.packed_o = build_packed_indices(self.layout_o)
        lut_x = build_layout_indices(self.layout_x, self.n_x)
        self.grad_x = Product(_cabi.OP_NT, lut_x, self.packed_o, self.packed_w, self.rows, self.K, self.N)
        self.chunks = _chunk_count(self.rows, self.K * self.N)
        layout_w_chunks = torch.ones((self.chunks, self.K, self.N), dtype=torch.bool, device=self.layout_w.device)
        lut_w = build_layout_indices(layout_w_chunks, self.chunks * self.K * self.N)
        self.grad_w = Product(_cabi.OP_TN, lut_w, self.packed_x, self.packed_o, self.rows // self.chunks,
                              self.K, self.N)


def _bias_gradient(grad_output: Tensor, lut_o: Tensor, bs: int, n_cols: int) -> Tensor:
    grad = torch.zeros(n_cols, dtype=torch.float32, device=grad_output.device)
    grad_output = _cabi.aligned(grad_output)
    if grad_output.size(0):
        with torch.cuda.device(grad_output.device):
            _cabi.check(_cabi.lib().bsp_bias_grad(
                _cabi.ptr(grad_output), _cabi.ptr(lut_o), grad_output.size(0), bs,
                _cabi.DATA_DTYPE_CODES[grad_output.dtype], _cabi.ptr(grad), n_cols,
                _cabi.stream_handle(grad_output.device)), "bsp_bias_grad")
    return grad


def _fold_chunks(parts: Tensor, chunks: int) -> Tensor:
    if chunks == 1:
        return parts
    n = parts.size(0) // chunks
    out = torch.empty((n, parts.size(1), parts.size(2)), dtype=parts.dtype, device=parts.device)
    if out.numel():
        with torch.cuda.device(parts.device):
            _cabi.check(_cabi.lib().bsp_sum_chunks(
                _cabi.ptr(parts), chunks, out.numel(), _cabi.DATA_DTYPE_CODES[parts.dtype], _cabi.ptr(out),
                _cabi.stream_handle(parts.device)), "bsp_sum_chunks")
    return out


class _SparseLinear(torch.autograd.Function):
    """``x @ w_t (+ bias)`` on compressed blocks; differentiable in ``x``, ``w_t`` and ``bias``."""

    @staticmethod
    def forward(ctx, x: Tensor, w_t: Tensor, bias: Tensor | None, plans: _LinearPlans, bs: int):
        ctx.save_for_backward(x, w_t)
        ctx.plans, ctx.sparsity_block_size = plans, bs
        ctx.bias_cols = None if bias is None else bias.numel()
        return plans.forward.run(x, w_t, bs, bias)

    @staticmethod
    @torch.autograd.function.once_differentiable
    @plain_dispatch
    def backward(ctx, grad_output: Tensor):
        x, w_t = ctx.saved_tensors
        plans: _LinearPlans = ctx.plans
        bs = ctx.sparsity_block_size
        grad_output = grad_output.contiguous()
        if grad_output.dtype != x.dtype:
            grad_output = grad_output.to(x.dtype)
        plans.backward_plans()
        grad_x = plans.grad_x.run(grad_output, w_t, bs) if ctx.needs_input_grad[0] else None
        grad_w = None
        if ctx.needs_input_grad[1]:
            grad_w = _fold_chunks(plans.grad_w.run(x, grad_output, bs), plans.chunks)
        grad_b = None
        if ctx.bias_cols is not None and ctx.needs_input_grad[2]:
            grad_b = _bias_gradient(grad_output, plans.lut_o, bs, ctx.bias_cols).to(x.dtype)
        return grad_x, grad_w, grad_b, None, None


def _output_layout(sparsity_layout: Tensor, n_blocks: int, has_bias: bool) -> Tensor:
    """``(B, R, N)`` bool: every block when there is a bias (it makes every output block non-zero),
    else the rows of the input that hold a block (the reference's
    ``build_sparsity_layout_matmul_fast`` against an all-ones weight layout, processing.py:56-64)."""
    B, R, _ = sparsity_layout.shape
    if has_bias:
        return torch.ones((B, R, n_blocks), dtype=torch.bool, device=sparsity_layout.device)
    from ..layouting.sparsity_layout import build_sparsity_layout_matmul_fast
    weight_layout = torch.ones((B, sparsity_layout.size(2), n_blocks), dtype=torch.bool,
                               device=sparsity_layout.device)
    return build_sparsity_layout_matmul_fast(sparsity_layout, weight_layout)


def _compress_weight(w: Tensor, layout_w_t: Tensor, bs: int, layout_cache: dict | None) -> Tensor:
    from ..ops.conversion import to_sparse_shaped
    w_t_dense = w.transpose(-1, -2).unsqueeze(0).contiguous()
    return to_sparse_shaped(w_t_dense, layout_w_t, bs, layout_cache=layout_cache)


def _run(x: Tensor, sparsity_layout: Tensor, bs: int, w_t_bs: Tensor, b: Tensor | None, plans: _LinearPlans):
    x = ensure_contiguous(x)
    x, w_t = cast_for_autocast(x, w_t_bs.to(x.dtype))
    validate_dimensions(x)
    validate_contiguous(x)
    validate_dtype_float(x, w_t)
    validate_device(x, w_t, sparsity_layout)
    validate_sparsity(bs, (x, sparsity_layout), counts=(plans.n_x,))
    bias = None if b is None else b.to(x.dtype).contiguous()
    out = _SparseLinear.apply(x, w_t.as_subclass(Tensor).contiguous(), bias, plans, bs)
    return BlksprsTensor.wrap(out)


@torch.compiler.disable
@plain_dispatch
def _apply_eager(x, sparsity_layout, sparsity_block_size, linear, bias, layout_cache, cached: bool):
    w = linear.weight
    b = bias if bias is not None else linear.bias
    _validate_linear_dtypes(x, w, b)
    validate_sparsity_block_size(sparsity_block_size, w)
    k_blocks, n_blocks = w.size(1) // sparsity_block_size, w.size(0) // sparsity_block_size
    if b is not None and validation_enabled() and b.numel() != w.size(0):
        raise ValueError("Tensor sizes must be divisible by sparsity block size")

    if not cached:
        layout_w_t = torch.ones((1, k_blocks, n_blocks), dtype=torch.bool, device=x.device)
        w_t_bs = _compress_weight(w, layout_w_t, sparsity_block_size, None)
        layout_output = _output_layout(sparsity_layout, n_blocks, b is not None)
        plans = _LinearPlans(sparsity_layout, layout_output, k_blocks, n_blocks)
        return _run(x, sparsity_layout, sparsity_block_size, w_t_bs, b, plans), layout_output

    layout_cache = prepare_layout_cache(layout_cache, "apply_torch_linear", sparsity_layout, sparsity_block_size,
                                        x.device, x.dtype, torch.is_grad_enabled(), w, b)
    if "sparsity_layout_w_t" not in layout_cache:
        layout_cache["sparsity_layout_w_t"] = torch.ones((1, k_blocks, n_blocks), dtype=torch.bool, device=x.device)
    if "w_t_bs" not in layout_cache:
        layout_cache["w_t_bs"] = _compress_weight(w, layout_cache["sparsity_layout_w_t"], sparsity_block_size,
                                                  layout_cache.setdefault("weight_layout_cache", dict()))
    if "sparsity_layout_output" not in layout_cache:
        layout_cache["sparsity_layout_output"] = _output_layout(sparsity_layout, n_blocks, b is not None)
    if _PLANS not in layout_cache:
        layout_cache[_PLANS] = _LinearPlans(sparsity_layout, layout_cache["sparsity_layout_output"], k_blocks,
                                            n_blocks)
    out = _run(x, sparsity_layout, sparsity_block_size, layout_cache["w_t_bs"], b, layout_cache[_PLANS])
    output_layout = layout_cache["sparsity_layout_output"]
    finalize_layout_cache(layout_cache)
    return out, output_layout


@torch.amp.custom_fwd(device_type="cuda")
def apply_torch_linear(x: BlksprsTensor, sparsity_layout: Tensor, sparsity_block_size: int,
                       linear: nn.Linear, bias: nn.Parameter | None = None) -> tuple[BlksprsTensor, Tensor]:
    """Applies a PyTorch linear layer to a block-sparse tensor.

    Args:
        x (BlksprsTensor): The compressed input tensor.
        sparsity_layout (Tensor): The sparsity layout of ``x``.
        sparsity_block_size (int): The size of the sparsity blocks.
        linear (nn.Linear): The linear layer to apply.
        bias (nn.Parameter, optional): An explicit bias overriding ``linear.bias`` (default ``None``).

    Returns:
        tuple[BlksprsTensor, Tensor]: The projected tensor in compressed form and its sparsity layout.
    """
    return _apply_eager(x, sparsity_layout, sparsity_block_size, linear, bias, None, False)


@torch.amp.custom_fwd(device_type="cuda")
def apply_torch_linear_cached(x: BlksprsTensor, sparsity_layout: Tensor, sparsity_block_size: int,
                              linear: nn.Linear, bias: nn.Parameter | None = None,
                              layout_cache: dict | None = None) -> tuple[BlksprsTensor, Tensor]:
    """Applies a PyTorch linear layer while caching its compressed parameters.

    Args:
        x (BlksprsTensor): The compressed input tensor.
        sparsity_layout (Tensor): The sparsity layout of ``x``.
        sparsity_block_size (int): The size of the sparsity blocks.
        linear (nn.Linear): The linear layer to apply.
        bias (nn.Parameter, optional): An explicit bias overriding ``linear.bias`` (default ``None``).
        layout_cache (dict, optional): Reusable layout and parameter cache (default ``None``).

    Returns:
        tuple[BlksprsTensor, Tensor]: The projected tensor in compressed form and its sparsity layout.
    """
    return _apply_eager(x, sparsity_layout, sparsity_block_size, linear, bias, layout_cache, True)
