"""Scaled block-sparse matmul with the row-wise softmax fused behind it.

``matmul_softmax(x, sl_x, y, sl_y, sl_o, bs, scale)`` returns
``softmax(scale * matmul(x, y))`` over the active blocks of each output row, optionally in another
dtype.  It equals the chain of three reference ops used for attention by parts
(test/cases/test_blocksparse.py:1517-1529): ``matmul`` (blksprs/ops/matmul.py:17-67), a
multiplication by ``scale``, and ``softmax`` (blksprs/ops/softmax.py:23-144; inactive blocks count as
``-inf``), followed by a cast.  The reference has no single call for it, and its softmax takes fp32
only, so its chain writes the scores, reads them for the cast, and sweeps them several more times.

Here the scores never leave the matmul kernel as such: its epilogue scales the fp32 accumulators,
takes the maximum ``m`` of every matrix row inside the block, and writes ``exp(s - m)`` in the
operands' dtype together with ``(m, sum)`` per row and block (8 bytes per ``bs`` elements).  A
second light pass (``bsp_softmax_normalize``) reads each element once, rescales it with the
row-wide maximum and sum, and writes the probabilities in ``out_dtype``.  For block sizes 16 and 32
(no tensor-memory kernel) the op runs the mma.sync product and one softmax pass that scales, reads the
scores in their dtype and writes ``out_dtype`` (``bsp_softmax_fwd_scaled``).
"""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _cabi
from ..plan import status_word
from ..utils.blksprs_tensor import BlksprsTensor
from ..utils.tools import build_packed_indices, cast_for_autocast, implicit_layout_cache, layout_cache_is_current, \
    plain_dispatch
from ..utils.validation import ensure_contiguous, validation_enabled
from .matmul import _PLANS, _MatmulPlans, _backward_plans, _validate_cold, _validate_warm, \
    matmul_build_layout_cache

_OUT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def _row_first(plans: _MatmulPlans) -> Tensor:
    """int32 ``(B * R + 1)``: index of the first compressed block of every block row of the output
    layout (the blocks of a block row are consecutive: the LUT order is batch, row, column)."""
    cached = getattr(plans, "row_first_o", None)
    if cached is None:
        sl_o = plans.layouts[2]
        per_row = (sl_o.reshape(-1, sl_o.size(-1)) != 0).sum(dim=1, dtype=torch.int64)
        cached = torch.zeros(per_row.numel() + 1, dtype=torch.int32, device=sl_o.device)
        cached[1:] = torch.cumsum(per_row, 0).to(torch.int32)
        plans.row_first_o = cached
    return cached


def _softmax_rows(scores: Tensor, plans: _MatmulPlans, bs: int) -> Tensor:
    """fp32 row-wise softmax over the active blocks (the stand-alone kernel)."""
    if plans.packed_o is None:
        plans.packed_o = build_packed_indices(plans.layouts[2])
    B, R, C = plans.layouts[2].shape
    out = torch.empty_like(scores)
    with _cabi.device_guard(scores.device):
        _cabi.check(_cabi.lib().bsp_softmax_fwd(_cabi.ptr(scores), scores.size(0), _cabi.ptr(plans.packed_o), B, R, C,
                                                bs, _cabi.ptr(out), _cabi.stream_handle(scores.device)),
                    "bsp_softmax_fwd")
    return out


def _forward(x: Tensor, y: Tensor, plans: _MatmulPlans, bs: int, scale: float, out_dtype: torch.dtype) -> Tensor:
    product = plans.forward
    n_out = product.n_out
    device = x.device
    if n_out == 0:
        return torch.empty((0, bs, bs), dtype=out_dtype, device=device)
    kernel, width = product.choose(bs, x.dtype, x.size(0), y.size(0))
    if kernel != "umma":
        # mma.sync product, then scale, softmax and cast in one pass over the scores
        scores = product.run(x, y, bs)
        if plans.packed_o is None:
            plans.packed_o = build_packed_indices(plans.layouts[2])
        B, R, C = plans.layouts[2].shape
        out = torch.empty((n_out, bs, bs), dtype=out_dtype, device=device)
        with _cabi.device_guard(device):
            status = _cabi.lib().bsp_softmax_fwd_scaled(
                scores.data_ptr(), _cabi.DATA_DTYPE_CODES[scores.dtype], n_out, plans.packed_o.data_ptr(), B, R, C, bs,
                float(scale), out.data_ptr(), _cabi.DATA_DTYPE_CODES[out_dtype], _cabi.stream_handle(device))
        if status == _cabi.ERR_UNSUPPORTED:
            # very wide layouts: separate steps around the general fp32 softmax kernel
            scores = scores.float()
            if scale != 1.0:
                scores = scores * scale
            return _softmax_rows(scores, plans, bs).to(out_dtype)
        _cabi.check(status, "bsp_softmax_fwd_scaled")
        return out
    sp = product.step_plan(bs, x.dtype, width)
    x, y = _cabi.aligned(x), _cabi.aligned(y)
    e = torch.empty((n_out, bs, bs), dtype=x.dtype, device=device)
    stats = torch.empty((n_out, bs, 2), dtype=torch.float32, device=device)
    out = torch.empty((n_out, bs, bs), dtype=out_dtype, device=device)
    row_first = _row_first(plans)
    lib = _cabi.lib()
    with _cabi.device_guard(device):
        stream = _cabi.stream_handle(device)
        _cabi.check(lib.bsp_matmul_umma_softmax(
            x.data_ptr(), x.size(0), y.data_ptr(), y.size(0), e.data_ptr(), n_out, stats.data_ptr(), float(scale),
            *sp.launch_args(), sp.sched_ptr(stream), sp.width, bs, _cabi.DATA_DTYPE_CODES[x.dtype],
            status_word(device).data_ptr(), stream), "bsp_matmul_umma_softmax")
        _cabi.check(lib.bsp_softmax_normalize(
            e.data_ptr(), _cabi.DATA_DTYPE_CODES[x.dtype], stats.data_ptr(), n_out, row_first.data_ptr(),
            row_first.numel() - 1, bs, out.data_ptr(), _cabi.DATA_DTYPE_CODES[out_dtype], stream),
            "bsp_softmax_normalize")
    return out


class _MatmulSoftmax(torch.autograd.Function):
    """Differentiable in ``x`` and ``y``.  With P the result and S the scaled scores:
    dS = P * (dP - rowsum(dP * P)), dX = scale * dS Y^T, dY = scale * X^T dS."""

    @staticmethod
    def forward(ctx, x: Tensor, y: Tensor, packed_x: Tensor, packed_y: Tensor, plans: _MatmulPlans, bs: int,
                scale: float, out_dtype: torch.dtype):
        out = _forward(x, y, plans, bs, scale, out_dtype)
        ctx.save_for_backward(x, y, packed_x, packed_y, out)
        ctx.plans, ctx.sparsity_block_size, ctx.scale = plans, bs, scale
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    @plain_dispatch
    def backward(ctx, grad_output: Tensor):
        x, y, packed_x, packed_y, out = ctx.saved_tensors
        plans: _MatmulPlans = ctx.plans
        bs = ctx.sparsity_block_size
        _backward_plans(plans, packed_x, packed_y, x.size(0), y.size(0))
        B, R, C = plans.layouts[2].shape
        grad = _cabi.aligned(grad_output.contiguous())
        if grad.dtype not in _OUT_DTYPES:
            grad = grad.to(torch.float32)
        n_out = out.size(0)
        # dS, the scale and the cast to the operands' dtype in one pass over probabilities and their gradient
        grad_scores = torch.empty((n_out, bs, bs), dtype=x.dtype, device=out.device)
        status = _cabi.OK
        if n_out:
            with _cabi.device_guard(out.device):
                status = _cabi.lib().bsp_softmax_bwd_scaled(
                    grad.data_ptr(), _cabi.DATA_DTYPE_CODES[grad.dtype], out.data_ptr(), _cabi.DATA_DTYPE_CODES[out.dtype],
                    n_out, plans.packed_o.data_ptr(), B, R, C, bs, float(ctx.scale), grad_scores.data_ptr(),
                    _cabi.DATA_DTYPE_CODES[x.dtype], _cabi.stream_handle(out.device))
        if status == _cabi.ERR_UNSUPPORTED:
            # very wide layouts: separate steps around the general fp32 kernel
            probs, grad = out.to(torch.float32), grad.to(torch.float32)
            grad_scores = torch.empty_like(probs)
            with _cabi.device_guard(probs.device):
                _cabi.check(_cabi.lib().bsp_softmax_bwd(_cabi.ptr(grad), _cabi.ptr(probs), probs.size(0),
                                                        _cabi.ptr(plans.packed_o), B, R, C, bs, _cabi.ptr(grad_scores),
                                                        _cabi.stream_handle(probs.device)), "bsp_softmax_bwd")
            if ctx.scale != 1.0:
                grad_scores = grad_scores * ctx.scale
            grad_scores = grad_scores.to(x.dtype)
        else:
            _cabi.check(status, "bsp_softmax_bwd_scaled")
        grad_x = plans.grad_x.run(grad_scores, y, bs) if ctx.needs_input_grad[0] else None
        grad_y = plans.grad_y.run(x, grad_scores, bs) if ctx.needs_input_grad[1] else None
        return grad_x, grad_y, None, None, None, None, None, None


@torch.compiler.disable
@plain_dispatch
def _matmul_softmax_eager(x, sparsity_layout_x, y, sparsity_layout_y, sparsity_layout_output, sparsity_block_size,
                          scale, out_dtype, layout_cache):
    x, y = ensure_contiguous(x, y)
    x, y = cast_for_autocast(x, y)
    if out_dtype is None:
        out_dtype = x.dtype
    if out_dtype not in _OUT_DTYPES:
        raise ValueError("Output dtype must be float16, bfloat16, or float32")
    if layout_cache is None:
        # no caller-owned cache: a small library-owned one, with the same reuse rule (tools.implicit_layout_cache)
        layout_cache = implicit_layout_cache("matmul", sparsity_layout_x, sparsity_layout_y, sparsity_layout_output)
    plans = None
    if layout_cache_is_current(layout_cache, "matmul", sparsity_layout_x, sparsity_layout_y, sparsity_layout_output):
        plans = layout_cache.get(_PLANS)
    if plans is not None and plans.forward is not None and (plans.layouts_validated or not validation_enabled()):
        if validation_enabled():
            _validate_warm(x, y, plans, sparsity_block_size)
    else:
        checked = validation_enabled()
        if checked:
            _validate_cold(x, sparsity_layout_x, y, sparsity_layout_y, sparsity_layout_output, sparsity_block_size)
        layout_cache = matmul_build_layout_cache(layout_cache, sparsity_layout_x, sparsity_layout_y,
                                                 sparsity_layout_output)
        plans = layout_cache[_PLANS]
        if checked:
            plans.n_x, plans.n_y = x.size(0), y.size(0)
            plans.layouts_validated = True
    if torch.is_grad_enabled() and (x.requires_grad or y.requires_grad):
        out = _MatmulSoftmax.apply(x, y, layout_cache["packed_indices_x"], layout_cache["packed_indices_y"], plans,
                                   sparsity_block_size, float(scale), out_dtype)
    else:
        out = _forward(x, y, plans, sparsity_block_size, float(scale), out_dtype)
    return BlksprsTensor.wrap(out)


@torch.amp.custom_fwd(device_type="cuda")
def matmul_softmax(x: BlksprsTensor, sparsity_layout_x: Tensor,
                   y: BlksprsTensor, sparsity_layout_y: Tensor,
                   sparsity_layout_output: Tensor,
                   sparsity_block_size: int, scale: float = 1.0, out_dtype: torch.dtype | None = None,
                   layout_cache: dict | None = None) -> BlksprsTensor:
    """``softmax(scale * (x @ y))`` over the active blocks of every output row, in compressed form.

    The arguments up to ``sparsity_block_size`` and ``layout_cache`` are those of :func:`matmul` (the
    same cache can be shared with it); output blocks without a common inner block hold scores of
    zero and take part in the softmax like any other active block.

    Args:
        scale (float): Factor applied to the scores before the softmax (default ``1.0``).
        out_dtype (torch.dtype, optional): dtype of the result: float16, bfloat16 or float32
            (default: the dtype of ``x``).

    Returns:
        BlksprsTensor: The probabilities on ``sparsity_layout_output``.
    """
    return _matmul_softmax_eager(x, sparsity_layout_x, y, sparsity_layout_y, sparsity_layout_output,
                                 sparsity_block_size, scale, out_dtype, layout_cache)
