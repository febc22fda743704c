"""Block-sparse matrix product ``bs.ops.matmul`` on the B200-native kernels.

Drop-in for the reference op (blksprs/ops/matmul.py:17-67): same signature,
same validation errors, same layout-cache entries (``packed_indices_x``,
``packed_indices_y``, ``layout_indices_o``, ``n_sparse_blocks`` — bit-identical
tensors), same ``BlksprsTensor`` result.  The forward product and the two
backward products (``dX = dO·Yᵀ`` on x's layout, ``dY = Xᵀ·dO`` on y's layout,
blksprs/ops/matmul.py:130-145) each run as one launch of the native library on a
pre-built plan; no transposed copy of an operand is ever materialised.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _cabi
from ..plan import Product, prepare_products
from ..utils.blksprs_tensor import BlksprsTensor
from ..utils.tools import build_layout_indices, build_packed_indices, cast_for_autocast, \
    finalize_layout_cache, implicit_layout_cache, layout_cache_is_current, plain_dispatch, prepare_layout_cache
from ..utils.validation import ensure_contiguous, validate_contiguous, validate_device, validate_dimensions, \
    validate_dtype_float, validate_shape, validate_sparsity, validate_sparsity_block_size, \
    validate_sparsity_layout, validation_enabled

_PLANS = "_b200_plans"


class _MatmulPlans:
    """Private cache entry: the plans of the three products and the extra LUTs the backward products need.

    Lives in the layout cache as one opaque value, so filling in the backward
    plans later does not change the cache's recorded state.
    """

    def __init__(self, sl_x: Tensor, sl_y: Tensor, sl_o: Tensor):
        self.layouts = (sl_x, sl_y, sl_o)
        self.n_x: int | None = None
        self.n_y: int | None = None
        self.layouts_validated = False  # the layout-only checks passed for this cache
        self.forward: Product | None = None
        self.grad_x: Product | None = None
        self.grad_y: Product | None = None
        self.packed_o: Tensor | None = None

    def dims(self):
        sl_x, sl_y, _ = self.layouts
        return sl_x.size(1), sl_x.size(2), sl_y.size(2)  # R, K, C


def matmul_build_layout_cache(layout_cache: dict | None, sparsity_layout_x: Tensor, sparsity_layout_y: Tensor,
                              sparsity_layout_output: Tensor) -> dict:
    """Builds or reuses the matmul metadata (blksprs/ops/matmul.py:256-279 plus the plans of the native kernels)."""
    layout_cache = prepare_layout_cache(layout_cache, "matmul", sparsity_layout_x, sparsity_layout_y,
                                        sparsity_layout_output)

    if "packed_indices_x" not in layout_cache:
        layout_cache["packed_indices_x"] = build_packed_indices(sparsity_layout_x)
    if "packed_indices_y" not in layout_cache:
        layout_cache["packed_indices_y"] = build_packed_indices(sparsity_layout_y)
    if "layout_indices_o" not in layout_cache:
        # counted once: the LUT's row count is the number of active output blocks
        layout_cache["layout_indices_o"] = build_layout_indices(sparsity_layout_output,
                                                                layout_cache.get("n_sparse_blocks"))
    if "n_sparse_blocks" not in layout_cache:
        layout_cache["n_sparse_blocks"] = layout_cache["layout_indices_o"].size(0)
    if _PLANS not in layout_cache:
        layout_cache[_PLANS] = _MatmulPlans(sparsity_layout_x, sparsity_layout_y, sparsity_layout_output)
    plans: _MatmulPlans = layout_cache[_PLANS]
    if plans.forward is None:
        R, K, C = plans.dims()
        plans.forward = Product(_cabi.OP_NN, layout_cache["layout_indices_o"],
                                layout_cache["packed_indices_x"], layout_cache["packed_indices_y"], R, K, C)

    validate_contiguous(sparsity_layout_x, layout_cache["packed_indices_x"],
                        sparsity_layout_y, layout_cache["packed_indices_y"],
                        sparsity_layout_output, layout_cache["layout_indices_o"])
    return finalize_layout_cache(layout_cache)


def _backward_plans(plans: _MatmulPlans, packed_x: Tensor, packed_y: Tensor, n_x: int, n_y: int) -> None:
    """Fills in the plans of the two backward products (once per layout triple)."""
    if plans.grad_x is not None and plans.grad_y is not None:
        return
    sl_x, sl_y, sl_o = plans.layouts
    R, K, C = plans.dims()
    if plans.packed_o is None:
        plans.packed_o = build_packed_indices(sl_o)
    if plans.grad_x is None:
        lut_x = build_layout_indices(sl_x, n_x)
        plans.grad_x = Product(_cabi.OP_NT, lut_x, plans.packed_o, packed_y, R, K, C)
    if plans.grad_y is None:
        lut_y = build_layout_indices(sl_y, n_y)
        plans.grad_y = Product(_cabi.OP_TN, lut_y, packed_x, plans.packed_o, R, K, C)


class _BlockSparseMatmul(torch.autograd.Function):
    """Differentiable in ``x`` and ``y``; layouts, LUTs and plans are constants."""

    @staticmethod
    def forward(ctx, x: Tensor, y: Tensor, packed_x: Tensor, packed_y: Tensor, plans: _MatmulPlans, bs: int):
        ctx.save_for_backward(x, y, packed_x, packed_y)
        ctx.plans = plans
        ctx.sparsity_block_size = bs
        return plans.forward.run(x, y, bs)

    @staticmethod
    @torch.autograd.function.once_differentiable
    @plain_dispatch
    def backward(ctx, grad_output: Tensor):
        x, y, packed_x, packed_y = ctx.saved_tensors
        plans: _MatmulPlans = ctx.plans
        bs = ctx.sparsity_block_size
        grad_output = grad_output.contiguous()
        if grad_output.dtype != x.dtype:
            grad_output = grad_output.to(x.dtype)
        need_x, need_y = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        _backward_plans(plans, packed_x, packed_y, x.size(0), y.size(0))
        grad_x = plans.grad_x.run(grad_output, y, bs) if need_x else None
        grad_y = plans.grad_y.run(x, grad_output, bs) if need_y else None
        return grad_x, grad_y, None, None, None, None


# ---- registered ops ------------------------------------------------------------------------------
# The reference registers its forward as ``torch.library.triton_op("blksprs::matmul_forward")`` with autograd
# attached (blksprs/ops/matmul.py:70-75, 283-293).  The same positional schema is registered here under the
# ``blksprs_b200`` namespace, for callers that address the op through ``torch.ops`` or want it inside a
# ``torch.compile`` graph without a graph break (pre-built LUTs, validation off).  The ops are opaque to the
# compiler; they find their plans through the layout tensors (library-owned cache, ``utils/tools.py``).  The eager
# ``matmul`` wrapper keeps using the lighter ``autograd.Function`` above.

@torch.library.custom_op("blksprs_b200::matmul_forward", mutates_args=(), device_types="cuda")
def matmul_forward(x: Tensor, y: Tensor,
                   sparsity_layout_x: Tensor, sparsity_reverse_lut_x: Tensor,
                   sparsity_layout_y: Tensor, sparsity_reverse_lut_y: Tensor,
                   sparsity_layout_o: Tensor, sparsity_lut_o: Tensor,
                   sparsity_block_size: int, n_sparse_blocks: int) -> Tensor:
    cache = matmul_build_layout_cache(None, sparsity_layout_x, sparsity_layout_y, sparsity_layout_o)
    return cache[_PLANS].forward.run(x.contiguous(), y.contiguous(), sparsity_block_size)


@matmul_forward.register_fake
def _(x, y, sparsity_layout_x, sparsity_reverse_lut_x, sparsity_layout_y, sparsity_reverse_lut_y,
      sparsity_layout_o, sparsity_lut_o, sparsity_block_size, n_sparse_blocks):
    return x.new_empty((n_sparse_blocks, sparsity_block_size, sparsity_block_size))


@torch.library.custom_op("blksprs_b200::matmul_backward", mutates_args=(), device_types="cuda")
def matmul_backward(grad_output: Tensor, x: Tensor, y: Tensor, sparsity_layout_x: Tensor, sparsity_layout_y: Tensor,
                    sparsity_layout_o: Tensor, sparsity_block_size: int) -> tuple[Tensor, Tensor]:
    """dX = dO * Y^T on x's layout, dY = X^T * dO on y's layout (blksprs/ops/matmul.py:130-145)."""
    cache = matmul_build_layout_cache(None, sparsity_layout_x, sparsity_layout_y, sparsity_layout_o)
    plans: _MatmulPlans = cache[_PLANS]
    x, y = x.contiguous(), y.contiguous()
    _backward_plans(plans, cache["packed_indices_x"], cache["packed_indices_y"], x.size(0), y.size(0))
    grad_output = grad_output.contiguous().to(x.dtype)
    return (plans.grad_x.run(grad_output, y, sparsity_block_size),
            plans.grad_y.run(x, grad_output, sparsity_block_size))


@matmul_backward.register_fake
def _(grad_output, x, y, sparsity_layout_x, sparsity_layout_y, sparsity_layout_o, sparsity_block_size):
    return torch.empty_like(x), torch.empty_like(y)


def _registered_setup_context(ctx, inputs, output):
    x, y, sl_x, _, sl_y, _, sl_o, _, sparsity_block_size, _ = inputs
    ctx.save_for_backward(x, y, sl_x, sl_y, sl_o)
    ctx.sparsity_block_size = sparsity_block_size


def _registered_backward(ctx, grad_output):
    x, y, sl_x, sl_y, sl_o = ctx.saved_tensors
    grad_x, grad_y = torch.ops.blksprs_b200.matmul_backward(grad_output, x, y, sl_x, sl_y, sl_o,
                                                            ctx.sparsity_block_size)
    return grad_x, grad_y, None, None, None, None, None, None, None, None


matmul_forward.register_autograd(_registered_backward, setup_context=_registered_setup_context)


def _validate_warm(x: Tensor, y: Tensor, plans: _MatmulPlans, sparsity_block_size: int) -> None:
    """The checks that depend on ``x`` and ``y`` (messages as in the full validation); everything that
    depends on the layouts alone was checked when this cache was built and the cache key pins the layouts."""
    validate_dimensions(x, y)
    validate_contiguous(x, y)
    validate_dtype_float(x, y)
    validate_device(x, y, plans.layouts[2])
    for tensor, layout, n_blocks in ((x, plans.layouts[0], plans.n_x), (y, plans.layouts[1], plans.n_y)):
        if tensor.device != layout.device:
            raise ValueError("Tensor and sparsity layout must be on same device")
        if not (tensor.size(-1) == tensor.size(-2) == sparsity_block_size):
            raise ValueError("Blocks not conforming to sparsity block size")
        if tensor.size(0) != n_blocks:
            raise ValueError("Mismatch between sparsity layout and blocks")
    validate_sparsity_block_size(sparsity_block_size, x, y)


def _validate_cold(x, sparsity_layout_x, y, sparsity_layout_y, sparsity_layout_output, sparsity_block_size) -> None:
    validate_dimensions(x, y)
    validate_contiguous(x, y, sparsity_layout_output)
    validate_dtype_float(x, y)
    validate_device(x, y, sparsity_layout_output)
    validate_sparsity(sparsity_block_size, (x, sparsity_layout_x), (y, sparsity_layout_y))
    validate_sparsity_layout(sparsity_layout_output)
    if sparsity_layout_x.size(0) != sparsity_layout_y.size(0):
        raise ValueError("Batch dimensions of tensors must match")
    if sparsity_layout_x.size(-1) != sparsity_layout_y.size(-2):
        raise ValueError("Inner dimensions of tensors must match")
    validate_shape(sparsity_layout_output,
                   (sparsity_layout_x.size(0), sparsity_layout_x.size(1), sparsity_layout_y.size(2)),
                   "Output sparsity layout")
    validate_sparsity_block_size(sparsity_block_size, x, y)


@plain_dispatch
def _matmul_eager(x, sparsity_layout_x, y, sparsity_layout_y, sparsity_layout_output, sparsity_block_size,
                  layout_cache):
    x, y = ensure_contiguous(x, y)
    x, y = cast_for_autocast(x, y)

    # A warm cache (same layout objects, unchanged) has the plans and already knows that the layouts are
    # valid and how many blocks each holds: only the checks on x and y remain, without a device read.
    if layout_cache is None:
        # no caller-owned cache: a small library-owned one, with the same reuse rule (tools.implicit_layout_cache)
        layout_cache = implicit_layout_cache("matmul", sparsity_layout_x, sparsity_layout_y, sparsity_layout_output)
    plans = None
    if layout_cache_is_current(layout_cache, "matmul", sparsity_layout_x, sparsity_layout_y,
                               sparsity_layout_output):
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
            # validate_sparsity has just confirmed the block counts against the layouts
            plans.n_x, plans.n_y = x.size(0), y.size(0)
            plans.layouts_validated = True
        requests = [(plans.forward, sparsity_block_size, x.dtype, x.size(0), y.size(0))]
        if torch.is_grad_enabled() and (x.requires_grad or y.requires_grad):
            # a training step will need them: build the plans of dX and dY with the forward plan, so that all
            # cold-path device reads of a layout triple happen in its first forward call
            _backward_plans(plans, layout_cache["packed_indices_x"], layout_cache["packed_indices_y"], x.size(0),
                            y.size(0))
            n_o = plans.forward.n_out
            requests += [(plans.grad_x, sparsity_block_size, x.dtype, n_o, y.size(0)),
                         (plans.grad_y, sparsity_block_size, x.dtype, x.size(0), n_o)]
        # the sizes of all plans this call (and its backward) will use arrive in one device->host copy
        prepare_products(requests)

    if torch.is_grad_enabled() and (x.requires_grad or y.requires_grad):
        out = _BlockSparseMatmul.apply(x, y, layout_cache["packed_indices_x"], layout_cache["packed_indices_y"],
                                       plans, sparsity_block_size)
    else:
        # nothing to differentiate: the product without the autograd node
        out = plans.forward.run(x, y, sparsity_block_size)
    return BlksprsTensor.wrap(out)


_matmul_no_compile = torch.compiler.disable(_matmul_eager)


@torch.amp.custom_fwd(device_type="cuda")
def matmul(x: BlksprsTensor, sparsity_layout_x: Tensor,
           y: BlksprsTensor, sparsity_layout_y: Tensor,
           sparsity_layout_output: Tensor,
           sparsity_block_size: int, layout_cache: dict | None = None) -> BlksprsTensor:
    """Multiplies two compressed block-sparse tensors.

    Only blocks marked active by ``sparsity_layout_output`` are calculated; active output
    blocks without a common inner block are zero.

    Args:
        x (BlksprsTensor): The compressed left operand.
        sparsity_layout_x (Tensor): The sparsity layout of ``x``.
        y (BlksprsTensor): The compressed right operand.
        sparsity_layout_y (Tensor): The sparsity layout of ``y``.
        sparsity_layout_output (Tensor): The sparsity layout of the output tensor.
        sparsity_block_size (int): The size of the sparsity blocks.
        layout_cache (dict, optional): Reusable layout metadata cache (default ``None``).

    Returns:
        BlksprsTensor: The matrix product in compressed form.
    """
    # torch.compile sees an opaque call (graph break, as for the reference's custom op); eager calls skip
    # the wrapper that enforces it
    impl = _matmul_no_compile if torch.compiler.is_compiling() else _matmul_eager
    return impl(x, sparsity_layout_x, y, sparsity_layout_y, sparsity_layout_output, sparsity_block_size,
                layout_cache)
