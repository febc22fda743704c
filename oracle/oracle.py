"""CPU restatement of the blksprs block-sparse matmul path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (the ``blksprs_b200`` package) imports this module; it is
the checker used by ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Parity pin: every function here is checked against outputs of the reference
itself — ``tests/golden/reference_vectors.npz`` holds LUTs, inferred layouts,
transposes and matmul results produced by importing the reference package
(its LUT/layout helpers unchanged on CPU tensors, its Triton kernels under the
Triton interpreter) with ``tests/golden/make_golden.py``.

Each function cites the reference lines it restates (paths inside the blksprs
repository).
"""
from __future__ import annotations

import numpy as np
import torch
from torch import Tensor


# ---- LUTs ---------------------------------------------------------------------

def layout_indices(layout) -> np.ndarray:
    """LUT: int64 (n, 3) coordinates of the non-zero layout entries in row-major order.

    Restates ``build_layout_indices`` = ``torch.nonzero(layout).contiguous()``
    (blksprs/utils/tools.py:33-35).
    """
    a = _as_numpy(layout)
    return np.ascontiguousarray(np.argwhere(a != 0).astype(np.int64).reshape(-1, a.ndim))


def packed_indices(layout) -> np.ndarray:
    """Reverse LUT: flat int64; rank among entries equal to one, else -1.

    Restates ``build_packed_indices`` (blksprs/utils/tools.py:38-57):
    ``flat = layout.reshape(-1).to(int64)``; ``where(flat == 1, cumsum(flat) - 1, -1)``.
    """
    flat = _as_numpy(layout).reshape(-1)
    flat = np.trunc(flat).astype(np.int64) if flat.dtype.kind == "f" else flat.astype(np.int64)
    csum = np.cumsum(flat, dtype=np.int64)
    return np.where(flat == 1, csum - 1, -1).astype(np.int64)


def n_sparse_blocks(layout) -> int:
    """``torch.sum(layout.to(torch.int)).item()`` (blksprs/ops/matmul.py:270-273)."""
    a = _as_numpy(layout)
    a = np.trunc(a).astype(np.int64) if a.dtype.kind == "f" else a.astype(np.int64)
    return int(a.sum())


# ---- output-layout inference ----------------------------------------------------

def layout_matmul(lx, ly) -> np.ndarray:
    """Exact structural product ``(lx.float() @ ly.float()).to(bool)``
    (blksprs/layouting/sparsity_layout.py:244-258)."""
    x = _as_numpy(lx).astype(np.float32)
    y = _as_numpy(ly).astype(np.float32)
    return np.matmul(x, y) != 0


def layout_matmul_fast(lx, ly) -> np.ndarray:
    """``any(lx, -1, keepdim) & any(ly, -2).unsqueeze(1)`` (blksprs/layouting/sparsity_layout.py:261-282)."""
    x = _as_numpy(lx) != 0
    y = _as_numpy(ly) != 0
    return np.logical_and(x.any(-1, keepdims=True), y.any(-2)[:, None, :])


def layout_matmul_outer(lx, ly) -> np.ndarray:
    """Same with ``|`` (blksprs/layouting/sparsity_layout.py:285-309)."""
    x = _as_numpy(lx) != 0
    y = _as_numpy(ly) != 0
    return np.logical_or(x.any(-1, keepdims=True), y.any(-2)[:, None, :])


# ---- compressed <-> dense (harness helpers; plain gathers) ----------------------

def to_sparse(dense: Tensor, layout, bs: int) -> Tensor:
    """Gathers the active blocks of a dense (B, rows, cols) tensor in LUT order."""
    lut = layout_indices(layout)
    B, rows, cols = dense.shape
    blocks = dense.reshape(B, rows // bs, bs, cols // bs, bs).permute(0, 1, 3, 2, 4)
    idx = torch.from_numpy(lut)
    return blocks[idx[:, 0], idx[:, 1], idx[:, 2]].contiguous()


def to_dense(compressed: Tensor, layout, bs: int, fill_value: float = 0.0) -> Tensor:
    """Scatters compressed blocks back to a dense tensor, ``fill_value`` elsewhere."""
    a = _as_numpy(layout)
    B, R, C = a.shape
    lut = torch.from_numpy(layout_indices(a))
    out = torch.full((B, R, C, bs, bs), fill_value, dtype=compressed.dtype)
    out[lut[:, 0], lut[:, 1], lut[:, 2]] = compressed
    return out.permute(0, 1, 3, 2, 4).reshape(B, R * bs, C * bs).contiguous()


# ---- transpose --------------------------------------------------------------------

def transpose(x: Tensor, layout, bs: int):
    """Compressed transpose (blksprs/ops/transpose.py:45-51,63-88; blksprs/ops/flow.py:64-111).

    ``layout_t = layout.transpose(-1, -2)``; output block p, the p-th non-zero (b, r, c) of
    ``layout_t``, is the transposed source block ``packed(layout)[b, c, r]``.
    """
    a = _as_numpy(layout)
    layout_t = np.ascontiguousarray(np.swapaxes(a, -1, -2))
    packed = packed_indices(a).reshape(a.shape)
    lut_t = layout_indices(layout_t)
    src = packed[lut_t[:, 0], lut_t[:, 2], lut_t[:, 1]]
    out = torch.zeros((lut_t.shape[0], bs, bs), dtype=x.dtype)
    ok = src >= 0
    if ok.any():
        out[torch.from_numpy(np.nonzero(ok)[0])] = x[torch.from_numpy(src[ok])].transpose(-1, -2)
    return out.contiguous(), layout_t


# ---- matmul -----------------------------------------------------------------------

def matmul_forward_blocks(x: Tensor, lx, y: Tensor, ly, lo, bs: int) -> Tensor:
    """Block-by-block restatement of ``matmul_kernel`` (blksprs/ops/matmul.py:178-253).

    For every active output block (b, i, j): fp32 accumulator, add ``X[px] @ Y[py]`` for every
    k with ``px = packed_x[b, i, k] >= 0`` and ``py = packed_y[b, k, j] >= 0``; cast to the
    input dtype.  Blocks without a common k stay zero.  Python loops: small cases only.
    """
    ax, ay = _as_numpy(lx), _as_numpy(ly)
    px = packed_indices(ax).reshape(ax.shape)
    py = packed_indices(ay).reshape(ay.shape)
    lut = layout_indices(lo)
    out = torch.zeros((lut.shape[0], bs, bs), dtype=torch.float32)
    xf, yf = x.float(), y.float()
    for p, (b, i, j) in enumerate(lut):
        for k in range(ax.shape[2]):
            if px[b, i, k] >= 0 and py[b, k, j] >= 0:
                out[p] += xf[px[b, i, k]] @ yf[py[b, k, j]]
    return out.to(x.dtype)


def matmul_forward(x: Tensor, lx, y: Tensor, ly, lo, bs: int, accumulate=torch.float32) -> Tensor:
    """Dense masked-matmul form of the same product (the reference test's own check,
    test/cases/test_blocksparse.py:479-504): expand with zeros, ``torch.matmul`` in fp32,
    compress by the output layout."""
    xd = to_dense(x.to(accumulate), lx, bs)
    yd = to_dense(y.to(accumulate), ly, bs)
    return to_sparse(torch.matmul(xd, yd), lo, bs).to(x.dtype)


def matmul_backward(grad_out: Tensor, x: Tensor, lx, y: Tensor, ly, lo, bs: int, accumulate=torch.float32):
    """``dX = dO·Yᵀ`` on x's layout and ``dY = Xᵀ·dO`` on y's layout
    (``matmul_wrapper_backward``, blksprs/ops/matmul.py:130-145), in dense masked form."""
    xd = to_dense(x.to(accumulate), lx, bs)
    yd = to_dense(y.to(accumulate), ly, bs)
    gd = to_dense(grad_out.to(accumulate), lo, bs)
    gx = to_sparse(torch.matmul(gd, yd.transpose(-1, -2)), lx, bs).to(x.dtype)
    gy = to_sparse(torch.matmul(xd.transpose(-1, -2), gd), ly, bs).to(y.dtype)
    return gx, gy


def matmul_backward_via_transpose(grad_out: Tensor, x: Tensor, lx, y: Tensor, ly, lo, bs: int):
    """The backward exactly as the reference composes it: two compressed transposes and two
    forward products (blksprs/ops/matmul.py:135-143).  Python loops: small cases only."""
    x_t, lx_t = transpose(x, lx, bs)
    y_t, ly_t = transpose(y, ly, bs)
    gx = matmul_forward_blocks(grad_out, lo, y_t, ly_t, lx, bs)
    gy = matmul_forward_blocks(x_t, lx_t, grad_out, lo, ly, bs)
    return gx, gy


# ---- softmax ------------------------------------------------------------------------

def softmax(x: Tensor, layout, bs: int) -> Tensor:
    """Row-wise softmax over the active blocks of every row; inactive blocks count as ``-inf``
    (blksprs/ops/softmax.py:58-61, 93-144), in dense form."""
    dense = to_dense(x.double(), layout, bs, fill_value=float("-inf"))
    out = torch.softmax(dense, dim=-1)
    out = torch.nan_to_num(out, nan=0.0)  # rows without any active block
    return to_sparse(out, layout, bs).to(x.dtype)


def softmax_backward(grad_out: Tensor, out: Tensor, layout, bs: int) -> Tensor:
    """``o * (g - sum_row(g * o))`` (blksprs/ops/softmax.py:157-208)."""
    gd = to_dense(grad_out.double(), layout, bs)
    od = to_dense(out.double(), layout, bs)
    s = (gd * od).sum(-1, keepdim=True)
    return to_sparse(od * (gd - s), layout, bs).to(out.dtype)


def matmul_softmax(x: Tensor, lx, y: Tensor, ly, lo, bs: int, scale: float) -> Tensor:
    """The attention-by-parts chain of the reference's benchmark (test/cases/test_blocksparse.py:1517-1529):
    ``softmax(matmul(x, y) * scale)`` over the active blocks of each output row, in float64.  Active output
    blocks without a common inner block hold zeros (blksprs/ops/matmul.py:187, 245-253) and take part."""
    scores = to_sparse(torch.matmul(to_dense(x.double(), lx, bs), to_dense(y.double(), ly, bs)), lo, bs) * scale
    return softmax(scores, lo, bs)


def matmul_softmax_backward(grad_out: Tensor, x: Tensor, lx, y: Tensor, ly, lo, bs: int, scale: float):
    """Gradients of :func:`matmul_softmax` with respect to ``x`` and ``y`` (float64): softmax backward
    (blksprs/ops/softmax.py:157-208), the scale, then the two products of the matmul backward
    (blksprs/ops/matmul.py:130-145)."""
    probs = matmul_softmax(x, lx, y, ly, lo, bs, scale)
    grad_scores = softmax_backward(grad_out.double(), probs, lo, bs) * scale
    return matmul_backward(grad_scores, x.double(), lx, y.double(), ly, lo, bs, accumulate=torch.float64)


# ---- linear layer on a compressed tensor ---------------------------------------------

def linear(x: Tensor, layout, bs: int, weight: Tensor, bias: Tensor | None = None):
    """``apply_torch_linear`` in dense form (blksprs/utils/processing.py:26-86): expand ``x`` with
    zeros, ``x @ weight.T (+ bias)`` in fp32, compress by the output layout — all blocks when a bias
    is present, else the block rows of ``x`` that hold a block (processing.py:56-64).  This is the
    check the reference's own test makes against ``torch.nn.Linear``
    (test/cases/test_blocksparse.py:1158-1184).  Returns (compressed result, output layout)."""
    a = _as_numpy(layout) != 0
    B, R, _ = a.shape
    n_blocks = weight.shape[0] // bs
    out = to_dense(x.float(), layout, bs) @ weight.float().transpose(-1, -2)
    if bias is not None:
        out = out + bias.float()
        layout_out = np.ones((B, R, n_blocks), dtype=bool)
    else:
        layout_out = np.broadcast_to(a.any(-1, keepdims=True), (B, R, n_blocks)).copy()
    return to_sparse(out, layout_out, bs).to(x.dtype), layout_out


def linear_backward(grad_out: Tensor, layout_out, x: Tensor, layout, bs: int, weight: Tensor, has_bias: bool):
    """Gradients of :func:`linear` in dense form: ``dX = dO @ W`` on x's layout, ``dW = dO^T @ X``
    summed over batch and rows, ``db = sum(dO)`` (what autograd derives for processing.py:48-84)."""
    gd = to_dense(grad_out.float(), layout_out, bs)
    xd = to_dense(x.float(), layout, bs)
    gx = to_sparse(gd @ weight.float(), layout, bs).to(x.dtype)
    gw = torch.einsum("brn,brk->nk", gd, xd)
    gb = gd.sum((0, 1)) if has_bias else None
    return gx, gw, gb


# ---- work model ---------------------------------------------------------------------

def pair_count(lx, ly, lo) -> int:
    """Number of (output block, k) triples the forward product contracts:
    ``(lx.float() @ ly.float())[lo].sum()``."""
    x = (_as_numpy(lx) != 0).astype(np.int64)
    y = (_as_numpy(ly) != 0).astype(np.int64)
    o = _as_numpy(lo) != 0
    return int(np.matmul(x, y)[o].sum())


def _as_numpy(layout) -> np.ndarray:
    if isinstance(layout, Tensor):
        t = layout.detach().cpu()
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.numpy()
    return np.asarray(layout)
