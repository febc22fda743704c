"""Block-sparse softmax on the GPU against the CPU oracle and the reference's Triton op, and the attention
chain matmul -> softmax -> matmul the reference benchmarks (test/cases/test_blocksparse.py:1517-1529)."""
import os
import sys

import pytest
import torch

from gpu_util import DEV, random_layout, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("bsz,B,R,C,kept", [(16, 2, 3, 5, 0.6), (32, 3, 4, 4, 0.5), (64, 2, 8, 8, 0.3), (128, 2, 2, 3, 1.0),
                                             (64, 1, 4, 64, 0.25)])
def test_forward_and_backward(bsz, B, R, C, kept):
    import blksprs_b200 as bs
    g = torch.Generator().manual_seed(bsz + C)
    layout = random_layout(B, R, C, kept, g)
    x = torch.randn((int(layout.sum()), bsz, bsz), generator=g) * 3
    xd = x.to(DEV).requires_grad_(True)
    out = bs.ops.softmax(xd, layout.to(DEV), bsz)
    want = oracle.softmax(x, layout, bsz)
    assert isinstance(out, bs.BlksprsTensor)
    assert torch.allclose(out.detach().cpu().as_subclass(torch.Tensor), want, atol=1e-6, rtol=1e-5)
    grad = torch.randn(out.shape, generator=g)
    out.backward(grad.to(DEV))
    want_grad = oracle.softmax_backward(grad, want, layout, bsz)
    assert torch.allclose(xd.grad.cpu(), want_grad, atol=1e-6, rtol=1e-4)
    for fn in (bs.ops.softmax_regular, bs.ops.softmax_fused):
        assert torch.equal(fn(x.to(DEV), layout.to(DEV), bsz).as_subclass(torch.Tensor), out.detach().as_subclass(torch.Tensor))


def test_rows_sum_to_one_and_errors():
    import blksprs_b200 as bs
    bsz = 32
    layout = torch.tensor([[[1, 0, 1], [0, 0, 1]]], dtype=torch.bool)
    x = torch.randn((3, bsz, bsz))
    out = bs.ops.softmax(x.to(DEV), layout.to(DEV), bsz)
    dense = oracle.to_dense(out.cpu().as_subclass(torch.Tensor), layout, bsz)
    assert torch.allclose(dense.sum(-1), torch.ones(1, 2 * bsz), atol=1e-5)
    with pytest.raises(ValueError, match="float32"):
        bs.ops.softmax(x.to(DEV).half(), layout.to(DEV), bsz)
    empty = torch.zeros((0, bsz, bsz), device=DEV)
    assert bs.ops.softmax(empty, torch.zeros((1, 2, 3), dtype=torch.bool, device=DEV), bsz).shape == (0, bsz, bsz)


def test_attention_by_parts_matches_dense_attention():
    """scores = Q K^T on a banded layout, softmax, P V: against dense masked attention."""
    import blksprs_b200 as bs
    bsz, B, S, D = 64, 3, 512, 128
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn((B, S, D), generator=g) for _ in range(3))
    n = S // bsz
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    lo = ((j <= i) & ((i - j <= 2) | (j == 0)))[None].expand(B, n, n).contiguous()
    lq = torch.ones((B, n, D // bsz), dtype=torch.bool)
    lk = torch.ones((B, D // bsz, n), dtype=torch.bool)
    dev = lambda t: t.to(DEV)
    qc = bs.ops.to_sparse(dev(q), dev(lq), bsz)
    kc = bs.ops.to_sparse(dev(k.transpose(1, 2).contiguous()), dev(lk), bsz)
    vc = bs.ops.to_sparse(dev(v), dev(lq), bsz)
    scores = bs.ops.matmul(qc, dev(lq), kc, dev(lk), dev(lo), bsz) * (D ** -0.5)
    probs = bs.ops.softmax(scores, dev(lo), bsz)
    out = bs.ops.to_dense(bs.ops.matmul(probs, dev(lo), vc, dev(lq), dev(lq), bsz), dev(lq), bsz)
    mask = lo.repeat_interleave(bsz, 1).repeat_interleave(bsz, 2)
    dense_scores = (q @ k.transpose(1, 2)) * (D ** -0.5)
    want = torch.softmax(dense_scores.masked_fill(~mask, float("-inf")), -1) @ v
    assert rel_err(out, want) <= 2.5e-3   # two TF32 products and a softmax


def test_matches_reference_softmax():
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "blksprs")):
        pytest.skip("reference package not installed under baseline/_ref")
    os.environ.setdefault("BLKSPRS_AUTOTUNE", "TEST")
    sys.path.insert(0, ref_dir)
    try:
        import blksprs as ref
    finally:
        sys.path.remove(ref_dir)
    import blksprs_b200 as ours
    bsz = 32
    g = torch.Generator().manual_seed(4)
    layout = random_layout(2, 6, 6, 0.5, g).to(DEV)
    x = (torch.randn((int(layout.sum()), bsz, bsz), generator=g) * 2).to(DEV)
    grad = torch.randn(x.shape, generator=g).to(DEV)
    res = []
    for lib in (ref, ours):
        xd = x.clone().requires_grad_(True)
        out = lib.ops.softmax(xd, layout, bsz)
        out.backward(grad)
        res.append((out.detach().as_subclass(torch.Tensor), xd.grad))
    assert torch.allclose(res[0][0], res[1][0], atol=1e-6, rtol=1e-5)
    assert torch.allclose(res[0][1], res[1][1], atol=1e-6, rtol=1e-4)


def test_very_wide_block_rows_use_the_plain_kernels():
    """More block columns than a CTA lists in shared memory (8192): the one-warp-per-row kernels take over."""
    import blksprs_b200 as bs
    bsz, C = 16, 8200
    g = torch.Generator().manual_seed(3)
    layout = (torch.rand((1, 2, C), generator=g) < 0.5)
    x = torch.randn((int(layout.sum()), bsz, bsz), generator=g) * 2
    xd = x.to(DEV).requires_grad_(True)
    out = bs.ops.softmax(xd, layout.to(DEV), bsz)
    want = oracle.softmax(x, layout, bsz)
    assert torch.allclose(out.detach().cpu().as_subclass(torch.Tensor), want, atol=1e-6, rtol=1e-5)
    grad = torch.randn(out.shape, generator=g)
    out.backward(grad.to(DEV))
    assert torch.allclose(xd.grad.cpu(), oracle.softmax_backward(grad, want, layout, bsz), atol=1e-6, rtol=1e-4)


_DT = (torch.float16, torch.bfloat16, torch.float32)


@pytest.mark.parametrize("out_dtype", _DT, ids=["to-fp16", "to-bf16", "to-fp32"])
@pytest.mark.parametrize("in_dtype", _DT, ids=["fp16", "bf16", "fp32"])
def test_scaled_entry_points_for_every_type_combination(in_dtype, out_dtype):
    """``bsp_softmax_fwd_scaled`` / ``bsp_softmax_bwd_scaled`` through the C ABI: softmax(scale * x) with x in
    one data type and the result in another, and its gradient with the gradient in a third, against the
    fp32 oracle applied to the same (already rounded) inputs."""
    from blksprs_b200 import _cabi
    from blksprs_b200.utils.tools import build_packed_indices
    bsz, B, R, C, scale = 32, 2, 3, 6, 0.37
    g = torch.Generator().manual_seed(77)
    layout = random_layout(B, R, C, 0.6, g)
    n = int(layout.sum())
    x = (torch.randn((n, bsz, bsz), generator=g) * 3).to(in_dtype)
    packed = build_packed_indices(layout.to(DEV))
    xd = x.to(DEV)
    out = torch.empty((n, bsz, bsz), dtype=out_dtype, device=DEV)
    lib = _cabi.lib()
    _cabi.check(lib.bsp_softmax_fwd_scaled(xd.data_ptr(), _cabi.DATA_DTYPE_CODES[in_dtype], n, packed.data_ptr(), B, R, C,
                                           bsz, scale, out.data_ptr(), _cabi.DATA_DTYPE_CODES[out_dtype],
                                           _cabi.stream_handle(torch.device(DEV))), "bsp_softmax_fwd_scaled")
    want = oracle.softmax(x.float() * scale, layout, bsz)
    tol = 1e-5 if out_dtype == torch.float32 else (1e-3 if out_dtype == torch.float16 else 8e-3)
    assert float((out.float().cpu() - want).abs().max()) <= tol
    # gradient: probabilities as stored (out_dtype), their gradient in in_dtype, the result in every type
    grad = (torch.randn((n, bsz, bsz), generator=g)).to(in_dtype)
    want_grad = oracle.softmax_backward(grad.float(), out.float().cpu(), layout, bsz) * scale
    for x_dtype in _DT:
        gx = torch.empty((n, bsz, bsz), dtype=x_dtype, device=DEV)
        _cabi.check(lib.bsp_softmax_bwd_scaled(grad.to(DEV).data_ptr(), _cabi.DATA_DTYPE_CODES[in_dtype], out.data_ptr(),
                                               _cabi.DATA_DTYPE_CODES[out_dtype], n, packed.data_ptr(), B, R, C, bsz, scale,
                                               gx.data_ptr(), _cabi.DATA_DTYPE_CODES[x_dtype],
                                               _cabi.stream_handle(torch.device(DEV))), "bsp_softmax_bwd_scaled")
        ref_max = float(want_grad.abs().max())
        rel = float((gx.float().cpu() - want_grad).abs().max()) / ref_max
        assert rel <= (1e-5 if x_dtype == torch.float32 else (2e-3 if x_dtype == torch.float16 else 1e-2)), (x_dtype, rel)
