"""to_sparse / to_dense on the GPU: bit-exact against the CPU oracle (pure data movement), gradients, the
reference's own end-to-end matmul test pattern (dense -> to_sparse -> matmul -> to_dense with autograd), and the
reference's Triton ops where installed."""
import os
import sys

import pytest
import torch

import cases
from gpu_util import DEV, oracle_tolerance, random_layout, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("bsz", [16, 32, 64, 128])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.float64, torch.uint8])
def test_roundtrip_bit_exact(bsz, dtype):
    import blksprs_b200 as bs
    g = torch.Generator().manual_seed(bsz)
    layout = random_layout(3, 5, 4, 0.5, g)
    dense = (torch.randn((3, 5 * bsz, 4 * bsz), generator=g) * 8).to(dtype)
    comp = bs.ops.to_sparse(dense.to(DEV), layout.to(DEV), bsz)
    assert isinstance(comp, bs.BlksprsTensor) and comp.dtype == dtype
    assert torch.equal(comp.cpu().as_subclass(torch.Tensor), oracle.to_sparse(dense, layout, bsz))
    for fill in (0, 3):
        back = bs.ops.to_dense(comp, layout.to(DEV), bsz, fill_value=fill)
        assert type(back) is torch.Tensor
        assert torch.equal(back.cpu(), oracle.to_dense(oracle.to_sparse(dense, layout, bsz), layout, bsz, fill))


def test_empty_full_and_single_block_layouts():
    import blksprs_b200 as bs
    bsz = 32
    dense = torch.randn((2, 64, 96), device=DEV)
    empty = torch.zeros((2, 2, 3), dtype=torch.bool, device=DEV)
    comp = bs.ops.to_sparse(dense, empty, bsz)
    assert comp.shape == (0, bsz, bsz)
    assert torch.equal(bs.ops.to_dense(comp, empty, bsz, fill_value=-1), torch.full_like(dense, -1))
    full = torch.ones((2, 2, 3), device=DEV)   # float layout
    assert torch.equal(bs.ops.to_dense(bs.ops.to_sparse(dense, full, bsz), full, bsz), dense)
    one = torch.ones((2, 1, 1), dtype=torch.bool, device=DEV)
    blk = torch.randn((2, bsz, bsz), device=DEV)
    assert bs.ops.to_sparse(blk, one, bsz).data_ptr() == blk.data_ptr()   # the reference returns the input itself


def test_misaligned_views_fall_back_to_narrow_accesses():
    import blksprs_b200 as bs
    bsz = 16
    base = torch.randn(2 * 32 * 32 + 1, device=DEV, dtype=torch.float16)
    dense = base[1:].view(2, 32, 32)            # contiguous but only 2-byte aligned
    layout = torch.tensor([[[1, 0], [1, 1]], [[0, 1], [0, 0]]], dtype=torch.bool)
    comp = bs.ops.to_sparse(dense, layout.to(DEV), bsz)
    assert torch.equal(comp.cpu().as_subclass(torch.Tensor), oracle.to_sparse(dense.cpu(), layout, bsz))


def test_gradients():
    import blksprs_b200 as bs
    bsz = 32
    g = torch.Generator().manual_seed(1)
    layout = random_layout(2, 3, 3, 0.6, g)
    dense = torch.randn((2, 96, 96), generator=g)
    x = dense.to(DEV).requires_grad_(True)
    comp = bs.ops.to_sparse(x, layout.to(DEV), bsz)
    w = torch.randn(comp.shape, generator=g)
    (comp * w.to(DEV)).sum().backward()
    assert torch.equal(x.grad.cpu(), oracle.to_dense(w, layout, bsz))
    c = oracle.to_sparse(dense, layout, bsz).to(DEV).requires_grad_(True)
    back = bs.ops.to_dense(c, layout.to(DEV), bsz, fill_value=7.0)
    w2 = torch.randn(back.shape, generator=g)
    (back * w2.to(DEV)).sum().backward()
    assert torch.equal(c.grad.cpu(), oracle.to_sparse(w2, layout, bsz))


@pytest.mark.parametrize("shape", [(2, 128, 128, 128, 32, 0.75), (3, 448, 320, 192, 64, 0.5), (2, 256, 256, 256, 128, 0.75)])
@pytest.mark.parametrize("use_amp", [True, False])
def test_dense_in_dense_out_matmul_like_the_reference_test(shape, use_amp):
    """test/cases/test_blocksparse.py:449-504: dense x, y -> to_sparse -> matmul -> to_dense, L1 loss, backward."""
    import blksprs_b200 as bs
    B, m, n, k, bsz, kept = shape
    g = torch.Generator().manual_seed(17)
    lx = random_layout(B, m // bsz, k // bsz, kept, g)
    ly = random_layout(B, k // bsz, n // bsz, kept, g)
    lo = torch.from_numpy(oracle.layout_matmul_fast(lx, ly))
    xd = oracle.to_dense(oracle.to_sparse(torch.randn((B, m, k), generator=g), lx, bsz), lx, bsz)
    yd = oracle.to_dense(oracle.to_sparse(torch.randn((B, k, n), generator=g), ly, bsz), ly, bsz)
    target = torch.randn((B, m, n), generator=g)
    xs, ys = xd.clone().requires_grad_(True), yd.clone().requires_grad_(True)
    stock = torch.matmul(xs, ys)
    torch.nn.L1Loss()(stock * lo.repeat_interleave(bsz, 1).repeat_interleave(bsz, 2), target).backward()
    xo, yo = xd.to(DEV).requires_grad_(True), yd.to(DEV).requires_grad_(True)
    with torch.amp.autocast(device_type="cuda", enabled=use_amp):
        out = bs.ops.matmul(bs.ops.to_sparse(xo, lx.to(DEV), bsz), lx.to(DEV),
                            bs.ops.to_sparse(yo, ly.to(DEV), bsz), ly.to(DEV), lo.to(DEV), bsz)
        dense_out = bs.ops.to_dense(out, lo.to(DEV), bsz)
    torch.nn.L1Loss()(dense_out.float(), target.to(DEV)).backward()
    atol, rtol = (4e-2, 2e-2) if use_amp else (6e-2, 1.5e-2)   # the reference test's tolerances
    masked = stock.detach() * lo.repeat_interleave(bsz, 1).repeat_interleave(bsz, 2)
    assert torch.allclose(dense_out.float().cpu(), masked, atol=atol, rtol=rtol)
    assert torch.allclose(xo.grad.cpu(), xs.grad, atol=atol, rtol=rtol)
    assert torch.allclose(yo.grad.cpu(), ys.grad, atol=atol, rtol=rtol)


def test_matches_reference_conversion_ops():
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
    bsz = 64
    g = torch.Generator().manual_seed(3)
    layout = random_layout(4, 6, 5, 0.4, g).to(DEV)
    dense = torch.randn((4, 6 * bsz, 5 * bsz), generator=g).to(torch.bfloat16).to(DEV)
    r = ref.ops.to_sparse(dense, layout, bsz)
    o = ours.ops.to_sparse(dense, layout, bsz)
    assert torch.equal(r.as_subclass(torch.Tensor), o.as_subclass(torch.Tensor))
    assert torch.equal(ref.ops.to_dense(r, layout, bsz, fill_value=2.5), ours.ops.to_dense(o, layout, bsz, fill_value=2.5))
