"""``matmul_softmax`` (scaled matmul with the softmax fused into the kernel's epilogue plus a light
normalising pass) against the float64 oracle of the chain matmul -> scale -> softmax, against the
package's own unfused chain, and against the reference's three ops on the same GPU
(test/cases/test_blocksparse.py:1517-1529).  Tolerance: 1e-2 * max|ref| for 16-bit data, 1e-3 for fp32."""
import os
import sys

import pytest
import torch

from gpu_util import DEV, make_case, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _band_layout(B, n, width):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return ((j <= i) & ((i - j < width) | (j == 0)))[None].expand(B, n, n).contiguous()


def _attention_case(B, S, D, bsz, dtype, seed, width=3):
    g = torch.Generator().manual_seed(seed)
    n, d = S // bsz, D // bsz
    lq = torch.ones((B, n, d), dtype=torch.bool)
    lkt = torch.ones((B, d, n), dtype=torch.bool)
    lo = _band_layout(B, n, width)
    q = torch.randn((int(lq.sum()), bsz, bsz), generator=g).to(dtype)
    kt = torch.randn((int(lkt.sum()), bsz, bsz), generator=g).to(dtype)
    return q, lq, kt, lkt, lo


@pytest.mark.parametrize("out_dtype", [None, torch.bfloat16, torch.float32], ids=["same", "bf16", "fp32"])
@pytest.mark.parametrize("bsz,dtype", [(64, torch.float16), (64, torch.bfloat16), (128, torch.bfloat16), (64, torch.float32),
                                        (128, torch.float32), (32, torch.float16), (16, torch.float32),
                                        (16, torch.bfloat16), (32, torch.float32)],
                         ids=["bs64-fp16", "bs64-bf16", "bs128-bf16", "bs64-fp32", "bs128-fp32", "bs32-fp16", "bs16-fp32",
                              "bs16-bf16", "bs32-fp32"])
def test_attention_scores_forward_and_backward(bsz, dtype, out_dtype):
    import blksprs_b200 as bs
    B, S, D = 3, 8 * bsz, 2 * bsz
    q, lq, kt, lkt, lo = _attention_case(B, S, D, bsz, dtype, seed=bsz)
    scale = 1.0 / (D ** 0.5)
    qd = q.to(DEV).requires_grad_(True)
    ktd = kt.to(DEV).requires_grad_(True)
    out = bs.ops.matmul_softmax(qd, lq.to(DEV), ktd, lkt.to(DEV), lo.to(DEV), bsz, scale=scale, out_dtype=out_dtype)
    assert isinstance(out, bs.BlksprsTensor)
    assert out.dtype == (out_dtype or dtype)
    want = oracle.matmul_softmax(q, lq, kt, lkt, lo, bsz, scale)
    # fp32 operands run as TF32 (like the reference's tl.dot): a score error of ~1e-3 * max|score| becomes a
    # relative error of that size in the probabilities, so the fp32 bound here is 5e-3 * max|ref|; against
    # the reference's own TF32 chain on the same GPU the 1e-3 bound holds (test below)
    tol = 5e-3 if (dtype == torch.float32 and out.dtype == torch.float32) else 1e-2
    assert rel_err(out.detach(), want) <= tol, rel_err(out.detach(), want)
    # every row of probabilities sums to one
    dense = oracle.to_dense(out.detach().float().cpu().as_subclass(torch.Tensor), lo, bsz)
    assert torch.allclose(dense.sum(-1), torch.ones(B, S), atol=2e-2 if out.dtype != torch.float32 else 2e-3)
    g = torch.Generator().manual_seed(77)
    grad = torch.randn(out.shape, generator=g)
    out.backward(grad.to(DEV).to(out.dtype))
    wq, wk = oracle.matmul_softmax_backward(grad.to(out.dtype).double(), q, lq, kt, lkt, lo, bsz, scale)
    btol = 2e-2 if dtype != torch.float32 else 1e-2
    assert rel_err(qd.grad, wq.float()) <= btol, rel_err(qd.grad, wq.float())
    assert rel_err(ktd.grad, wk.float()) <= btol, rel_err(ktd.grad, wk.float())


@pytest.mark.parametrize("bsz", [64, 128])
def test_random_layouts_with_blocks_that_have_no_pair(bsz):
    """Sparse operands on an all-ones output layout: many output blocks have no common inner block; their
    scores are zero and they take part in the softmax of their rows."""
    import blksprs_b200 as bs
    case = make_case(2, 4 * bsz, 6 * bsz, 3 * bsz, bsz, 0.35, torch.bfloat16, seed=4, out_layout="ones")
    x, lx, y, ly, lo = (case[k] for k in ("x", "lx", "y", "ly", "lo"))
    x, y = x * 0.2, y * 0.2
    out = bs.ops.matmul_softmax(x.to(DEV), lx.to(DEV), y.to(DEV), ly.to(DEV), lo.to(DEV), bsz, scale=0.7)
    want = oracle.matmul_softmax(x, lx, y, ly, lo, bsz, 0.7)
    assert rel_err(out, want) <= 1e-2, rel_err(out, want)
    # both panel widths of the tcgen05 kernel
    from blksprs_b200 import plan
    for kernel in ("umma", "panel"):
        plan.set_kernel(kernel)
        try:
            got = bs.ops.matmul_softmax(x.to(DEV), lx.to(DEV), y.to(DEV), ly.to(DEV), lo.to(DEV), bsz, scale=0.7)
        finally:
            plan.set_kernel("auto")
        assert rel_err(got, want) <= 1e-2, (kernel, rel_err(got, want))


def test_equals_the_unfused_chain_of_this_package_and_shares_the_matmul_cache():
    import blksprs_b200 as bs
    bsz = 64
    q, lq, kt, lkt, lo = _attention_case(4, 1024, 128, bsz, torch.float16, seed=2, width=5)
    qd, ktd, lqd, lktd, lod = q.to(DEV), kt.to(DEV), lq.to(DEV), lkt.to(DEV), lo.to(DEV)
    cache = {}
    scale = 128 ** -0.5
    scores = bs.ops.matmul(qd, lqd, ktd, lktd, lod, bsz, cache)
    chain = bs.ops.softmax((scores.float() * scale), lod, bsz).to(torch.bfloat16)
    fused = bs.ops.matmul_softmax(qd, lqd, ktd, lktd, lod, bsz, scale=scale, out_dtype=torch.bfloat16, layout_cache=cache)
    # the chain rounds the scores to fp16 before the softmax, the fused op does not: compare at the tolerance
    assert rel_err(fused, chain.float().cpu()) <= 1e-2


def test_matches_reference_chain_on_this_gpu():
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "blksprs")):
        pytest.skip("reference package not installed under baseline/_ref")
    sys.path.insert(0, ref_dir)
    os.environ.setdefault("BLKSPRS_AUTOTUNE", "TEST")
    import blksprs as ref
    import blksprs_b200 as bs
    bsz = 64
    q, lq, kt, lkt, lo = _attention_case(2, 512, 128, bsz, torch.float32, seed=5)
    qd, ktd, lqd, lktd, lod = q.to(DEV), kt.to(DEV), lq.to(DEV), lkt.to(DEV), lo.to(DEV)
    scale = 128 ** -0.5
    scores = ref.ops.matmul(qd, lqd, ktd, lktd, lod, bsz)
    want = ref.ops.softmax(scores * scale, lod, bsz)
    got = bs.ops.matmul_softmax(qd, lqd, ktd, lktd, lod, bsz, scale=scale)
    assert rel_err(got, want.cpu().as_subclass(torch.Tensor)) <= 1e-3
    want_bf16 = want.to(torch.bfloat16)
    got_bf16 = bs.ops.matmul_softmax(qd, lqd, ktd, lktd, lod, bsz, scale=scale, out_dtype=torch.bfloat16)
    assert rel_err(got_bf16, want_bf16.float().cpu().as_subclass(torch.Tensor)) <= 1e-2


def test_errors_and_empty_output():
    import blksprs_b200 as bs
    bsz = 64
    q, lq, kt, lkt, lo = _attention_case(1, 256, 64, bsz, torch.bfloat16, seed=1)
    args = (q.to(DEV), lq.to(DEV), kt.to(DEV), lkt.to(DEV))
    with pytest.raises(ValueError, match="float16, bfloat16, or float32"):
        bs.ops.matmul_softmax(*args, lo.to(DEV), bsz, out_dtype=torch.float64)
    with pytest.raises(ValueError, match="Output sparsity layout"):
        bs.ops.matmul_softmax(*args, lo[:, :2].contiguous().to(DEV), bsz)
    empty = torch.zeros_like(lo).to(DEV)
    out = bs.ops.matmul_softmax(*args, empty, bsz)
    assert out.shape == (0, bsz, bsz)
