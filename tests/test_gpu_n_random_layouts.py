"""Randomly drawn small problems: arbitrary layout shapes and densities (including empty rows, empty columns,
empty operands and an empty output layout), output layouts that are unrelated to the operands' layouts (the output
layout is an input of the op, blksprs/ops/matmul.py:24,77: active blocks without a common inner block are zero,
inactive ones are not computed), all block sizes and dtypes, forward and both gradients against the CPU oracle.
Seeded: every case is reproducible from its number."""
import pytest
import torch

from gpu_util import DEV, oracle_tolerance, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu


def _draw(case_no: int):
    g = torch.Generator().manual_seed(10_000 + case_no)

    def r(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=g))

    bs = (16, 32, 64, 128)[case_no % 4]
    dtype = (torch.bfloat16, torch.float16, torch.float32)[(case_no // 4) % 3]
    top = 6 if bs <= 32 else (5 if bs == 64 else 3)
    B, R, K, C = r(1, 3), r(1, top), r(1, top), r(1, top)
    density = (0.0, 0.15, 0.5, 0.85, 1.0)

    def layout(shape):
        d = density[r(0, 4)]
        return torch.rand(shape, generator=g) < d

    lx, ly, lo = layout((B, R, K)), layout((B, K, C)), layout((B, R, C))
    x = torch.randn((int(lx.sum()), bs, bs), generator=g).to(dtype)
    y = torch.randn((int(ly.sum()), bs, bs), generator=g).to(dtype)
    grad = torch.randn((int(lo.sum()), bs, bs), generator=g).to(dtype)
    return dict(x=x, lx=lx, y=y, ly=ly, lo=lo, bs=bs, grad=grad)


@pytest.mark.parametrize("case_no", range(48))
def test_random_problem_matches_oracle(case_no):
    import blksprs_b200 as bs
    from blksprs_b200 import plan
    case = _draw(case_no)
    x, lx, y, ly, lo, bsz, grad = (case[k] for k in ("x", "lx", "y", "ly", "lo", "bs", "grad"))
    xd = x.to(DEV).requires_grad_(True)
    yd = y.to(DEV).requires_grad_(True)
    out = bs.ops.matmul(xd, lx.to(DEV), yd, ly.to(DEV), lo.to(DEV), bsz)
    assert out.shape == (int(lo.sum()), bsz, bsz) and out.dtype == x.dtype
    out.backward(grad.to(DEV))
    plan.check_device_status()
    want = oracle.matmul_forward(x, lx, y, ly, lo, bsz)
    wgx, wgy = oracle.matmul_backward(grad, x, lx, y, ly, lo, bsz)
    tol = oracle_tolerance(x.dtype)
    assert rel_err(out.detach(), want) <= tol
    # gradients exist on the operands' layouts even where no output block uses a block (zeros there)
    assert xd.grad.shape == x.shape and yd.grad.shape == y.shape
    assert rel_err(xd.grad, wgx) <= tol
    assert rel_err(yd.grad, wgy) <= tol
