"""The five benchmark workloads (batch reduced where the dense CPU oracle would not fit a quick test):
forward + backward through the public op against the CPU oracle, plus properties that do not need the
oracle at full size (two independent kernel families agree, linearity in x)."""
import pytest
import torch

import bench
from gpu_util import DEV, rel_err, tolerance
from oracle import oracle

pytestmark = pytest.mark.gpu

CASES = [("config1", None), ("config2", 4), ("config3", 4), ("config4", 2), ("config5", 2)]


def _run(name, batch, kernel="auto", scale_x=1.0, seed=0):
    import blksprs_b200 as bs
    from blksprs_b200 import plan
    lx, ly, lo, bsz, dtype = bench.workload_layouts(name, batch=batch)
    x, y, g = bench.workload_values(name, lx, ly, lo, bsz, dtype, seed=seed)
    plan.set_kernel(kernel)
    try:
        xd = (x.to(DEV) * scale_x).requires_grad_(True)
        yd = y.to(DEV).requires_grad_(True)
        out = bs.ops.matmul(xd, lx.to(DEV), yd, ly.to(DEV), lo.to(DEV), bsz)
        out.backward(g.to(DEV))
        plan.check_device_status()
    finally:
        plan.set_kernel("auto")
    return (x, y, g, lx, ly, lo, bsz), (out.detach(), xd.grad, yd.grad)


@pytest.mark.parametrize("name,batch", CASES, ids=[c[0] for c in CASES])
def test_workload_matches_oracle(name, batch):
    (x, y, g, lx, ly, lo, bsz), (out, gx, gy) = _run(name, batch)
    tol = tolerance(x.dtype)
    want = oracle.matmul_forward(x, lx, y, ly, lo, bsz)
    wgx, wgy = oracle.matmul_backward(g, x, lx, y, ly, lo, bsz)
    assert rel_err(out, want) <= tol
    assert rel_err(gx, wgx) <= tol
    assert rel_err(gy, wgy) <= tol


@pytest.mark.parametrize("name,batch", [("config2", None), ("config3", 32), ("config4", 16), ("config5", 16)],
                         ids=["config2-full", "config3-b32", "config4-b16", "config5-b16"])
def test_kernel_families_agree_at_scale(name, batch):
    """tcgen05 (auto) and mma.sync results on the same inputs: independent kernels, same fp32 accumulation,
    different summation order only."""
    _, auto = _run(name, batch, "auto")
    _, mma = _run(name, batch, "mma")
    for a, m in zip(auto, mma):
        assert a.shape == m.shape
        assert rel_err(a, m.cpu()) <= 2e-3


def test_linearity_in_x_at_full_size():
    """matmul(2x, y) == 2 matmul(x, y) exactly (a power-of-two scale commutes with every rounding)."""
    _, one = _run("config2", None, "auto", 1.0)
    _, two = _run("config2", None, "auto", 2.0)
    assert torch.equal(two[0].float(), 2 * one[0].float())
    assert torch.equal(two[2].float(), 2 * one[2].float())   # dY = X^T dO scales with x
    assert torch.equal(two[1], one[1])                       # dX = dO Y^T does not depend on x
