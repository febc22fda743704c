"""Operands and results beyond 2^31 - 1 elements, and the benchmark workloads at their full size.

The reference switches its kernels to 64-bit index arithmetic when a participating buffer holds more
than 2^31 - 1 elements (blksprs/utils/tools.py:231-260) and tests that with sampled blocks of a large
product against an fp32 dense reference (test/cases/test_blocksparse.py:2018-2103, matmul part
2085-2103).  The kernels here compute element offsets in 64 bits throughout; these tests run them on
both sides of the limit with the same method: sampled output blocks (the first, the last, random
ones) against an fp32 product of the same compressed operand blocks computed with torch on the GPU.
Sizes are chosen for a 180 GB device; the tests skip on smaller ones.
"""
import pytest
import torch

import bench
from gpu_util import DEV

pytestmark = pytest.mark.gpu
INT32_MAX = 2 ** 31 - 1


def _need_gb(gb):
    free, _ = torch.cuda.mem_get_info()
    if free < gb * 2 ** 30:
        pytest.skip(f"needs {gb} GiB of free device memory")


def _check(name, batch, backward, tol, kernel="auto", need_gb=40):
    import blksprs_b200 as bs
    from blksprs_b200 import plan
    _need_gb(need_gb)
    dev = torch.device(DEV)
    lx, ly, lo, bsz, dtype = bench.workload_layouts(name, batch=batch)
    x, y, g = bench.workload_values(name, lx, ly, lo, bsz, dtype, seed=0, device=dev)
    plan.set_kernel(kernel)
    try:
        if backward:
            x.requires_grad_(True)
            y.requires_grad_(True)
        out = bs.ops.matmul(x, lx.to(dev), y, ly.to(dev), lo.to(dev), bsz)
        if backward:
            out.backward(g)
        plan.check_device_status()
    finally:
        plan.set_kernel("auto")
    xd, yd = x.detach(), y.detach()
    rec = bench.sampled_block_check(xd, lx, yd, ly, lo, out.detach(), bsz, "nn", 48)
    assert rec["max_rel_err"] <= tol, ("forward", rec)
    if backward:
        rx = bench.sampled_block_check(g, lo, yd, ly, lx, x.grad, bsz, "nt", 32)
        ry = bench.sampled_block_check(xd, lx, g, lo, ly, y.grad, bsz, "tn", 32)
        assert rx["max_rel_err"] <= tol, ("grad_x", rx)
        assert ry["max_rel_err"] <= tol, ("grad_y", ry)
    return x, out


def test_config3_full_size_attention_scores():
    """fp16, block 64, 512 x (4096 x 128) x (128 x 4096) on the banded causal layout: 2.1 GiB of output."""
    _, out = _check("config3", None, backward=True, tol=1e-2)
    assert out.size(0) == 512 * 540


def test_config4_full_size_straddles_the_int32_limit():
    """bf16 P (512, 4096, 4096) at 25 %: about 2^31 elements; forward + backward at full size."""
    x, _ = _check("config4", None, backward=True, tol=1e-2)
    assert abs(x.numel() - 2 ** 31) < 2 ** 31 * 0.01   # the draw lands within 1 % of the limit


def test_config5_full_size_forward():
    _check("config5", None, backward=False, tol=1e-2)


def test_operand_clearly_beyond_int32_elements_tcgen05():
    """config4's generator at batch 640: P holds about 2.7e9 elements; forward + backward."""
    x, _ = _check("config4", 640, backward=True, tol=1e-2)
    assert x.numel() > INT32_MAX


def test_operand_beyond_int32_elements_mma_sync():
    """The mma.sync kernel (block 32, fp16, as in the reference's own large-index case):
    X (640, 4096, 4096) at 25 % = about 2.7e9 elements times a dense (640, 4096, 32) operand."""
    import blksprs_b200 as bs
    from blksprs_b200 import plan
    _need_gb(30)
    dev = torch.device(DEV)
    bsz = 32
    g = torch.Generator().manual_seed(11)
    lx = torch.rand((640, 128, 128), generator=g) < 0.25
    ly = torch.ones((640, 128, 1), dtype=torch.bool)
    lo = torch.ones((640, 128, 1), dtype=torch.bool)
    gd = torch.Generator(device=dev).manual_seed(12)
    x = torch.empty((int(lx.sum()), bsz, bsz), dtype=torch.float16, device=dev)
    for first in range(0, x.size(0), 1 << 18):
        x[first:first + (1 << 18)] = torch.randn((min(1 << 18, x.size(0) - first), bsz, bsz), generator=gd,
                                                 device=dev) * 0.05
    y = torch.randn((int(ly.sum()), bsz, bsz), generator=gd, device=dev).half()
    assert x.numel() > INT32_MAX
    out = bs.ops.matmul(x, lx.to(dev), y, ly.to(dev), lo.to(dev), bsz)
    plan.check_device_status()
    rec = bench.sampled_block_check(x, lx, y, ly, lo, out, bsz, "nn", 48)
    assert rec["max_rel_err"] <= 1e-2, rec
    # the last operand blocks (element offsets beyond 2^31) really took part: the last output block is not zero
    assert float(out[-1].float().abs().max()) > 0
