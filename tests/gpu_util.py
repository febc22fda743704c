"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import oracle

DEV = "cuda:0"


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max|got - want| / max|want| (the tolerance form the parity target is stated in)."""
    want = want.float()
    denom = float(want.abs().max()) if want.numel() else 0.0
    if got.numel() == 0:
        return 0.0
    return float((got.float().cpu() - want).abs().max()) / max(denom, 1e-6)


def tolerance(dtype) -> float:
    """The parity target: max|err| <= 1e-2 * max|ref| for fp16/bf16 (fp32 accumulation), 1e-3 * max|ref|
    for fp32 (TF32).  It is stated against the reference's Triton result and, for the fp32 plumbing
    workload (K = 128), against the CPU oracle."""
    return 1e-3 if dtype == torch.float32 else 1e-2


def oracle_tolerance(dtype) -> float:
    """Tolerance against the IEEE-fp32 CPU oracle for arbitrary shapes.  fp32 inputs run as TF32 with
    truncated operands exactly like the reference kernel, whose own error against fp32 grows with
    sqrt(K) (8e-4 * max|ref| at K = 128); 2.5e-3 covers the shapes of the test matrix."""
    return 2.5e-3 if dtype == torch.float32 else 1e-2


def random_layout(B, R, C, kept: float, gen: torch.Generator) -> torch.Tensor:
    """Keeps ``kept`` of the blocks of every batch, like the reference tests' layout helper
    (test/cases/test_blocksparse.py:1583-1594)."""
    layout = torch.ones((B, R, C), dtype=torch.bool)
    n_zero = int(R * C * (1 - kept))
    for b in range(B):
        idx = torch.randperm(R * C, generator=gen)[:n_zero]
        layout[b, idx // C, idx % C] = False
    return layout


def make_case(B, m, n, k, bs, kept, dtype, seed, out_layout="fast"):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    lx = random_layout(B, m // bs, k // bs, kept, g)
    ly = random_layout(B, k // bs, n // bs, kept, g)
    if out_layout == "ones":
        lo = torch.ones((B, m // bs, n // bs), dtype=torch.bool)
    elif out_layout == "fast":
        lo = torch.from_numpy(oracle.layout_matmul_fast(lx, ly))
    else:
        lo = torch.from_numpy(oracle.layout_matmul(lx, ly))
    x = torch.randn((int(lx.sum()), bs, bs), generator=g).to(dtype)
    y = torch.randn((int(ly.sum()), bs, bs), generator=g).to(dtype)
    grad = torch.randn((int(lo.sum()), bs, bs), generator=g).to(dtype)
    return dict(x=x, lx=lx, y=y, ly=ly, lo=lo, bs=bs, grad=grad)


def run_ours(case, layout_cache=None, layout_dtype=None):
    """Forward + backward through the public op; returns (out, grad_x, grad_y) on the GPU."""
    import blksprs_b200 as bs
    cast = (lambda t: t) if layout_dtype is None else (lambda t: t.to(layout_dtype))
    lx, ly, lo = (cast(case[k]).to(DEV) for k in ("lx", "ly", "lo"))
    x = case["x"].to(DEV).requires_grad_(True)
    y = case["y"].to(DEV).requires_grad_(True)
    out = bs.ops.matmul(x, lx, y, ly, lo, case["bs"], layout_cache)
    out.backward(case["grad"].to(DEV))
    return out.detach(), x.grad, y.grad


def check_case(case, tol=None):
    out, gx, gy = run_ours(case)
    x, lx, y, ly, lo, bs, g = (case[k] for k in ("x", "lx", "y", "ly", "lo", "bs", "grad"))
    want = oracle.matmul_forward(x, lx, y, ly, lo, bs)
    wgx, wgy = oracle.matmul_backward(g, x, lx, y, ly, lo, bs)
    tol = oracle_tolerance(x.dtype) if tol is None else tol
    assert out.shape == want.shape and out.dtype == x.dtype
    assert rel_err(out, want) <= tol, ("forward", rel_err(out, want))
    assert rel_err(gx, wgx) <= tol, ("grad_x", rel_err(gx, wgx))
    assert rel_err(gy, wgy) <= tol, ("grad_y", rel_err(gy, wgy))
