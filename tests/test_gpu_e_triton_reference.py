"""Against the reference package itself on the same GPU (its Triton kernels, installed under
baseline/_ref): LUT cache entries and inferred layouts bit-exact, matmul forward / backward within the
parity tolerances (1e-2 * max|ref| for fp16 / bf16, 1e-3 * max|ref| for fp32 = TF32 in both).
Skipped where the reference is not installed."""
import os
import sys

import pytest
import torch

import bench
from gpu_util import DEV, rel_err, tolerance

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not os.path.isdir(os.path.join(REF_DIR, "blksprs")):
        pytest.skip("reference package not installed under baseline/_ref")
    os.environ.setdefault("BLKSPRS_AUTOTUNE", "TEST")
    sys.path.insert(0, REF_DIR)
    try:
        import blksprs
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference not importable: {exc!r}")
    finally:
        sys.path.remove(REF_DIR)
    return blksprs


CASES = [("config1", None), ("config2", 2), ("config3", 2), ("config4", 1), ("config5", 1)]


@pytest.mark.parametrize("name,batch", CASES, ids=[c[0] for c in CASES])
def test_matches_reference_triton_op(ref, name, batch):
    import blksprs_b200 as ours
    lx, ly, lo, bsz, dtype = bench.workload_layouts(name, batch=batch)
    x, y, g = bench.workload_values(name, lx, ly, lo, bsz, dtype, seed=3)
    lxd, lyd, lod = lx.to(DEV), ly.to(DEV), lo.to(DEV)
    results, caches = [], []
    for lib in (ref, ours):
        xd = x.to(DEV).requires_grad_(True)
        yd = y.to(DEV).requires_grad_(True)
        cache = {}
        out = lib.ops.matmul(xd, lxd, yd, lyd, lod, bsz, cache)
        out.backward(g.to(DEV))
        torch.cuda.synchronize()
        results.append(tuple(t.detach().as_subclass(torch.Tensor) for t in (out, xd.grad, yd.grad)))
        caches.append(cache)
    for key in ("packed_indices_x", "packed_indices_y", "layout_indices_o"):
        assert torch.equal(caches[0][key], caches[1][key]), key
        assert caches[0][key].dtype == caches[1][key].dtype == torch.int64
    assert caches[0]["n_sparse_blocks"] == caches[1]["n_sparse_blocks"]
    tol = tolerance(dtype)
    for r, o, what in zip(results[0], results[1], ("out", "grad_x", "grad_y")):
        assert r.shape == o.shape and r.dtype == o.dtype
        assert rel_err(o, r.cpu()) <= tol, (what, rel_err(o, r.cpu()))


def test_layout_helpers_match_reference(ref):
    import blksprs_b200 as ours
    lx, ly, _, _, _ = bench.workload_layouts("config2", batch=3)
    lxd, lyd = lx.to(DEV), ly.to(DEV)
    for fn in ("build_sparsity_layout_matmul", "build_sparsity_layout_matmul_fast",
               "build_sparsity_layout_matmul_outer"):
        assert torch.equal(getattr(ref.layouting, fn)(lxd, lyd), getattr(ours.layouting, fn)(lxd, lyd)), fn
    # float 0/1 layouts too
    assert torch.equal(ref.layouting.build_sparsity_layout_matmul(lxd.float(), lyd.float()),
                       ours.layouting.build_sparsity_layout_matmul(lxd.float(), lyd.float()))


def test_transpose_matches_reference(ref):
    import blksprs_b200 as ours
    lx, _, _, bsz, dtype = bench.workload_layouts("config2", batch=2)
    g = torch.Generator().manual_seed(5)
    x = torch.randn((int(lx.sum()), bsz, bsz), generator=g).to(dtype).to(DEV)
    r_out, r_layout = ref.ops.transpose(x, lx.to(DEV), bsz)
    o_out, o_layout = ours.ops.transpose(x, lx.to(DEV), bsz)
    assert torch.equal(r_layout, o_layout)
    assert torch.equal(r_out.as_subclass(torch.Tensor), o_out.as_subclass(torch.Tensor))


@pytest.mark.parametrize("bsz", [64, 128])
def test_fp32_tensor_memory_path_matches_reference_tf32(ref, bsz):
    """fp32 at block size 64 / 128 runs as `kind::tf32` on the tcgen05 kernel: the operands lose the same
    mantissa bits as in the reference's TF32 `tl.dot`, only the order of the fp32 additions differs."""
    import blksprs_b200 as ours
    from gpu_util import make_case
    case = make_case(3, 8 * bsz, 6 * bsz, 10 * bsz, bsz, 0.5, torch.float32, seed=77 + bsz, out_layout="exact")
    lx, ly, lo = (case[k].to(DEV) for k in ("lx", "ly", "lo"))
    results = []
    for lib in (ref, ours):
        x = case["x"].to(DEV).requires_grad_(True)
        y = case["y"].to(DEV).requires_grad_(True)
        out = lib.ops.matmul(x, lx, y, ly, lo, bsz)
        out.backward(case["grad"].to(DEV))
        torch.cuda.synchronize()
        results.append(tuple(t.detach().as_subclass(torch.Tensor) for t in (out, x.grad, y.grad)))
    for r, o, what in zip(results[0], results[1], ("out", "grad_x", "grad_y")):
        assert r.shape == o.shape and r.dtype == o.dtype
        assert rel_err(o, r.cpu()) <= 1e-4, (what, rel_err(o, r.cpu()))
