"""The ops registered with ``torch.library`` under the reference's positional schema
(``blksprs::matmul_forward``, blksprs/ops/matmul.py:70-75, with autograd attached, :283-293): direct calls through
``torch.ops`` equal the public wrapper, registration checks pass, and the op sits inside a ``torch.compile`` graph
without a graph break (the reference's README only promises compilation with graph breaks, README.md:287-300)."""
import pytest
import torch

from gpu_util import DEV, make_case

pytestmark = pytest.mark.gpu


def _args(bsz=64, dtype=torch.bfloat16):
    from blksprs_b200.ops.matmul import matmul_build_layout_cache
    case = make_case(2, 4 * bsz, 3 * bsz, 5 * bsz, bsz, 0.5, dtype, seed=17, out_layout="exact")
    lx, ly, lo = (case[k].to(DEV) for k in ("lx", "ly", "lo"))
    cache = matmul_build_layout_cache({}, lx, ly, lo)
    x, y, g = case["x"].to(DEV), case["y"].to(DEV), case["grad"].to(DEV)
    luts = (lx, cache["packed_indices_x"], ly, cache["packed_indices_y"], lo, cache["layout_indices_o"], bsz,
            cache["n_sparse_blocks"])
    return x, y, g, luts, (lx, ly, lo, bsz)


@pytest.mark.parametrize("bsz,dtype", [(64, torch.bfloat16), (16, torch.float32)])
def test_direct_call_equals_the_wrapper_forward_and_backward(bsz, dtype):
    import blksprs_b200 as bs
    x, y, g, luts, (lx, ly, lo, _) = _args(bsz, dtype)
    xa, ya = x.clone().requires_grad_(True), y.clone().requires_grad_(True)
    out = torch.ops.blksprs_b200.matmul_forward(xa, ya, *luts)
    out.backward(g)
    xb, yb = x.clone().requires_grad_(True), y.clone().requires_grad_(True)
    want = bs.ops.matmul(xb, lx, yb, ly, lo, bsz)
    want.backward(g)
    assert torch.equal(out, want.as_subclass(torch.Tensor))
    assert torch.equal(xa.grad, xb.grad) and torch.equal(ya.grad, yb.grad)


def test_registration_checks():
    x, y, _, luts, _ = _args()
    args = (x.clone().requires_grad_(True), y.clone().requires_grad_(True), *luts)
    torch.library.opcheck(torch.ops.blksprs_b200.matmul_forward.default, args,
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))


def test_inside_a_compiled_graph_without_graph_break():
    x, y, g, luts, _ = _args()

    def f(a, b):
        return torch.ops.blksprs_b200.matmul_forward(a * 1.0, b, *luts) * 2.0

    compiled = torch.compile(f, fullgraph=True)
    xa, ya = x.clone().requires_grad_(True), y.clone().requires_grad_(True)
    got = compiled(xa, ya)
    got.backward(g)
    xb, yb = x.clone().requires_grad_(True), y.clone().requires_grad_(True)
    want = f(xb, yb)
    want.backward(g)
    assert torch.allclose(got.float(), want.float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(xa.grad.float(), xb.grad.float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(ya.grad.float(), yb.grad.float(), atol=1e-2, rtol=1e-2)
