"""``apply_torch_linear`` / ``apply_torch_linear_cached`` on the GPU: against ``torch.nn.Linear`` on the
dense tensor (the reference's own check, test/cases/test_blocksparse.py:1158-1184), against the CPU
oracle, against the reference package where it is installed, and the cache / error behaviour the
reference pins in test/cases/test_regressions.py:535-790."""
import os
import sys

import pytest
import torch

from gpu_util import DEV, random_layout, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

# (B, m, n, k, block size, fraction of blocks kept)
CONFIGS = [(2, 64, 64, 64, 16, 0.75), (2, 64, 128, 64, 32, 0.5), (4, 128, 64, 128, 32, 1.0),
           (3, 256, 128, 192, 64, 0.4), (2, 256, 256, 128, 64, 1.0), (2, 512, 256, 384, 128, 0.5),
           (5, 384, 128, 256, 128, 0.3), (1, 128, 64, 64, 64, 0.0)]


def _tol(dtype):
    return 2.5e-3 if dtype == torch.float32 else 1.5e-2


def _case(B, m, n, k, bsz, kept, dtype, seed, bias):
    g = torch.Generator().manual_seed(seed)
    layout = random_layout(B, m // bsz, k // bsz, kept, g)
    x = torch.randn((int(layout.sum()), bsz, bsz), generator=g).to(dtype)
    linear = torch.nn.Linear(k, n, bias=bias)
    with torch.no_grad():
        linear.weight.copy_(torch.randn((n, k), generator=g) / k ** 0.5)
        if bias:
            linear.bias.copy_(torch.randn(n, generator=g))
    return layout, x, linear.to(dtype)


@pytest.mark.parametrize("cached", [False, True], ids=["plain", "cached"])
@pytest.mark.parametrize("bias", [False, True], ids=["nobias", "bias"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("cfg", CONFIGS, ids=[f"b{c[0]}m{c[1]}n{c[2]}k{c[3]}bs{c[4]}" for c in CONFIGS])
def test_forward_backward_against_oracle(cfg, dtype, bias, cached):
    import blksprs_b200 as bs
    B, m, n, k, bsz, kept = cfg
    layout, x, linear = _case(B, m, n, k, bsz, kept, dtype, seed=m + n + bsz, bias=bias)
    want, want_layout = oracle.linear(x, layout, bsz, linear.weight.detach(), linear.bias.detach() if bias else None)
    linear = linear.to(DEV)
    xd = x.to(DEV).requires_grad_(True)
    if cached:
        out, out_layout = bs.utils.apply_torch_linear_cached(xd, layout.to(DEV), bsz, linear, layout_cache={})
    else:
        out, out_layout = bs.utils.apply_torch_linear(xd, layout.to(DEV), bsz, linear)
    assert isinstance(out, bs.BlksprsTensor) and out.dtype == dtype
    assert type(out_layout) is torch.Tensor and out_layout.dtype == torch.bool
    assert torch.equal(out_layout.cpu(), torch.from_numpy(want_layout))
    assert out.shape == want.shape
    assert rel_err(out.detach(), want) <= _tol(dtype), rel_err(out.detach(), want)

    g = torch.Generator().manual_seed(1)
    grad = torch.randn(want.shape, generator=g).to(dtype)
    out.backward(grad.to(DEV))
    wgx, wgw, wgb = oracle.linear_backward(grad, want_layout, x, layout, bsz, linear.weight.detach().cpu(), bias)
    assert rel_err(xd.grad, wgx) <= _tol(dtype), ("grad_x", rel_err(xd.grad, wgx))
    assert linear.weight.grad.shape == (n, k)
    assert rel_err(linear.weight.grad, wgw) <= _tol(dtype), ("grad_w", rel_err(linear.weight.grad, wgw))
    if bias:
        assert rel_err(linear.bias.grad, wgb) <= _tol(dtype), ("grad_b", rel_err(linear.bias.grad, wgb))


@pytest.mark.parametrize("use_amp", [True, False], ids=["amp", "noamp"])
@pytest.mark.parametrize("cfg", CONFIGS[:6], ids=[f"b{c[0]}m{c[1]}n{c[2]}k{c[3]}bs{c[4]}" for c in CONFIGS[:6]])
def test_matches_stock_linear_on_dense(cfg, use_amp):
    """The reference's test: sparse round trip of a dense input, projected, against ``linear(dense)``."""
    import blksprs_b200 as bs
    B, m, n, k, bsz, kept = cfg
    g = torch.Generator().manual_seed(7)
    with torch.amp.autocast(device_type="cuda", enabled=use_amp):
        x_d = torch.randn((B, m, k), generator=g).to(DEV)
        layouts = [torch.ones((B, m // bsz, k // bsz), device=DEV), random_layout(B, m // bsz, k // bsz, kept, g).to(DEV)]
        for with_bias in (True, False):
            linear = torch.nn.Linear(k, n, bias=with_bias, device=DEV)
            for layout in layouts:
                x = bs.ops.to_dense(bs.ops.to_sparse(x_d, layout, bsz), layout, bsz)
                x_stock = x.clone().requires_grad_(True)
                x_ours = x.clone().requires_grad_(True)
                stock = linear(x_stock)
                out, out_layout = bs.utils.apply_torch_linear(bs.ops.to_sparse(x_ours, layout, bsz), layout, bsz, linear)
                dense = bs.ops.to_dense(out, out_layout, bsz)
                keep = bs.ops.to_dense(bs.ops.to_sparse(torch.ones_like(dense), out_layout, bsz), out_layout, bsz)
                assert out.dtype == stock.dtype
                assert torch.allclose(dense.to(stock.dtype), stock * keep, atol=4e-2, rtol=2e-2)
                grad = torch.randn_like(stock) * keep
                want = torch.autograd.grad(stock, (x_stock, linear.weight), grad)
                got = torch.autograd.grad(dense, (x_ours, linear.weight), grad)
                # the sparse path has no gradient for input blocks outside the layout
                active = bs.ops.to_dense(bs.ops.to_sparse(torch.ones_like(x), layout, bsz), layout, bsz)
                assert torch.allclose(got[0], want[0] * active, atol=6e-2, rtol=3e-2)
                assert torch.allclose(got[1], want[1], atol=6e-2, rtol=3e-2)


def test_rejects_non_divisible_weight_and_mixed_dtypes():
    import blksprs_b200 as bs
    bsz = 16
    layout = torch.ones((1, 1, 1), dtype=torch.bool, device=DEV)
    x = bs.BlksprsTensor.wrap(torch.zeros((1, bsz, bsz), device=DEV))
    linear = torch.nn.Linear(bsz + 1, bsz, bias=False, device=DEV)
    with pytest.raises(ValueError, match="divisible"):
        bs.utils.apply_torch_linear(x, layout, bsz, linear)
    half = bs.BlksprsTensor.wrap(torch.zeros((1, bsz, bsz), device=DEV, dtype=torch.float16))
    linear = torch.nn.Linear(bsz, bsz, dtype=torch.float32, device=DEV)
    for cached in (False, True):
        with pytest.raises(ValueError, match="same dtype"):
            if cached:
                bs.utils.apply_torch_linear_cached(half, layout, bsz, linear, layout_cache={})
            else:
                bs.utils.apply_torch_linear(half, layout, bsz, linear)
    linear = torch.nn.Linear(2 * bsz, bsz, device=DEV)
    with pytest.raises(ValueError, match="Inner dimensions"):
        bs.utils.apply_torch_linear(x, layout, bsz, linear)


def test_cache_invalidates_for_another_input_layout():
    import blksprs_b200 as bs
    bsz = 16
    first = torch.tensor([[[True], [False]]], device=DEV)
    second = torch.tensor([[[False], [True]]], device=DEV)
    linear = torch.nn.Linear(bsz, bsz, bias=False, device=DEV)
    cache = {}
    dense = torch.zeros((1, 2 * bsz, bsz), device=DEV)
    dense[:, :bsz] = 1
    bs.utils.apply_torch_linear_cached(bs.ops.to_sparse(dense, first, bsz), first, bsz, linear, layout_cache=cache)
    dense.fill_(0)
    dense[:, bsz:] = 2
    sparse = bs.ops.to_sparse(dense, second, bsz)
    got, got_layout = bs.utils.apply_torch_linear_cached(sparse, second, bsz, linear, layout_cache=cache)
    want, want_layout = bs.utils.apply_torch_linear_cached(sparse, second, bsz, linear, layout_cache={})
    assert torch.equal(got_layout, want_layout)
    assert torch.equal(got_layout, second.expand(1, 2, 1))
    assert torch.allclose(got, want)


@pytest.mark.parametrize("parameter_name", ["weight", "bias"])
@pytest.mark.parametrize("initial,updated", [(False, True), (True, False)])
def test_cache_follows_parameter_gradient_state(parameter_name, initial, updated):
    import blksprs_b200 as bs
    bsz = 16
    layout = torch.ones((1, 1, 1), dtype=torch.bool, device=DEV)
    dense = torch.randn((1, bsz, bsz), device=DEV, requires_grad=True)
    sparse = bs.ops.to_sparse(dense, layout, bsz)
    linear = torch.nn.Linear(bsz, bsz, bias=True, device=DEV)
    linear.weight.requires_grad_(parameter_name == "weight" and initial)
    linear.bias.requires_grad_(parameter_name == "bias" and initial)
    cache = {}
    bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache=cache)
    first_weight = cache["w_t_bs"]
    parameter = getattr(linear, parameter_name)
    parameter.requires_grad_(updated)
    parameter.grad = None
    got, _ = bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache=cache)
    want, _ = bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache={})
    assert cache["w_t_bs"] is not first_weight
    if parameter_name == "weight":
        assert cache["w_t_bs"].requires_grad is updated
    assert torch.allclose(got, want)
    got.sum().backward()
    assert (parameter.grad is not None) is updated


@pytest.mark.parametrize("use_bias", [False, True])
def test_cache_rebuilds_after_no_grad_evaluation_and_is_reused_while_training(use_bias):
    import blksprs_b200 as bs
    bsz = 32
    layout = torch.ones((2, 2, 2), dtype=torch.bool, device=DEV)
    linear = torch.nn.Linear(2 * bsz, bsz, bias=use_bias, device=DEV)
    dense = torch.randn((2, 2 * bsz, 2 * bsz), device=DEV, requires_grad=True)
    sparse = bs.ops.to_sparse(dense, layout, bsz)
    cache = {}
    with torch.no_grad():
        bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache=cache)
    evaluation_weight = cache["w_t_bs"]
    assert not evaluation_weight.requires_grad
    out, _ = bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache=cache)
    assert cache["w_t_bs"] is not evaluation_weight and cache["w_t_bs"].requires_grad
    out.sum().backward()
    assert dense.grad is not None and linear.weight.grad is not None
    if use_bias:
        assert linear.bias.grad is not None
    # two more iterations on the same cache: the packed weight is reused and stays differentiable
    training_weight = cache["w_t_bs"]
    for _ in range(2):
        linear.weight.grad = None
        x = bs.ops.to_sparse(torch.randn_like(dense), layout, bsz)
        out, _ = bs.utils.apply_torch_linear_cached(x, layout, bsz, linear, layout_cache=cache)
        out.sum().backward()
        assert cache["w_t_bs"] is training_weight
        assert linear.weight.grad is not None
    # an optimiser step (in-place update) invalidates the packed weight
    with torch.no_grad():
        linear.weight.add_(1.0)
    bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache=cache)
    assert cache["w_t_bs"] is not training_weight


@pytest.mark.parametrize("cached", [False, True])
def test_bias_preserves_autocast_output_dtype_and_gradients(cached):
    import blksprs_b200 as bs
    bsz = 16
    layout = torch.ones((1, 1, 1), dtype=torch.bool, device=DEV)
    linear = torch.nn.Linear(bsz, bsz, bias=True, device=DEV)
    cache = {}
    for _ in range(2):
        dense = torch.randn((1, bsz, bsz), device=DEV, requires_grad=True)
        sparse = bs.ops.to_sparse(dense, layout, bsz)
        with torch.amp.autocast(device_type="cuda", dtype=torch.float16):
            want = linear(dense)
            if cached:
                got, got_layout = bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache=cache)
            else:
                got, got_layout = bs.utils.apply_torch_linear(sparse, layout, bsz, linear)
            got_dense = bs.ops.to_dense(got, got_layout, bsz)
        grad = torch.randn_like(want)
        inputs = (dense, linear.weight, linear.bias)
        want_grads = torch.autograd.grad(want, inputs, grad, retain_graph=True)
        got_grads = torch.autograd.grad(got_dense, inputs, grad)
        assert got.dtype == want.dtype
        assert torch.allclose(got_dense, want, atol=2e-2, rtol=1e-2)
        for a, b in zip(got_grads, want_grads):
            assert torch.allclose(a, b, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("cached", [False, True])
@pytest.mark.parametrize("batch,row_blocks,features", [(1, 2, 0), (1, 0, 16), (0, 2, 16)])
def test_bias_matches_torch_for_empty_dimensions(cached, batch, row_blocks, features):
    import blksprs_b200 as bs
    bsz = 16
    layout = torch.ones((batch, row_blocks, features // bsz), dtype=torch.bool, device=DEV)
    dense = torch.empty((batch, row_blocks * bsz, features), device=DEV, requires_grad=True)
    sparse = bs.ops.to_sparse(dense, layout, bsz)
    linear = torch.nn.Linear(features, bsz, bias=True, device=DEV)
    want = linear(dense)
    if cached:
        got, got_layout = bs.utils.apply_torch_linear_cached(sparse, layout, bsz, linear, layout_cache={})
    else:
        got, got_layout = bs.utils.apply_torch_linear(sparse, layout, bsz, linear)
    got_dense = bs.ops.to_dense(got, got_layout, bsz)
    grad = torch.randn_like(want)
    inputs = (dense, linear.weight, linear.bias)
    want_grads = torch.autograd.grad(want, inputs, grad, retain_graph=True)
    got_grads = torch.autograd.grad(got_dense, inputs, grad)
    assert type(got_layout) is torch.Tensor
    assert got_layout.shape == (batch, row_blocks, 1) and torch.all(got_layout)
    assert torch.allclose(got_dense, want)
    for a, b in zip(got_grads, want_grads):
        assert torch.allclose(a, b, atol=1e-6)


def test_weight_gradient_is_chunked_for_tall_inputs():
    """Many block rows against a small weight: the weight gradient runs as S side-by-side products."""
    import blksprs_b200 as bs
    from blksprs_b200.utils import processing
    bsz, B, R, K, N = 64, 16, 24, 4, 2
    g = torch.Generator().manual_seed(11)
    layout = random_layout(B, R, K, 0.5, g)
    x = torch.randn((int(layout.sum()), bsz, bsz), generator=g).to(torch.bfloat16)
    linear = torch.nn.Linear(K * bsz, N * bsz, bias=True).to(torch.bfloat16)
    want, want_layout = oracle.linear(x, layout, bsz, linear.weight.detach(), linear.bias.detach())
    grad = torch.randn(want.shape, generator=g).to(torch.bfloat16)
    wgx, wgw, wgb = oracle.linear_backward(grad, want_layout, x, layout, bsz, linear.weight.detach(), True)
    linear = linear.to(DEV)
    cache = {}
    out, _ = bs.utils.apply_torch_linear_cached(x.to(DEV), layout.to(DEV), bsz, linear, layout_cache=cache)
    out.backward(grad.to(DEV))
    chunks = cache[processing._PLANS].chunks
    assert chunks > 1 and (B * R) % chunks == 0 and chunks * K * N >= processing._MIN_GRAD_W_BLOCKS
    assert rel_err(out.detach(), want) <= 1e-2
    assert rel_err(linear.weight.grad, wgw) <= 1e-2
    assert rel_err(linear.bias.grad, wgb) <= 1e-2


@pytest.mark.parametrize("bias", [False, True], ids=["nobias", "bias"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_matches_reference_package(dtype, bias):
    if not os.path.isdir(os.path.join(REF_DIR, "blksprs")):
        pytest.skip("reference package not installed under baseline/_ref")
    os.environ.setdefault("BLKSPRS_AUTOTUNE", "TEST")
    sys.path.insert(0, REF_DIR)
    try:
        import blksprs as ref
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference not importable: {exc!r}")
    finally:
        sys.path.remove(REF_DIR)
    import blksprs_b200 as ours
    B, m, n, k, bsz, kept = 3, 256, 128, 192, 64, 0.5
    layout, x, linear = _case(B, m, n, k, bsz, kept, dtype, seed=21, bias=bias)
    linear = linear.to(DEV)
    grad = None
    results = []
    for lib in (ref, ours):
        linear.zero_grad(set_to_none=True)
        xd = x.to(DEV).requires_grad_(True)
        out, out_layout = lib.utils.apply_torch_linear_cached(xd, layout.to(DEV), bsz, linear, layout_cache={})
        if grad is None:
            grad = torch.randn(out.shape, generator=torch.Generator().manual_seed(2)).to(dtype).to(DEV)
        out.backward(grad)
        results.append([t.detach().as_subclass(torch.Tensor).clone() for t in
                        (out, out_layout, xd.grad, linear.weight.grad) + ((linear.bias.grad,) if bias else ())])
    r, o = results
    assert torch.equal(r[1], o[1])
    for a, b, what in zip(o[:1] + o[2:], r[:1] + r[2:], ("out", "grad_x", "grad_w", "grad_b")):
        assert a.shape == b.shape and a.dtype == b.dtype
        assert rel_err(a, b.cpu()) <= _tol(dtype), (what, rel_err(a, b.cpu()))
