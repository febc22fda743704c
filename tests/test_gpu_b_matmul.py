"""bs.ops.matmul forward + backward on the GPU against the CPU oracle and the reference vectors."""
import numpy as np
import pytest
import torch

import cases
from gpu_util import DEV, check_case, make_case, oracle_tolerance, rel_err, run_ours
from oracle import oracle

pytestmark = pytest.mark.gpu

# (batch, m, n, k, block size, kept fraction): the shape matrix of the reference's op tests
# (test/cases/test_blocksparse.py:21-84), duplicates removed.
SHAPES = [
    (2, 64, 64, 64, 64, 0), (2, 16, 16, 16, 16, .75), (2, 32, 32, 32, 32, .75), (2, 64, 64, 64, 64, .75),
    (2, 64, 64, 64, 64, 1), (2, 64, 64, 64, 16, .75), (2, 64, 64, 64, 32, .75), (2, 128, 128, 128, 64, 0),
    (2, 128, 128, 128, 16, .75), (2, 128, 128, 128, 32, .75), (2, 128, 128, 128, 64, .75),
    (2, 128, 128, 128, 64, 1), (2, 2048, 2048, 128, 64, .75), (2, 128, 128, 128, 32, 0),
    (16, 64, 32, 64, 32, .75), (16, 32, 64, 64, 32, .75), (8, 128, 64, 128, 64, .75), (8, 64, 128, 128, 64, .75),
    (4, 256, 128, 128, 64, 0), (4, 256, 128, 128, 64, .75), (4, 256, 128, 128, 64, 1), (4, 128, 256, 128, 64, .75),
    (2, 4096, 1024, 128, 64, .75), (2, 1024, 4096, 128, 64, .75), (2, 128, 128, 128, 64, .5),
    (2, 128, 128, 128, 64, .25), (2, 128, 128, 128, 64, .1), (2, 256, 128, 64, 32, .1), (2, 128, 256, 64, 32, .1),
    (2, 128, 128, 128, 16, .015625), (2, 64, 64, 64, 32, 0), (2, 64, 64, 64, 32, 1), (1, 64, 64, 64, 32, .25),
    (3, 112, 80, 48, 16, 0), (3, 112, 80, 48, 16, .25), (3, 112, 80, 48, 16, .5), (5, 112, 80, 48, 16, .75),
    (7, 112, 80, 48, 16, 1), (3, 224, 160, 96, 32, 0), (3, 224, 160, 96, 32, .25), (3, 224, 160, 96, 32, .5),
    (5, 224, 160, 96, 32, .75), (7, 224, 160, 96, 32, 1), (3, 448, 320, 192, 64, 0), (3, 448, 320, 192, 64, .25),
    (3, 448, 320, 192, 64, .5), (5, 448, 320, 192, 64, .75), (7, 448, 320, 192, 64, 1),
    # block 128 (not in the reference matrix; the multi-GPU workload uses it)
    (2, 256, 256, 256, 128, .75), (3, 384, 256, 512, 128, .5), (2, 128, 128, 128, 128, 1),
]


@pytest.fixture(params=["auto", "mma", "umma", "panel"])
def kernel_family(request):
    from blksprs_b200 import plan
    previous = plan._kernel_choice
    plan.set_kernel(request.param)
    yield request.param
    plan._kernel_choice = previous


@pytest.mark.parametrize("shape", SHAPES, ids=[f"{i}-b{s[0]}m{s[1]}n{s[2]}k{s[3]}bs{s[4]}p{s[5]}" for i, s in enumerate(SHAPES)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["fp32", "fp16", "bf16"])
def test_matmul_matrix(shape, dtype, kernel_family):
    B, m, n, k, bs, kept = shape
    if kernel_family != "auto" and bs < 64:
        pytest.skip("auto already selects the mma.sync kernel here")
    for i, out_layout in enumerate(("fast", "ones", "exact")):
        check_case(make_case(B, m, n, k, bs, kept, dtype, seed=1000 + i, out_layout=out_layout))


@pytest.mark.parametrize("name,case", cases.matmul_cases(), ids=[n for n, _ in cases.matmul_cases()])
def test_reference_kernel_vectors(golden, name, case):
    """Same inputs as the reference's own Triton kernels were given (recorded under the interpreter)."""
    out, gx, gy = run_ours(case)
    tol = oracle_tolerance(case["x"].dtype)  # the recorded vectors are IEEE fp32 (Triton interpreter)
    assert rel_err(out, torch.from_numpy(golden[f"matmul/{name}/out"])) <= tol
    assert rel_err(gx, torch.from_numpy(golden[f"matmul/{name}/grad_x"])) <= tol
    assert rel_err(gy, torch.from_numpy(golden[f"matmul/{name}/grad_y"])) <= tol


@pytest.mark.parametrize("use_amp", [True, False])
def test_autocast_and_float_layouts(use_amp):
    """Dense operands with float32 all-ones layouts under autocast (test/cases/test_blocksparse.py:449-504)."""
    import blksprs_b200 as bs
    g = torch.Generator().manual_seed(7)
    B, m, n, k, bsz = 2, 128, 64, 128, 32
    x = torch.randn((B * (m // bsz) * (k // bsz), bsz, bsz), generator=g)
    y = torch.randn((B * (k // bsz) * (n // bsz), bsz, bsz), generator=g)
    lx = torch.ones((B, m // bsz, k // bsz))
    ly = torch.ones((B, k // bsz, n // bsz))
    lo = torch.ones((B, m // bsz, n // bsz))
    xd, yd = x.to(DEV).requires_grad_(True), y.to(DEV).requires_grad_(True)
    with torch.amp.autocast(device_type="cuda", enabled=use_amp):
        out = bs.ops.matmul(xd, lx.to(DEV), yd, ly.to(DEV), lo.to(DEV), bsz)
    assert out.dtype == (torch.float16 if use_amp else torch.float32)
    assert isinstance(out, bs.BlksprsTensor)
    grad = torch.randn(out.shape, generator=g)
    out.backward(grad.to(DEV).to(out.dtype))
    cast = (lambda t: t.half()) if use_amp else (lambda t: t)
    want = oracle.matmul_forward(cast(x), lx, cast(y), ly, lo, bsz)
    wgx, wgy = oracle.matmul_backward(cast(grad), cast(x), lx, cast(y), ly, lo, bsz)
    tol = oracle_tolerance(torch.float16 if use_amp else torch.float32)
    assert rel_err(out, want) <= tol
    assert xd.grad.dtype == torch.float32 and rel_err(xd.grad, wgx) <= tol
    assert rel_err(yd.grad, wgy) <= tol


def test_empty_output_layout_and_empty_operands():
    import blksprs_b200 as bs
    bsz = 32
    lx = torch.zeros((2, 2, 2), dtype=torch.bool, device=DEV)
    lo = torch.zeros((2, 2, 2), dtype=torch.bool, device=DEV)
    x = torch.zeros((0, bsz, bsz), device=DEV, requires_grad=True)
    out = bs.ops.matmul(x, lx, x, lx, lo, bsz)
    assert out.shape == (0, bsz, bsz)
    # active output blocks, no operand blocks: zeros
    lo1 = torch.ones((2, 2, 2), dtype=torch.bool, device=DEV)
    out = bs.ops.matmul(x, lx, x, lx, lo1, bsz)
    assert out.shape == (8, bsz, bsz) and float(out.abs().max()) == 0.0
    out.sum().backward()
    assert x.grad.shape == (0, bsz, bsz)


def test_blocks_without_shared_inner_block_are_zero():
    """The output layout is an input: active blocks with no common k must be written as zeros."""
    import blksprs_b200 as bs
    for bsz, dtype in ((16, torch.float32), (64, torch.bfloat16), (128, torch.float16)):
        lx = torch.tensor([[[1, 0], [0, 1]]], dtype=torch.bool)
        ly = torch.tensor([[[1, 0], [0, 1]]], dtype=torch.bool)
        lo = torch.ones((1, 2, 2), dtype=torch.bool)
        g = torch.Generator().manual_seed(3)
        x = torch.randn((2, bsz, bsz), generator=g).to(dtype)
        y = torch.randn((2, bsz, bsz), generator=g).to(dtype)
        out = bs.ops.matmul(x.to(DEV), lx.to(DEV), y.to(DEV), ly.to(DEV), lo.to(DEV), bsz)
        want = oracle.matmul_forward_blocks(x, lx, y, ly, lo, bsz)
        assert float(out[1].abs().max()) == 0.0 and float(out[2].abs().max()) == 0.0
        assert rel_err(out, want) <= oracle_tolerance(dtype)


def test_non_contiguous_inputs_are_made_contiguous():
    import blksprs_b200 as bs
    case = make_case(2, 64, 64, 64, 32, 0.75, torch.float32, seed=5)
    x = case["x"].to(DEV)
    wide = torch.zeros((x.size(0), 32, 64), device=DEV)
    wide[:, :, :32] = x
    out = bs.ops.matmul(wide[:, :, :32], case["lx"].to(DEV), case["y"].to(DEV), case["ly"].to(DEV),
                        case["lo"].to(DEV), 32)
    want = oracle.matmul_forward(case["x"], case["lx"], case["y"], case["ly"], case["lo"], 32)
    assert rel_err(out, want) <= oracle_tolerance(torch.float32)


def test_deterministic_run_to_run():
    """No atomics on this path: two runs give identical bits (a cheap race detector)."""
    case = make_case(3, 448, 320, 192, 64, 0.5, torch.bfloat16, seed=9, out_layout="ones")
    a = run_ours(case)
    b = run_ours(case)
    for u, v in zip(a, b):
        assert torch.equal(u, v)


def test_layout_cache_reuse_and_invalidation():
    import blksprs_b200 as bs
    case = make_case(2, 128, 128, 128, 32, 0.5, torch.float32, seed=11)
    lx, ly, lo = (case[k].to(DEV) for k in ("lx", "ly", "lo"))
    x, y = case["x"].to(DEV), case["y"].to(DEV)
    cache = {}
    out1 = bs.ops.matmul(x, lx, y, ly, lo, 32, cache)
    lut_id = id(cache["layout_indices_o"])
    assert set(cache) >= {"packed_indices_x", "packed_indices_y", "layout_indices_o", "n_sparse_blocks"}
    assert isinstance(cache["n_sparse_blocks"], int)
    out2 = bs.ops.matmul(x, lx, y, ly, lo, 32, cache)
    assert id(cache["layout_indices_o"]) == lut_id and torch.equal(out1, out2)
    # a different (equal-valued) layout object rebuilds the cache
    bs.ops.matmul(x, lx.clone(), y, ly, lo, 32, cache)
    assert id(cache["layout_indices_o"]) != lut_id
    # an in-place mutation of a layout bumps its version and rebuilds too
    lut_id = id(cache["layout_indices_o"])
    lo2 = lo.clone()
    cache2 = {}
    bs.ops.matmul(x, lx, y, ly, lo2, 32, cache2)
    before = id(cache2["layout_indices_o"])
    lo2.logical_or_(lo2)
    bs.ops.matmul(x, lx, y, ly, lo2, 32, cache2)
    assert id(cache2["layout_indices_o"]) != before


def test_error_contract():
    """Exception types and messages of the reference (test_blocksparse.py:507-516, 1335-1421;
    test_regressions.py:694-711, 963-971, 1327-1346)."""
    import blksprs_b200 as bs
    bsz = 16
    ones = lambda *s: torch.ones(s, dtype=torch.bool, device=DEV)
    blk = lambda n, dt=torch.float32: torch.zeros((n, bsz, bsz), device=DEV, dtype=dt)
    with pytest.raises(ValueError, match="Output sparsity layout shape"):
        bs.ops.matmul(blk(2), ones(2, 1, 1), blk(2), ones(2, 1, 1), ones(2, 2, 1), bsz)
    with pytest.raises(ValueError, match="Batch dimensions"):
        bs.ops.matmul(blk(2), ones(2, 1, 1), blk(1), ones(1, 1, 1), ones(2, 1, 1), bsz)
    with pytest.raises(ValueError, match="Inner dimensions"):
        bs.ops.matmul(blk(2), ones(1, 1, 2), blk(1), ones(1, 1, 1), ones(1, 1, 1), bsz)
    with pytest.raises(ValueError, match="float16, bfloat16, or float32"):
        with torch.amp.autocast(device_type="cuda"):
            bs.ops.matmul(blk(1, torch.float64), ones(1, 1, 1), blk(1, torch.float64), ones(1, 1, 1), ones(1, 1, 1), bsz)
    with pytest.raises(ValueError, match="same dtype"):
        bs.ops.matmul(blk(1), ones(1, 1, 1), blk(1, torch.float16), ones(1, 1, 1), ones(1, 1, 1), bsz)
    with pytest.raises(ValueError, match="dimensions"):
        bs.ops.matmul(blk(1)[0], ones(1, 1, 1), blk(1), ones(1, 1, 1), ones(1, 1, 1), bsz)
    with pytest.raises(ValueError, match="GPU"):
        bs.ops.matmul(blk(1).cpu(), ones(1, 1, 1), blk(1).cpu(), ones(1, 1, 1), ones(1, 1, 1).cpu(), bsz)
    with pytest.raises(ValueError, match="Mismatch between sparsity layout and blocks"):
        bs.ops.matmul(blk(2), ones(1, 1, 1), blk(1), ones(1, 1, 1), ones(1, 1, 1), bsz)
    with pytest.raises(ValueError, match="0 or 1"):
        bs.ops.matmul(blk(1), 2 * torch.ones((1, 1, 1), device=DEV), blk(1), ones(1, 1, 1), ones(1, 1, 1), bsz)
    with pytest.raises(ValueError, match="complex"):
        bs.ops.matmul(blk(1), torch.ones((1, 1, 1), device=DEV, dtype=torch.complex64), blk(1), ones(1, 1, 1),
                      ones(1, 1, 1), bsz)
    with pytest.raises(ValueError, match="at least 16"):
        bs.ops.matmul(torch.zeros((1, 8, 8), device=DEV), ones(1, 1, 1), torch.zeros((1, 8, 8), device=DEV),
                      ones(1, 1, 1), ones(1, 1, 1), 8)
    with pytest.raises(ValueError, match="power of 2"):
        bs.ops.matmul(torch.zeros((1, 24, 24), device=DEV), ones(1, 1, 1), torch.zeros((1, 24, 24), device=DEV),
                      ones(1, 1, 1), ones(1, 1, 1), 24)
    with pytest.raises(TypeError, match="integer"):
        bs.ops.matmul(blk(1), ones(1, 1, 1), blk(1), ones(1, 1, 1), ones(1, 1, 1), 16.0)
    with pytest.raises(ValueError, match="Batch dimensions"):
        bs.layouting.build_sparsity_layout_matmul(ones(2, 2, 2), ones(3, 2, 2))
    with pytest.raises(ValueError, match="Inner dimensions"):
        bs.layouting.build_sparsity_layout_matmul_fast(ones(2, 2, 3), ones(2, 2, 2))
    with pytest.raises(ValueError, match="0 or 1"):
        bs.layouting.build_sparsity_layout_matmul_outer(3 * torch.ones((1, 1, 1), device=DEV), ones(1, 1, 1))
    # switches
    bs.utils.disable_validation()
    try:
        out = bs.ops.matmul(blk(1), ones(1, 1, 1), blk(1), ones(1, 1, 1), ones(1, 1, 1), bsz)
        assert out.shape == (1, bsz, bsz)
    finally:
        bs.utils.enable_validation()
    bs.utils.disable_contiguous()
    try:
        with pytest.raises(ValueError, match="contiguous"):
            bs.ops.matmul(torch.zeros((1, bsz, 2 * bsz), device=DEV)[:, :, :bsz], ones(1, 1, 1), blk(1),
                          ones(1, 1, 1), ones(1, 1, 1), bsz)
    finally:
        bs.utils.enable_contiguous()


def test_layout_helpers_return_base_tensors():
    import blksprs_b200 as bs

    class Sub(torch.Tensor):
        pass

    lx = torch.ones((1, 2, 2), dtype=torch.bool, device=DEV).as_subclass(Sub)
    out = bs.layouting.build_sparsity_layout_matmul(lx, lx)
    assert type(out) is torch.Tensor


def test_transpose_matches_oracle_and_backward():
    import blksprs_b200 as bs
    for bsz, dtype in ((16, torch.float32), (32, torch.float16), (64, torch.bfloat16), (128, torch.float32)):
        layout = cases.bernoulli_layout((3, 3, 5), 0.6, 60 + bsz)
        g = torch.Generator().manual_seed(bsz)
        x = torch.randn((int(layout.sum()), bsz, bsz), generator=g).to(dtype)
        xd = x.to(DEV).requires_grad_(True)
        out, layout_t = bs.ops.transpose(xd, layout.to(DEV), bsz)
        want, want_layout = oracle.transpose(x, layout, bsz)
        assert np.array_equal(layout_t.cpu().numpy(), want_layout)
        assert torch.equal(out.detach().cpu(), want)
        assert layout_t.data_ptr() != layout.data_ptr()
        grad = torch.randn(out.shape, generator=g).to(dtype)
        out.backward(grad.to(DEV))
        want_grad, _ = oracle.transpose(grad, want_layout, bsz)
        assert torch.equal(xd.grad.cpu(), want_grad)


def test_torch_compile_wrapper_runs():
    """torch.compile(bs.ops.matmul) with graph breaks allowed (README usage of the reference)."""
    import blksprs_b200 as bs
    case = make_case(2, 64, 64, 64, 32, 1, torch.float32, seed=13)
    fn = torch.compile(bs.ops.matmul)
    out = fn(case["x"].to(DEV), case["lx"].to(DEV), case["y"].to(DEV), case["ly"].to(DEV), case["lo"].to(DEV), 32)
    want = oracle.matmul_forward(case["x"], case["lx"], case["y"], case["ly"], case["lo"], 32)
    assert rel_err(out, want) <= oracle_tolerance(torch.float32)


@pytest.mark.parametrize("schedule", ["dynamic", "static"])
def test_one_plan_on_two_streams_and_both_schedules(schedule, monkeypatch):
    """The same layout cache used from two CUDA streams at once (each stream has its own scheduling
    counters), under the counter-driven and the round-robin hand-out of units."""
    import blksprs_b200 as bs
    from blksprs_b200 import plan
    monkeypatch.setattr(plan, "SCHEDULE", schedule)
    case = make_case(16, 1024, 1024, 1024, 64, 0.5, torch.bfloat16, seed=31, out_layout="exact")
    want = oracle.matmul_forward(case["x"], case["lx"], case["y"], case["ly"], case["lo"], 64)
    lx, ly, lo = (case[k].to(DEV) for k in ("lx", "ly", "lo"))
    x, y = case["x"].to(DEV), case["y"].to(DEV)
    cache = {}
    first = bs.ops.matmul(x, lx, y, ly, lo, 64, cache)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(DEV), torch.cuda.Stream(DEV)]
    outs = [[], []]
    for _ in range(8):
        for s, acc in zip(streams, outs):
            with torch.cuda.stream(s):
                acc.append(bs.ops.matmul(x, lx, y, ly, lo, 64, cache))
    torch.cuda.synchronize()
    plan.check_device_status(torch.device(DEV))
    assert rel_err(first, want) <= oracle_tolerance(torch.bfloat16)
    for acc in outs:
        for out in acc:
            assert torch.equal(out, first)


def test_bounded_wait_expires_with_a_status_instead_of_hanging():
    """Failure detection without a GPU fault: a wait that nothing satisfies runs out after its limit,
    the kernel returns, the status word says BSP_ERR_DEVICE_TIMEOUT and the context stays usable."""
    from blksprs_b200 import _cabi
    lib = _cabi.lib()
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    _cabi.check(lib.bsp_selftest_wait_limit(20000, word.data_ptr(), _cabi.stream_handle(torch.device(DEV))),
                "bsp_selftest_wait_limit")
    torch.cuda.synchronize()
    assert int(word.item()) == _cabi.ERR_DEVICE_TIMEOUT
    assert lib.bsp_selftest_wait_limit(0, word.data_ptr(), None) == _cabi.ERR_INVALID_ARG
    # the device still works
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0


def test_calls_without_a_cache_reuse_library_owned_metadata():
    """``layout_cache=None`` (the reference's default) does not rebuild LUTs and plans on every call: a small
    library-owned cache with the caller-cache reuse rule serves repeated calls on the same layout objects."""
    import blksprs_b200 as bs
    from blksprs_b200.ops.matmul import _PLANS
    from blksprs_b200.utils import tools
    case = make_case(2, 256, 192, 128, 64, 0.5, torch.bfloat16, seed=31, out_layout="exact")
    lx, ly, lo = (case[k].to(DEV) for k in ("lx", "ly", "lo"))
    x, y = case["x"].to(DEV), case["y"].to(DEV)
    tools.clear_implicit_layout_caches()
    first = bs.ops.matmul(x, lx, y, ly, lo, 64)
    entry = tools.implicit_layout_cache("matmul", lx, ly, lo)
    plans = entry[_PLANS]
    second = bs.ops.matmul(x, lx, y, ly, lo, 64)
    assert torch.equal(first, second)
    assert tools.implicit_layout_cache("matmul", lx, ly, lo)[_PLANS] is plans          # reused, not rebuilt
    # wrong block count on a warm entry: the reference's message, without a device read
    with pytest.raises(ValueError, match="Mismatch between sparsity layout and blocks"):
        bs.ops.matmul(x[:-1], lx, y, ly, lo, 64)
    lo.logical_or_(lo)                                                                 # same content, new version
    third = bs.ops.matmul(x, lx, y, ly, lo, 64)
    assert torch.equal(first, third)
    assert tools.implicit_layout_cache("matmul", lx, ly, lo)[_PLANS] is not plans      # rebuilt for the new version
    bs.utils.set_implicit_layout_caches(False)
    try:
        fourth = bs.ops.matmul(x, lx, y, ly, lo, 64)
        assert torch.equal(first, fourth)
        assert tools.implicit_layout_cache("matmul", lx, ly, lo) is None
    finally:
        bs.utils.set_implicit_layout_caches(True)


@pytest.mark.parametrize("bs,dtype", [(16, torch.bfloat16), (32, torch.float32), (64, torch.bfloat16)])
def test_operands_that_start_off_a_16_byte_boundary(bs, dtype):
    """A contiguous view into the middle of a larger buffer may start at any element; the kernels move
    16-byte vectors.  The op gives the same bits as with aligned operands (it copies such an operand
    first), and the C entry point refuses a misaligned pointer instead of launching."""
    import blksprs_b200 as bsp
    from blksprs_b200 import _cabi, plan
    from blksprs_b200.ops.matmul import matmul_build_layout_cache, _PLANS
    case = make_case(2, 4 * bs, 4 * bs, 4 * bs, bs, 0.6, dtype, seed=17)
    lx, ly, lo = (case[k].to(DEV) for k in ("lx", "ly", "lo"))
    x, y = case["x"].to(DEV), case["y"].to(DEV)

    def shifted(t):
        base = torch.zeros(t.numel() + 8, dtype=t.dtype, device=t.device)
        view = base[1:1 + t.numel()].view(t.shape)
        view.copy_(t)
        assert view.is_contiguous() and view.data_ptr() % 16 != 0
        return view

    want = bsp.ops.matmul(x, lx, y, ly, lo, bs)
    got = bsp.ops.matmul(shifted(x), lx, shifted(y), ly, lo, bs)
    assert torch.equal(got, want)
    xs, ys = shifted(x).requires_grad_(True), shifted(y).requires_grad_(True)
    g = shifted(case["grad"].to(DEV))
    bsp.ops.matmul(xs, lx, ys, ly, lo, bs).backward(g)
    xa, ya = x.clone().requires_grad_(True), y.clone().requires_grad_(True)
    bsp.ops.matmul(xa, lx, ya, ly, lo, bs).backward(case["grad"].to(DEV))
    assert torch.equal(xs.grad, xa.grad) and torch.equal(ys.grad, ya.grad)
    # the C entry point itself: no launch, an error code
    product = matmul_build_layout_cache(None, lx, ly, lo)[_PLANS].forward
    p = product.pair
    out = torch.empty((p.n_out, bs, bs), dtype=dtype, device=DEV)
    status = _cabi.lib().bsp_matmul_mma(
        shifted(x).data_ptr(), x.size(0), y.data_ptr(), y.size(0), out.data_ptr(), p.n_out, p.offsets.data_ptr(),
        p.pairs.data_ptr(), bs, _cabi.DATA_DTYPE_CODES[dtype], p.op, plan.status_word(x.device).data_ptr(),
        _cabi.stream_handle(x.device))
    assert status == _cabi.ERR_INVALID_ARG
    torch.cuda.synchronize()
