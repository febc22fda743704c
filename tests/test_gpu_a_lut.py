"""LUT, reverse LUT and inferred layouts from the CUDA library: bit-exact against the reference vectors."""
import numpy as np
import pytest
import torch

import cases
from gpu_util import DEV
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,layout", cases.lut_layouts(), ids=[n for n, _ in cases.lut_layouts()])
def test_luts_bit_exact(golden, name, layout):
    from blksprs_b200.utils import tools
    dev = layout.to(DEV)
    lut = tools.build_layout_indices(dev)
    packed = tools.build_packed_indices(dev)
    assert type(lut) is torch.Tensor and lut.dtype == torch.int64 and lut.is_contiguous()
    assert packed.dtype == torch.int64 and packed.dim() == 1
    assert np.array_equal(lut.cpu().numpy(), golden[f"lut/{name}/layout_indices"])
    assert np.array_equal(packed.cpu().numpy(), golden[f"lut/{name}/packed_indices"])
    assert tools.count_active_blocks(dev) == int(golden[f"lut/{name}/n_sparse_blocks"])


def test_luts_bfloat16_layout():
    from blksprs_b200.utils import tools
    layout = cases.bernoulli_layout((3, 9, 11), 0.4, 50)
    dev = layout.to(torch.bfloat16).to(DEV)
    assert np.array_equal(tools.build_layout_indices(dev).cpu().numpy(), oracle.layout_indices(layout))
    assert np.array_equal(tools.build_packed_indices(dev).cpu().numpy(), oracle.packed_indices(layout))


@pytest.mark.parametrize("name,lx,ly", cases.layout_pairs(), ids=[n for n, _, _ in cases.layout_pairs()])
def test_layout_inference_bit_exact(golden, name, lx, ly):
    import blksprs_b200 as bs
    for fn, key in ((bs.layouting.build_sparsity_layout_matmul, "exact"),
                    (bs.layouting.build_sparsity_layout_matmul_fast, "fast"),
                    (bs.layouting.build_sparsity_layout_matmul_outer, "outer")):
        got = fn(lx.to(DEV), ly.to(DEV))
        assert type(got) is torch.Tensor and got.dtype == torch.bool
        assert np.array_equal(got.cpu().numpy(), golden[f"infer/{name}/{key}"]), key


def test_benchmark_layouts_bit_exact(golden):
    """Config-2 sized layouts: LUT digests recorded from the reference."""
    import hashlib
    import blksprs_b200 as bs
    from blksprs_b200.ops.matmul import matmul_build_layout_cache

    def digest(t):
        return hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()

    for name, lx, ly in cases.big_layout_pairs():
        lx, ly = lx.to(DEV), ly.to(DEV)
        lo = bs.layouting.build_sparsity_layout_matmul(lx, ly)
        cache = matmul_build_layout_cache(None, lx, ly, lo)
        got = [digest(cache["packed_indices_x"]), digest(cache["packed_indices_y"]),
               digest(cache["layout_indices_o"]), digest(lo.to(torch.uint8))]
        assert got == list(golden[f"big/{name}/digest"])
        assert cache["n_sparse_blocks"] == int(golden[f"big/{name}/n_sparse_blocks"])


def test_exact_layout_is_subset_of_fast():
    """test/cases/test_blocksparse.py:1011-1022."""
    import blksprs_b200 as bs
    lx = cases.bernoulli_layout((4, 16, 12), 0.2, 51).to(DEV)
    ly = cases.bernoulli_layout((4, 12, 20), 0.2, 52).to(DEV)
    exact = bs.layouting.build_sparsity_layout_matmul(lx, ly)
    fast = bs.layouting.build_sparsity_layout_matmul_fast(lx, ly)
    outer = bs.layouting.build_sparsity_layout_matmul_outer(lx, ly)
    assert bool(torch.all(fast | ~exact)) and bool(torch.all(outer | ~fast))


def test_large_layout_helpers():
    """4096 x 512 x 1 layouts (test/cases/test_blocksparse.py:2523-2549), against the oracle."""
    import blksprs_b200 as bs
    lx = cases.bernoulli_layout((64, 512, 1), 0.5, 53)
    ly = cases.bernoulli_layout((64, 1, 4), 0.5, 54)
    for fn, ofn in ((bs.layouting.build_sparsity_layout_matmul, oracle.layout_matmul),
                    (bs.layouting.build_sparsity_layout_matmul_fast, oracle.layout_matmul_fast),
                    (bs.layouting.build_sparsity_layout_matmul_outer, oracle.layout_matmul_outer)):
        assert np.array_equal(fn(lx.to(DEV), ly.to(DEV)).cpu().numpy(), ofn(lx, ly))


def test_pair_plan_matches_oracle():
    from blksprs_b200.ops.matmul import matmul_build_layout_cache, _backward_plans, _PLANS
    lx = cases.bernoulli_layout((3, 7, 9), 0.4, 55)
    ly = cases.bernoulli_layout((3, 9, 5), 0.4, 56)
    lo = cases.bernoulli_layout((3, 7, 5), 0.6, 57)
    cache = matmul_build_layout_cache(None, lx.to(DEV), ly.to(DEV), lo.to(DEV))
    plans = cache[_PLANS]
    _backward_plans(plans, cache["packed_indices_x"], cache["packed_indices_y"], int(lx.sum()), int(ly.sum()))
    px = oracle.packed_indices(lx).reshape(lx.shape)
    py = oracle.packed_indices(ly).reshape(ly.shape)
    po = oracle.packed_indices(lo).reshape(lo.shape)

    def expect(lut, fa, fb, T):
        offs, pairs = [0], []
        for b, r, c in lut:
            for t in range(T):
                ia, ib = fa(b, r, c, t), fb(b, r, c, t)
                if ia >= 0 and ib >= 0:
                    pairs.append((ia, ib))
            offs.append(len(pairs))
        return np.array(offs), np.array(pairs).reshape(-1, 2)

    checks = [
        (plans.forward, oracle.layout_indices(lo), lambda b, i, j, t: px[b, i, t], lambda b, i, j, t: py[b, t, j], 9),
        (plans.grad_x, oracle.layout_indices(lx), lambda b, i, k, t: po[b, i, t], lambda b, i, k, t: py[b, k, t], 5),
        (plans.grad_y, oracle.layout_indices(ly), lambda b, k, j, t: px[b, t, k], lambda b, k, j, t: po[b, t, j], 7),
    ]
    for product, lut, fa, fb, T in checks:
        plan = product.pair
        offs, pairs = expect(lut, fa, fb, T)
        assert np.array_equal(plan.offsets.cpu().numpy(), offs)
        assert plan.n_pairs == len(pairs)
        got = plan.pairs.cpu().numpy()[:plan.n_pairs]
        assert np.array_equal(got & np.array([0x3fffffff, -1]), pairs)
        # bit 30 of the a-index marks the last pair of every non-empty output block
        last = np.zeros(len(pairs), dtype=bool)
        last[offs[1:][np.diff(offs) > 0] - 1] = True
        assert np.array_equal((got[:, 0] >> 30) & 1, last.astype(got.dtype))
        # step plans: single-block steps reproduce the pairs; two-block panels cover them exactly
        for width in (1, 2):
            sp = product.step_plan(64, torch.bfloat16, width)
            steps = sp.steps.cpu().numpy()[:sp.n_steps]
            first = sp.panel_first.cpu().numpy()
            so = sp.step_offsets.cpu().numpy()
            up = sp.unit_panel.cpu().numpy()
            assert up[0] == 0 and up[-1] == sp.n_panels and np.all(np.diff(up) >= 0)
            assert np.array_equal(sp.unit_step.cpu().numpy(), so[up])
            rebuilt = [[] for _ in range(plan.n_out)]
            for pn in range(sp.n_panels):
                g = first[pn + 1] - first[pn]
                assert 1 <= g <= width
                seen = 0
                for s in range(so[pn], so[pn + 1]):
                    a_blk, ctrl = steps[s, 0], steps[s, 5]
                    present, fresh = ctrl & 0xF, (ctrl >> 4) & 0xF
                    assert present != 0 and (present >> g) == 0 and fresh == (present & ~seen)
                    assert bool(ctrl & 0x100) == (s == so[pn + 1] - 1) and ((ctrl >> 12) & 7) == g
                    seen |= present
                    for q in range(g):
                        if (present >> q) & 1:
                            rebuilt[first[pn] + q].append((a_blk, steps[s, 1 + q]))
                assert seen == sp.touched.cpu().numpy()[pn]
            flat = [p for blk in rebuilt for p in blk]
            assert np.array_equal(np.array(flat).reshape(-1, 2), pairs)
            assert [len(b) for b in rebuilt] == list(np.diff(offs))


def test_single_block_plan_taken_from_the_two_block_walk():
    """The automatic choice walks the LUTs once, for panels of two blocks; when it settles on single-block
    steps, their counts come out of that walk (per-block pair counts) instead of a second one.  The plan
    built that way equals the one counted directly, entry for entry, for all three products."""
    from blksprs_b200 import _cabi, plan
    from blksprs_b200.ops.matmul import matmul_build_layout_cache, _backward_plans, _PLANS
    lx = cases.bernoulli_layout((3, 9, 11), 0.35, 61)
    ly = cases.bernoulli_layout((3, 11, 7), 0.35, 62)
    lo = cases.bernoulli_layout((3, 9, 7), 0.7, 63)
    n_x, n_y = int(lx.sum()), int(ly.sum())

    def products():
        cache = matmul_build_layout_cache(None, lx.to(DEV), ly.to(DEV), lo.to(DEV))
        plans = cache[_PLANS]
        _backward_plans(plans, cache["packed_indices_x"], cache["packed_indices_y"], n_x, n_y)
        return plans.forward, plans.grad_x, plans.grad_y

    old_ratio = plan.PANEL_STEP_RATIO
    plan.PANEL_STEP_RATIO = 0.0   # two-block panels never pay off: the automatic choice falls to width 1
    try:
        derived = []
        for product in products():
            assert product.choose(64, torch.bfloat16, 5, 5) == ("umma", 1)
            assert 2 in product._counted and product._counted[1].block_counts is None
            derived.append(product.step_plan(64, torch.bfloat16, 1))
    finally:
        plan.PANEL_STEP_RATIO = old_ratio
    for got, product in zip(derived, products()):
        n_ctas = _cabi.lib().bsp_umma_num_ctas(_cabi.DATA_DTYPE_CODES[torch.bfloat16], 64, 1)
        want = plan.build_step_plan(product.op, product.lut_out, product.packed_a, product.packed_b, *product.dims,
                                    1, n_ctas, 64)
        assert (got.n_panels, got.n_steps, got.n_units) == (want.n_panels, want.n_steps, want.n_units)
        for name in ("panel_first", "step_offsets", "touched", "unit_panel", "unit_step"):
            assert torch.equal(getattr(got, name), getattr(want, name)), name
        assert torch.equal(got.steps[:got.n_steps], want.steps[:want.n_steps])
