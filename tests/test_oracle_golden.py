"""The CPU oracle against vectors produced by the reference package itself (tests/golden)."""
import hashlib

import numpy as np
import pytest
import torch

import cases
from oracle import oracle


@pytest.mark.parametrize("name,layout", cases.lut_layouts(), ids=[n for n, _ in cases.lut_layouts()])
def test_luts_bit_exact(golden, name, layout):
    assert np.array_equal(oracle.layout_indices(layout), golden[f"lut/{name}/layout_indices"])
    assert np.array_equal(oracle.packed_indices(layout), golden[f"lut/{name}/packed_indices"])
    assert oracle.n_sparse_blocks(layout) == int(golden[f"lut/{name}/n_sparse_blocks"])


@pytest.mark.parametrize("name,lx,ly", cases.layout_pairs(), ids=[n for n, _, _ in cases.layout_pairs()])
def test_layout_inference_bit_exact(golden, name, lx, ly):
    assert np.array_equal(oracle.layout_matmul(lx, ly), golden[f"infer/{name}/exact"])
    assert np.array_equal(oracle.layout_matmul_fast(lx, ly), golden[f"infer/{name}/fast"])
    assert np.array_equal(oracle.layout_matmul_outer(lx, ly), golden[f"infer/{name}/outer"])


def _digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_benchmark_layout_digests(golden):
    for name, lx, ly in cases.big_layout_pairs():
        lo = oracle.layout_matmul(lx, ly)
        want = list(golden[f"big/{name}/digest"])
        got = [_digest(oracle.packed_indices(lx)), _digest(oracle.packed_indices(ly)),
               _digest(oracle.layout_indices(lo)), _digest(lo.astype(np.uint8))]
        assert got == want
        assert oracle.n_sparse_blocks(lo) == int(golden[f"big/{name}/n_sparse_blocks"])


@pytest.mark.parametrize("name,case", cases.matmul_cases(), ids=[n for n, _ in cases.matmul_cases()])
def test_matmul_and_transpose_vs_reference_kernels(golden, name, case):
    x, lx, y, ly, lo, bs, g = (case[k] for k in ("x", "lx", "y", "ly", "lo", "bs", "grad"))
    ref_out = torch.from_numpy(golden[f"matmul/{name}/out"])
    ref_gx = torch.from_numpy(golden[f"matmul/{name}/grad_x"])
    ref_gy = torch.from_numpy(golden[f"matmul/{name}/grad_y"])
    # the interpreter runs the reference kernel in IEEE arithmetic: tight tolerance
    tol = dict(atol=1e-4, rtol=1e-4) if x.dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    for fwd in (oracle.matmul_forward_blocks, oracle.matmul_forward):
        out = fwd(x, lx, y, ly, lo, bs)
        assert out.shape == ref_out.shape and out.dtype == x.dtype
        assert torch.allclose(out.float(), ref_out, **tol)
    for bwd in (oracle.matmul_backward, oracle.matmul_backward_via_transpose):
        gx, gy = bwd(g, x, lx, y, ly, lo, bs)
        assert torch.allclose(gx.float(), ref_gx, **tol)
        assert torch.allclose(gy.float(), ref_gy, **tol)
    x_t, lx_t = oracle.transpose(x, lx, bs)
    assert np.array_equal(lx_t, golden[f"matmul/{name}/layout_x_t"])
    assert torch.equal(x_t.float(), torch.from_numpy(golden[f"matmul/{name}/x_t"]))


def test_work_model_matches_bruteforce():
    lx = cases.bernoulli_layout((2, 5, 6), 0.5, 40)
    ly = cases.bernoulli_layout((2, 6, 4), 0.5, 41)
    lo = torch.ones((2, 5, 4), dtype=torch.bool)
    brute = sum(int(lx[b, i, k] and ly[b, k, j]) for b in range(2) for i in range(5) for j in range(4)
                for k in range(6))
    assert oracle.pair_count(lx, ly, lo) == brute


def test_linear_and_softmax_restatements_match_their_dense_definitions():
    """``oracle.linear`` / ``oracle.softmax`` are the dense forms the reference's own tests check against
    (``torch.nn.Linear`` on the expanded input, test/cases/test_blocksparse.py:1158-1184; softmax over a row's
    active blocks, blksprs/ops/softmax.py:58-61): here against plain torch on a case with full layouts."""
    g = torch.Generator().manual_seed(4)
    bs, B, R, K, N = 16, 2, 3, 2, 4
    layout = torch.ones((B, R, K), dtype=torch.bool)
    dense = torch.randn((B, R * bs, K * bs), generator=g)
    x = oracle.to_sparse(dense, layout, bs)
    weight, bias = torch.randn((N * bs, K * bs), generator=g), torch.randn(N * bs, generator=g)
    out, out_layout = oracle.linear(x, layout, bs, weight, bias)
    want = torch.nn.functional.linear(dense, weight, bias)
    assert out_layout.shape == (B, R, N) and out_layout.all()
    assert torch.allclose(oracle.to_dense(out, out_layout, bs), want, atol=1e-5)
    grad = torch.randn(out.shape, generator=g)
    dense_req, w_req, b_req = (t.clone().requires_grad_(True) for t in (dense, weight, bias))
    torch.nn.functional.linear(dense_req, w_req, b_req).backward(oracle.to_dense(grad, out_layout, bs))
    gx, gw, gb = oracle.linear_backward(grad, out_layout, x, layout, bs, weight, True)
    assert torch.allclose(oracle.to_dense(gx, layout, bs), dense_req.grad, atol=1e-4)
    assert torch.allclose(gw, w_req.grad, atol=1e-4) and torch.allclose(gb, b_req.grad, atol=1e-4)
    # without a bias only the block rows that hold an input block appear in the output
    sparse_layout = torch.tensor([[[1, 0], [0, 0], [0, 1]], [[0, 0], [1, 1], [0, 0]]], dtype=torch.bool)
    xs = oracle.to_sparse(dense, sparse_layout, bs)
    _, lo = oracle.linear(xs, sparse_layout, bs, weight)
    assert np.array_equal(lo[..., 0], sparse_layout.any(-1).numpy()) and (lo == lo[..., :1]).all()
    # softmax
    sm = oracle.softmax(x, layout, bs)
    assert torch.allclose(oracle.to_dense(sm, layout, bs), torch.softmax(dense, -1), atol=1e-6)
    masked = oracle.to_dense(oracle.softmax(xs, sparse_layout, bs), sparse_layout, bs)
    rows_with_blocks = torch.from_numpy(np.repeat(sparse_layout.any(-1).numpy(), bs, axis=1))
    assert torch.allclose(masked.sum(-1)[rows_with_blocks], torch.ones(int(rows_with_blocks.sum())), atol=1e-5)
