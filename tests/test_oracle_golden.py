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
