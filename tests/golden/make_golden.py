"""Generates ``reference_vectors.npz`` from the reference blksprs package itself.

Run where the reference checkout is importable (CPU is enough):

    BLKSPRS_REFERENCE=/path/to/blksprs python tests/golden/make_golden.py

What is recorded (all produced by reference code, none by this repository):
  * LUTs: ``build_layout_indices`` / ``build_packed_indices`` on CPU layouts of several dtypes
  * inferred layouts: ``build_sparsity_layout_matmul`` / ``_fast`` / ``_outer`` (validation off,
    their validator insists on CUDA tensors)
  * transposes: ``transpose_build_layout_cache`` + the ``flow_pull_kernel`` Triton kernel run
    under the Triton interpreter
  * matmul forward / backward: ``matmul_build_layout_cache`` + the ``matmul_kernel`` Triton
    kernel under the interpreter, backward composed exactly as ``matmul_wrapper_backward`` does
  * SHA-256 digests of the LUTs of the benchmark-sized layouts (config 2 of the workload list)
Inputs are regenerated in the tests from the seeds stored alongside.
"""
import hashlib
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("BLKSPRS_AUTOTUNE", "TEST")
REF = os.environ.get("BLKSPRS_REFERENCE")
if not REF:
    raise SystemExit("set BLKSPRS_REFERENCE to the checkout of the reference blksprs package")
sys.path.insert(0, REF)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import numpy as np  # noqa: E402
import torch  # noqa: E402

import blksprs as bs  # noqa: E402
import blksprs.ops.matmul  # noqa: E402,F401
import blksprs.ops.flow  # noqa: E402,F401
from blksprs.ops.transpose import transpose_build_layout_cache  # noqa: E402
from blksprs.utils.tools import build_layout_indices, build_packed_indices, stride  # noqa: E402

import cases  # noqa: E402

mm = sys.modules["blksprs.ops.matmul"]
flow = sys.modules["blksprs.ops.flow"]


def ref_matmul(x, lx, y, ly, lo, bs_, tile=16):
    cache = mm.matmul_build_layout_cache(None, lx, ly, lo)
    n = cache["n_sparse_blocks"]
    out = torch.zeros((n, bs_, bs_), dtype=x.dtype)
    if n == 0:
        return out
    x_b, x_r, x_c = x.size(); x_b_s, x_r_s, x_c_s = stride(x)
    lxb, lxr, lxc = lx.size(); lxbs, lxrs, lxcs = stride(lx)
    y_b, y_r, y_c = y.size(); y_b_s, y_r_s, y_c_s = stride(y)
    lyb, lyr, lyc = ly.size(); lybs, lyrs, lycs = stride(ly)
    o_b, o_r, o_c = out.size(); o_b_s, o_r_s, o_c_s = stride(out)
    lidx = cache["layout_indices_o"]
    lr, lc = lidx.size(); lrs, lcs = stride(lidx)
    grid = (o_b, o_r // tile, o_c // tile)
    mm.matmul_kernel.fn[grid](x, x_b, x_b_s, x_r_s, x_c_s, lxb, lxr, lxbs, lxrs, lxc, lxcs,
                              cache["packed_indices_x"],
                              y, y_b, y_b_s, y_r_s, y_c_s, lyb, lyr, lybs, lyrs, lyc, lycs,
                              cache["packed_indices_y"],
                              out, o_b, o_b_s, o_r_s, o_c_s, lidx, lr, lrs, lcs, bs_,
                              USE_INT64=False, TRITON_BLOCK_SIZE=tile)
    return out


def ref_transpose(x, layout, bs_, tile=16):
    cache = transpose_build_layout_cache(None, layout)
    n = cache["n_sparse_blocks"]
    lt = cache["sparsity_layout_t"]
    out = torch.zeros((n, bs_, bs_), dtype=x.dtype)
    if n == 0:
        return out, lt
    x_t = x.transpose(-1, -2).contiguous()
    x_b, x_r, x_c = x_t.size(); x_b_s, x_r_s, x_c_s = stride(x_t)
    o_b, o_r, o_c = out.size(); o_b_s, o_r_s, o_c_s = stride(out)
    lb, lr_, lc_ = lt.size(); lbs, lrs_, lcs_ = stride(lt)
    lidx = cache["layout_indices"]
    r, c = lidx.size(); rs, cs = stride(lidx)
    grid = (o_b, o_r // tile, o_c // tile)
    flow.flow_pull_kernel.fn[grid](x_t, x_b, x_b_s, x_r_s, x_c_s, out, o_b, o_b_s, o_r_s, o_c_s,
                                   lb, lbs, lrs_, lcs_, lidx, r, rs, cs, cache["packed_indices"], bs_,
                                   USE_INT64=False, TRITON_BLOCK_SIZE=tile)
    return out, lt


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def main():
    rec = {}
    # LUTs
    for name, layout in cases.lut_layouts():
        rec[f"lut/{name}/layout_indices"] = build_layout_indices(layout).numpy()
        rec[f"lut/{name}/packed_indices"] = build_packed_indices(layout).numpy()
        rec[f"lut/{name}/n_sparse_blocks"] = np.int64(torch.sum(layout.to(torch.int)).item())
    # inferred layouts
    bs.utils.disable_validation()
    for name, lx, ly in cases.layout_pairs():
        rec[f"infer/{name}/exact"] = bs.layouting.build_sparsity_layout_matmul(lx, ly).numpy()
        rec[f"infer/{name}/fast"] = bs.layouting.build_sparsity_layout_matmul_fast(lx, ly).numpy()
        rec[f"infer/{name}/outer"] = bs.layouting.build_sparsity_layout_matmul_outer(lx, ly).numpy()
    bs.utils.enable_validation()
    # benchmark-sized layouts: digests only
    for name, lx, ly in cases.big_layout_pairs():
        lo = torch.matmul(lx.float(), ly.float()).to(torch.bool)
        cache = mm.matmul_build_layout_cache(None, lx, ly, lo)
        rec[f"big/{name}/digest"] = np.array([digest(cache["packed_indices_x"]), digest(cache["packed_indices_y"]),
                                              digest(cache["layout_indices_o"]), digest(lo.to(torch.uint8))])
        rec[f"big/{name}/n_sparse_blocks"] = np.int64(cache["n_sparse_blocks"])
    # transposes and matmuls through the reference's Triton kernels (interpreter)
    for name, case in cases.matmul_cases():
        x, lx, y, ly, lo, bs_, g = case["x"], case["lx"], case["y"], case["ly"], case["lo"], case["bs"], case["grad"]
        out = ref_matmul(x, lx, y, ly, lo, bs_)
        x_t, lx_t = ref_transpose(x, lx, bs_)
        y_t, ly_t = ref_transpose(y, ly, bs_)
        gx = ref_matmul(g, lo, y_t, ly_t, lx, bs_)
        gy = ref_matmul(x_t, lx_t, g, lo, ly, bs_)
        as_np = (lambda t: t.float().numpy()) if x.dtype != torch.float32 else (lambda t: t.numpy())
        rec[f"matmul/{name}/out"] = as_np(out)
        rec[f"matmul/{name}/grad_x"] = as_np(gx)
        rec[f"matmul/{name}/grad_y"] = as_np(gy)
        rec[f"matmul/{name}/x_t"] = as_np(x_t)
        rec[f"matmul/{name}/layout_x_t"] = lx_t.numpy()
        print(name, "ok", tuple(out.shape))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(path, **rec)
    print("wrote", path, os.path.getsize(path), "bytes,", len(rec), "arrays")


if __name__ == "__main__":
    main()
