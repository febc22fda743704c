"""Pair plans: the per-layout-triple metadata the matmul kernels consume.

The reference kernel re-derives, in every launch and for every output block,
which inner blocks both operands have in common by walking two reverse LUTs
(blksprs/ops/matmul.py:191-226).  Here that walk runs once per layout triple
(``bsp_plan_*`` in the native library) and its result is kept in the layout
cache next to the reference-visible LUT entries:

``offsets``      int32 ``(n_out + 1)``  CSR offsets into ``pairs`` per output block
``pairs``        int32 ``(total, 2)``   (a_block, b_block) indices, inner index ascending
``chunk_begin``  int32 ``(n_chunks+1)`` output-block ranges of the persistent CTAs (tcgen05 kernel)
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
from torch import Tensor

from . import _cabi

# Cost of an output block in the schedule, in units of one (a, b) pair: the
# epilogue (accumulator drain + store) of a block weighs about one pair.
BLOCK_COST = 1


@dataclass
class PairPlan:
    op: int
    n_out: int
    n_pairs: int
    offsets: Tensor
    pairs: Tensor
    chunk_begin: Tensor | None
    n_chunks: int


def _walk_strides(op: int, R: int, K: int, C: int):
    """(a_sb, a_sr, a_st), (b_sb, b_st, b_sc), T for the reverse-LUT walk of one product.

    Layout grids: x is (B, R, K), y is (B, K, C), o is (B, R, C).
      NN  out = o(b, i, j): a = x[b, i, t], b = y[b, t, j], t over K
      NT  out = x(b, i, k): a = o[b, i, t], b = y[b, k, t], t over C      (dX = dO * Y^T)
      TN  out = y(b, k, j): a = x[b, t, k], b = o[b, t, j], t over R      (dY = X^T * dO)
    """
    if op == _cabi.OP_NN:
        return (R * K, K, 1), (K * C, C, 1), K
    if op == _cabi.OP_NT:
        return (R * C, C, 1), (K * C, 1, C), C
    if op == _cabi.OP_TN:
        return (R * K, 1, K), (R * C, C, 1), R
    raise ValueError(f"unknown op {op}")


def build_pair_plan(op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor,
                    R: int, K: int, C: int, n_chunks: int) -> PairPlan:
    """Builds the plan of one product; one device->host read (the total pair count)."""
    device = lut_out.device
    n_out = lut_out.size(0)
    (a_sb, a_sr, a_st), (b_sb, b_st, b_sc), T = _walk_strides(op, R, K, C)
    lib = _cabi.lib()
    with torch.cuda.device(device):
        stream = _cabi.stream_handle(device)
        counts = torch.empty(max(n_out, 1), dtype=torch.int32, device=device)
        offsets = torch.empty(n_out + 1, dtype=torch.int32, device=device)
        total = torch.empty(1, dtype=torch.int64, device=device)
        ws_bytes = lib.bsp_plan_workspace_bytes(n_out)
        ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=device)
        _cabi.check(lib.bsp_plan_count(_cabi.ptr(lut_out), n_out, _cabi.ptr(packed_a), a_sb, a_sr, a_st,
                                       _cabi.ptr(packed_b), b_sb, b_st, b_sc, T, _cabi.ptr(counts), stream),
                    "bsp_plan_count")
        _cabi.check(lib.bsp_plan_offsets(_cabi.ptr(counts), n_out, _cabi.ptr(offsets), _cabi.ptr(total),
                                         _cabi.ptr(ws), ws_bytes, stream), "bsp_plan_offsets")
        n_pairs = int(total.item())
        if n_pairs > 2_147_483_647:
            raise ValueError("blksprs_b200: pair plan exceeds 2^31-1 block pairs")
        pairs = torch.empty((max(n_pairs, 1), 2), dtype=torch.int32, device=device)
        _cabi.check(lib.bsp_plan_fill(_cabi.ptr(lut_out), n_out, _cabi.ptr(packed_a), a_sb, a_sr, a_st,
                                      _cabi.ptr(packed_b), b_sb, b_st, b_sc, T, _cabi.ptr(offsets),
                                      _cabi.ptr(pairs), stream), "bsp_plan_fill")
        chunk_begin = None
        if n_chunks > 0:
            chunk_begin = torch.empty(n_chunks + 1, dtype=torch.int32, device=device)
            _cabi.check(lib.bsp_plan_schedule(_cabi.ptr(offsets), n_out, BLOCK_COST, n_chunks,
                                              _cabi.ptr(chunk_begin), stream), "bsp_plan_schedule")
    return PairPlan(op, n_out, n_pairs, offsets, pairs, chunk_begin, n_chunks)


_status_words: dict[torch.device, Tensor] = {}


def status_word(device: torch.device) -> Tensor:
    """Per-device int32 word the kernels write BSP_ERR_DEVICE_* codes into (never cleared by them)."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _status_words.get(device)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = word
    return word


def check_device_status(device: torch.device | None = None) -> None:
    """Reads (one host sync) and clears the device status word; raises if a kernel recorded a problem."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise _cabi.NativeError(code, "device status word")


_KERNEL_NAMES = {"auto": _cabi.KERNEL_AUTO, "mma": _cabi.KERNEL_MMA, "umma": _cabi.KERNEL_UMMA}
_kernel_choice = _KERNEL_NAMES[os.environ.get("BLKSPRS_B200_KERNEL", "auto")]


def set_kernel(name: str) -> None:
    """Selects the kernel family for later launches: ``"auto"`` (tcgen05 where it applies, else
    mma.sync), ``"mma"`` or ``"umma"``.  Meant for tests and profiling; both families are sm_100a
    CUDA kernels of the same library."""
    global _kernel_choice
    _kernel_choice = _KERNEL_NAMES[name]


def run_pair_plan(plan: PairPlan, a: Tensor, b: Tensor, bs: int, kernel: int | None = None) -> Tensor:
    """Launches one block-sparse product on ``plan``; returns the compressed result ``(n_out, bs, bs)``."""
    if kernel is None:
        kernel = _kernel_choice
    device = a.device
    out = torch.empty((plan.n_out, bs, bs), dtype=a.dtype, device=device)
    if plan.n_out == 0:
        return out
    with torch.cuda.device(device):
        _cabi.check(_cabi.lib().bsp_matmul(
            _cabi.ptr(a), a.size(0), _cabi.ptr(b), b.size(0), _cabi.ptr(out), plan.n_out,
            _cabi.ptr(plan.offsets), _cabi.ptr(plan.pairs), _cabi.ptr(plan.chunk_begin), plan.n_chunks,
            bs, _cabi.DATA_DTYPE_CODES[a.dtype], plan.op, kernel, _cabi.ptr(status_word(device)),
            _cabi.stream_handle(device)), "bsp_matmul")
    return out
