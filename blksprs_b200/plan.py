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


_KERNEL_NAMES = {"auto": _cabi.KERNEL_AUTO, "mma": _cabi.KERNEL_MMA, "umma": _cabi.KERNEL_UMMA, "panel": 3}
_kernel_choice = _KERNEL_NAMES[os.environ.get("BLKSPRS_B200_KERNEL", "auto")]
KERNEL_PANEL = 3

# "auto" uses the wide-N kernel for block size 64 when panels merge enough work: steps / pairs at
# or below this ratio (0.5 = every step serves two (A, B) pairs).  Measured on B200: dense-B
# products (P*V, dO*V^T on an attention layout) gain 1.25-1.35x, random x random layouts (ratio
# ~0.85) lose, and for block size 128 the per-pair kernel is already at the L2/HBM limits.
PANEL_STEP_RATIO = float(os.environ.get("BLKSPRS_B200_PANEL_RATIO", "0.58"))
PANEL_AUTO_BLOCK_SIZES = (64,)


def set_kernel(name: str) -> None:
    """Selects the kernel family for later launches: ``"auto"`` (the wide-N tcgen05 kernel where
    panels pay off, the per-pair tcgen05 kernel for other 16-bit block-64/128 products, mma.sync
    otherwise), ``"mma"``, ``"umma"`` (per-pair tcgen05) or ``"panel"`` (wide-N tcgen05 wherever it
    applies).  Meant for tests and profiling; all families are sm_100a CUDA kernels of one library."""
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


@dataclass
class PanelPlan:
    op: int
    n_out: int
    n_panels: int
    n_steps: int
    width: int
    panel_first: Tensor
    step_offsets: Tensor
    steps: Tensor
    touched: Tensor
    chunk_begin: Tensor
    n_chunks: int


def build_panel_plan(op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor, R: int, K: int, C: int,
                     width: int, n_chunks: int) -> PanelPlan:
    """Groups the output blocks of every output row into panels of ``width`` and lists each panel's steps."""
    device = lut_out.device
    n_out = lut_out.size(0)
    (a_sb, a_sr, a_st), (b_sb, b_st, b_sc), T = _walk_strides(op, R, K, C)
    lib = _cabi.lib()
    with torch.cuda.device(device):
        stream = _cabi.stream_handle(device)
        # panel boundaries: position of every output block inside its (batch, row) run, modulo width
        idx = torch.arange(n_out, device=device)
        new_row = torch.ones(n_out, dtype=torch.bool, device=device)
        if n_out > 1:
            new_row[1:] = (lut_out[1:, 0] != lut_out[:-1, 0]) | (lut_out[1:, 1] != lut_out[:-1, 1])
        row_first = torch.cummax(torch.where(new_row, idx, torch.zeros_like(idx)), 0).values
        starts = torch.nonzero((idx - row_first) % width == 0).flatten()
        n_panels = starts.numel()
        panel_first = torch.empty(n_panels + 1, dtype=torch.int32, device=device)
        panel_first[:n_panels] = starts
        panel_first[n_panels] = n_out
        counts = torch.empty(max(n_panels, 1), dtype=torch.int32, device=device)
        touched = torch.empty(max(n_panels, 1), dtype=torch.int32, device=device)
        offsets = torch.empty(n_panels + 1, dtype=torch.int32, device=device)
        total = torch.empty(1, dtype=torch.int64, device=device)
        ws_bytes = lib.bsp_plan_workspace_bytes(n_panels)
        ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=device)
        walk = (_cabi.ptr(lut_out), _cabi.ptr(panel_first), n_panels, _cabi.ptr(packed_a), a_sb, a_sr, a_st,
                _cabi.ptr(packed_b), b_sb, b_st, b_sc, T)
        _cabi.check(lib.bsp_panel_count(*walk, _cabi.ptr(counts), _cabi.ptr(touched), stream), "bsp_panel_count")
        _cabi.check(lib.bsp_plan_offsets(_cabi.ptr(counts), n_panels, _cabi.ptr(offsets), _cabi.ptr(total),
                                         _cabi.ptr(ws), ws_bytes, stream), "bsp_plan_offsets")
        n_steps = int(total.item())
        if n_steps > 2_147_483_647 // 8:
            raise ValueError("blksprs_b200: panel plan too large")
        steps = torch.empty((max(n_steps, 1), 8), dtype=torch.int32, device=device)
        _cabi.check(lib.bsp_panel_fill(*walk, _cabi.ptr(offsets), _cabi.ptr(steps), stream), "bsp_panel_fill")
        chunk_begin = torch.empty(n_chunks + 1, dtype=torch.int32, device=device)
        _cabi.check(lib.bsp_plan_schedule(_cabi.ptr(offsets), n_panels, BLOCK_COST * width, n_chunks,
                                          _cabi.ptr(chunk_begin), stream), "bsp_plan_schedule")
    return PanelPlan(op, n_out, n_panels, n_steps, width, panel_first, offsets, steps, touched, chunk_begin, n_chunks)


def run_panel_plan(plan: PanelPlan, a: Tensor, b: Tensor, bs: int) -> Tensor:
    device = a.device
    out = torch.empty((plan.n_out, bs, bs), dtype=a.dtype, device=device)
    if plan.n_out == 0:
        return out
    with torch.cuda.device(device):
        _cabi.check(_cabi.lib().bsp_matmul_panel(
            _cabi.ptr(a), a.size(0), _cabi.ptr(b), b.size(0), _cabi.ptr(out), plan.n_out,
            _cabi.ptr(plan.panel_first), plan.n_panels, _cabi.ptr(plan.step_offsets), _cabi.ptr(plan.steps),
            _cabi.ptr(plan.touched), _cabi.ptr(plan.chunk_begin), plan.n_chunks, bs,
            _cabi.DATA_DTYPE_CODES[a.dtype], plan.op, _cabi.ptr(status_word(device)),
            _cabi.stream_handle(device)), "bsp_matmul_panel")
    return out


class Product:
    """One block-sparse product (forward, dX or dY) of a layout triple: its pair plan, and, built on
    first use for 16-bit data with block size 64 / 128, its panel plan."""

    def __init__(self, op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor, R: int, K: int, C: int,
                 n_chunks: int):
        self.op, self.dims = op, (R, K, C)
        self.lut_out, self.packed_a, self.packed_b = lut_out, packed_a, packed_b
        self.pair = build_pair_plan(op, lut_out, packed_a, packed_b, R, K, C, n_chunks)
        self._panels: dict[int, PanelPlan | None] = {}

    @property
    def n_chunks(self) -> int:
        return self.pair.n_chunks

    def panel(self, bs: int, dtype: torch.dtype) -> PanelPlan | None:
        """The panel plan for this block size, or ``None`` where the wide-N kernel does not apply."""
        if bs not in self._panels:
            lib = _cabi.lib()
            code = _cabi.DATA_DTYPE_CODES[dtype]
            width = lib.bsp_panel_width(code, bs)
            plan = None
            if width > 1 and self.pair.n_out > 0 and self.pair.n_pairs > 0:
                plan = build_panel_plan(self.op, self.lut_out, self.packed_a, self.packed_b, *self.dims, width,
                                        lib.bsp_matmul_panel_num_chunks(code, bs))
            self._panels[bs] = plan
        return self._panels[bs]

    def run(self, a: Tensor, b: Tensor, bs: int) -> Tensor:
        kernel = _kernel_choice
        if a.dtype in (torch.float16, torch.bfloat16) and a.size(0) > 0 and b.size(0) > 0 \
                and ((kernel == KERNEL_PANEL and bs in (64, 128))
                     or (kernel == _cabi.KERNEL_AUTO and bs in PANEL_AUTO_BLOCK_SIZES)):
            panel = self.panel(bs, a.dtype)
            if panel is not None and (kernel == KERNEL_PANEL
                                      or (bs in PANEL_AUTO_BLOCK_SIZES
                                          and panel.n_steps <= PANEL_STEP_RATIO * self.pair.n_pairs)):
                return run_panel_plan(panel, a, b, bs)
        if kernel == KERNEL_PANEL or a.size(0) == 0 or b.size(0) == 0:
            kernel = _cabi.KERNEL_AUTO  # without operand blocks only zero blocks are written
        return run_pair_plan(self.pair, a, b, bs, kernel)
