"""Plans: the per-layout-triple metadata the matmul kernels consume.

The reference kernel re-derives, in every launch and for every output block, which inner blocks
both operands have in common by walking two reverse LUTs (blksprs/ops/matmul.py:191-226).  Here
that walk runs once per layout triple in the native library and its result is kept in the layout
cache next to the reference-visible LUT entries.

Pair plan (``bsp_plan_*``; consumed by the mma.sync kernel, and the yardstick for panel merging):
``offsets`` int32 ``(n_out + 1)`` CSR offsets per output block, ``pairs`` int32 ``(total, 2)``
(a_block, b_block), inner index ascending.

Step plan (``bsp_panel_*``; consumed by the tcgen05 kernel): every ``width`` (1 or 2) consecutive
output blocks form a panel; a step is one inner index whose A block exists and that hits at least
one of the panel's B blocks (the blocks of a panel that share an output row share their A blocks; a
panel that runs across the end of a row is walked row by row).  ``unit_panel`` / ``unit_step`` cut the panels into
contiguous units of equal cost that the persistent CTAs take in order — drawn from a counter
(``SCHEDULE = "dynamic"``, small units) or round-robin (``"static"``, larger units) — so that all
SMs work on neighbouring output rows (same batch, same operand blocks in L2) at the same time.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
from torch import Tensor

from . import _cabi

# Cost of an output block in a schedule, in units of one (a, b) pair: the epilogue (accumulator
# drain + store) of a block weighs about one pair.
BLOCK_COST = 1
# A unit should hold about this much work (pairs + blocks): large enough to amortise the ring
# restart at a unit boundary, small enough that concurrently processed units share operands in L2.
UNIT_COST = 48
MAX_UNITS_PER_CTA = 64
# With the dynamic schedule a unit is the grain of load balancing: small, but large enough that
# drawing it from the counter stays invisible.  Measured optimum per block size (a pair of 128-blocks
# is eight times the work of a pair of 64-blocks).
# Small units everywhere also keep all CTAs inside a narrow window of the output at any time, which
# is what keeps the operand blocks they share in L2 (units that start large and shrink towards the
# end measured 5-15 % slower than uniform small ones).
UNIT_COST_DYNAMIC = {64: 24, 128: 12}
MAX_UNITS_PER_CTA_DYNAMIC = 1024

# How the persistent CTAs of the tcgen05 kernel get their units: "dynamic" = from a counter, so CTAs
# that run slower take fewer units; "static" = round-robin.
SCHEDULE = os.environ.get("BLKSPRS_B200_SCHED", "dynamic")

KERNELS = ("auto", "mma", "umma", "panel")
_kernel_choice = os.environ.get("BLKSPRS_B200_KERNEL", "auto")

# "auto" uses panels of two output blocks when they merge enough work: steps / pairs at or below
# this ratio (0.5 = every step serves two (A, B) pairs).  Measured on B200: dense-B products (P*V,
# dO*V^T on an attention layout, sparse x dense at block size 128) gain 1.15-1.35x, random x random
# layouts (ratio ~0.85) lose.
PANEL_STEP_RATIO = 0.58
PANEL_AUTO_BLOCK_SIZES = (64, 128)


def set_kernel(name: str) -> None:
    """Selects the kernel family for later launches: ``"auto"`` (tcgen05 for block
    size 64 / 128, with two-block panels where they pay off; mma.sync otherwise), ``"mma"``
    (mma.sync everywhere), ``"umma"`` (tcgen05, single-block steps) or ``"panel"`` (tcgen05,
    two-block panels).  Meant for tests and profiling; all are sm_100a kernels of one library."""
    global _kernel_choice
    if name not in KERNELS:
        raise ValueError(f"unknown kernel family {name!r}")
    _kernel_choice = name


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


@dataclass
class PairPlan:
    op: int
    n_out: int
    n_pairs: int
    offsets: Tensor
    pairs: Tensor


@dataclass
class _Counted:
    """The device half of a plan whose sizes the host has not read yet: per-block (per-panel)
    counts and their offsets are on the device, ``totals`` (int64: the total, and for a step plan
    the largest panel) waits to be read.  ``resolve_counts`` reads the totals of any number of these
    in one device->host copy."""
    width: int                      # 0 = pair plan, 1 / 2 = step plan of that panel width
    walk: tuple
    n_slots: int                    # output blocks (pair plan) or panels (step plan)
    offsets: Tensor
    totals: Tensor
    panel_first: Tensor | None = None
    touched: Tensor | None = None
    total: int | None = None
    largest: int | None = None
    pairs: int | None = None        # (A block, B block) pairs the plan stands for
    block_counts: Tensor | None = None   # panels of several blocks: the pairs of every single output block
    largest_block: int | None = None


def count_pairs(op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor, R: int, K: int, C: int) -> _Counted:
    """Counts the pairs of every output block and scans them; no device->host read."""
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
        walk = (_cabi.ptr(lut_out), n_out, _cabi.ptr(packed_a), a_sb, a_sr, a_st, _cabi.ptr(packed_b), b_sb, b_st,
                b_sc, T)
        _cabi.check(lib.bsp_plan_count(*walk, _cabi.ptr(counts), stream), "bsp_plan_count")
        _cabi.check(lib.bsp_plan_offsets(_cabi.ptr(counts), n_out, _cabi.ptr(offsets), _cabi.ptr(total),
                                         _cabi.ptr(ws), ws_bytes, stream), "bsp_plan_offsets")
    return _Counted(0, walk, n_out, offsets, total)


def finish_pair_plan(op: int, counted: _Counted) -> PairPlan:
    """Allocates and fills the pair list of a counted (and resolved) pair plan."""
    n_pairs = counted.total
    if n_pairs > 2_147_483_647:
        raise ValueError("blksprs_b200: pair plan exceeds 2^31-1 block pairs")
    device = counted.offsets.device
    with torch.cuda.device(device):
        pairs = torch.empty((max(n_pairs, 1), 2), dtype=torch.int32, device=device)
        _cabi.check(_cabi.lib().bsp_plan_fill(*counted.walk, _cabi.ptr(counted.offsets), _cabi.ptr(pairs),
                                              _cabi.stream_handle(device)), "bsp_plan_fill")
    return PairPlan(op, counted.n_slots, n_pairs, counted.offsets, pairs)


def resolve_counts(pending: list[_Counted]) -> None:
    """Reads the totals of all ``pending`` plans (of one device) in a single device->host copy."""
    pending = [c for c in pending if c.total is None]
    if not pending:
        return
    device = pending[0].totals.device
    values = read_with_status(torch.cat([c.totals for c in pending]), device)
    at = 0
    for c in pending:
        c.total = values[at]
        if c.totals.numel() > 1:
            c.largest, c.pairs, c.largest_block = values[at + 1], values[at + 2], values[at + 3]
        else:
            c.pairs = c.total
        at += c.totals.numel()


def build_pair_plan(op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor,
                    R: int, K: int, C: int) -> PairPlan:
    """Builds the pair plan of one product; one device->host read (the total pair count)."""
    counted = count_pairs(op, lut_out, packed_a, packed_b, R, K, C)
    resolve_counts([counted])
    return finish_pair_plan(op, counted)


@dataclass
class StepPlan:
    op: int
    n_out: int
    n_panels: int
    n_steps: int
    width: int
    panel_first: Tensor
    step_offsets: Tensor
    steps: Tensor
    touched: Tensor
    unit_panel: Tensor
    unit_step: Tensor
    n_units: int
    dynamic: bool = False  # units are handed out from a counter (else round-robin)

    def launch_args(self) -> tuple:
        """The plan's own arguments of ``bsp_matmul_umma`` (pointers are stable: the plan holds the tensors)."""
        args = self.__dict__.get("_launch_args")
        if args is None:
            args = (self.panel_first.data_ptr(), self.n_panels, self.step_offsets.data_ptr(), self.steps.data_ptr(),
                    self.touched.data_ptr(), self.unit_panel.data_ptr(), self.unit_step.data_ptr(), self.n_units)
            self.__dict__["_launch_args"] = args
        return args

    def sched_ptr(self, stream: int) -> int | None:
        """The scheduling counters (int32[2], zero between launches) for a launch on ``stream``, or
        None for the static round-robin schedule.  Launches of one stream run one after the other and
        share a pair; every other stream gets its own, and every launch recorded during a CUDA-graph
        capture gets a pair of its own (a replayed graph may overlap anything launched later), so that
        concurrent launches of one plan never draw from the same counter.  A graph must not be
        replayed concurrently with itself.  The pairs come from a pool allocated with the plan; when
        it is used up, launches fall back to the static schedule."""
        if not self.dynamic:
            return None
        pool: Tensor = self.__dict__["_sched_pool"]
        table = self.__dict__.setdefault("_sched", {})
        if torch.cuda.is_current_stream_capturing():
            slot = len(table)
            if 2 * slot + 2 > pool.numel():
                return None
            table[("capture", slot)] = slot
            return pool.data_ptr() + 8 * slot
        slot = table.get(stream)
        if slot is None:
            slot = len(table)
            if 2 * slot + 2 > pool.numel():
                return None
            table[stream] = slot
        return pool.data_ptr() + 8 * slot


SCHED_POOL_PAIRS = 64


def count_steps(op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor, R: int, K: int, C: int,
                width: int) -> _Counted:
    """Groups the output blocks into panels of ``width`` consecutive blocks (the walk splits a panel
    that runs across the end of a layout row into its rows), counts each panel's steps and scans
    them; no device->host read."""
    device = lut_out.device
    n_out = lut_out.size(0)
    (a_sb, a_sr, a_st), (b_sb, b_st, b_sc), T = _walk_strides(op, R, K, C)
    lib = _cabi.lib()
    with torch.cuda.device(device):
        stream = _cabi.stream_handle(device)
        n_panels = -(-n_out // width)
        panel_first = torch.arange(0, (n_panels + 1) * width, width, dtype=torch.int32, device=device)
        if n_panels:
            panel_first[n_panels] = n_out
        counts = torch.empty(max(n_panels, 1), dtype=torch.int32, device=device)
        touched = torch.empty(max(n_panels, 1), dtype=torch.int32, device=device)
        offsets = torch.empty(n_panels + 1, dtype=torch.int32, device=device)
        # total steps (from the scan); largest panel, pair count and largest single block (from the counting
        # kernel, which for panels of several blocks also leaves the pair count of every single block: the
        # counts of the single-block plan, should that one be chosen)
        totals = torch.zeros(4, dtype=torch.int64, device=device)
        block_counts = torch.empty(max(n_out, 1), dtype=torch.int32, device=device) if width > 1 else None
        ws_bytes = lib.bsp_plan_workspace_bytes(n_panels)
        ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=device)
        walk = (_cabi.ptr(lut_out), _cabi.ptr(panel_first), n_panels, _cabi.ptr(packed_a), a_sb, a_sr, a_st,
                _cabi.ptr(packed_b), b_sb, b_st, b_sc, T)
        _cabi.check(lib.bsp_panel_count(*walk, _cabi.ptr(counts), _cabi.ptr(touched), totals.data_ptr() + 8,
                                        _cabi.ptr(block_counts), stream), "bsp_panel_count")
        _cabi.check(lib.bsp_plan_offsets(_cabi.ptr(counts), n_panels, _cabi.ptr(offsets), _cabi.ptr(totals),
                                         _cabi.ptr(ws), ws_bytes, stream), "bsp_plan_offsets")
    return _Counted(width, walk, n_panels, offsets, totals, panel_first, touched, block_counts=block_counts)


def single_block_counts(op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor, R: int, K: int, C: int,
                        wide: _Counted) -> _Counted:
    """The counted half of the plan with one block per panel, taken from a resolved count of wider
    panels: its per-panel counts are the wide walk's per-block pair counts, its totals are known, so
    neither a second walk nor a second read is needed (only the scan of the counts)."""
    device = lut_out.device
    n_out = lut_out.size(0)
    (a_sb, a_sr, a_st), (b_sb, b_st, b_sc), T = _walk_strides(op, R, K, C)
    lib = _cabi.lib()
    with torch.cuda.device(device):
        stream = _cabi.stream_handle(device)
        panel_first = torch.arange(0, n_out + 1, dtype=torch.int32, device=device)
        counts = wide.block_counts
        touched = (counts > 0).to(torch.int32)
        offsets = torch.empty(n_out + 1, dtype=torch.int32, device=device)
        totals = torch.empty(4, dtype=torch.int64, device=device)
        ws_bytes = lib.bsp_plan_workspace_bytes(n_out)
        ws = torch.empty(ws_bytes // 8, dtype=torch.int64, device=device)
        walk = (_cabi.ptr(lut_out), _cabi.ptr(panel_first), n_out, _cabi.ptr(packed_a), a_sb, a_sr, a_st,
                _cabi.ptr(packed_b), b_sb, b_st, b_sc, T)
        _cabi.check(lib.bsp_plan_offsets(_cabi.ptr(counts), n_out, _cabi.ptr(offsets), _cabi.ptr(totals),
                                         _cabi.ptr(ws), ws_bytes, stream), "bsp_plan_offsets")
    return _Counted(1, walk, n_out, offsets, totals, panel_first, touched, total=wide.pairs,
                    largest=wide.largest_block, pairs=wide.pairs)


def finish_step_plan(op: int, n_out: int, counted: _Counted, n_ctas: int, bs: int) -> StepPlan:
    """Lists the steps of a counted (and resolved) step plan and cuts its panels into units."""
    width, n_panels, n_steps, max_panel_steps = counted.width, counted.n_slots, counted.total, counted.largest
    if n_steps > 2_147_483_647 // 8:
        raise ValueError("blksprs_b200: step plan too large")
    offsets = counted.offsets
    device = offsets.device
    lib = _cabi.lib()
    with torch.cuda.device(device):
        stream = _cabi.stream_handle(device)
        steps = torch.empty((max(n_steps, 1), 8), dtype=torch.int32, device=device)
        _cabi.check(lib.bsp_panel_fill(*counted.walk, _cabi.ptr(offsets), _cabi.ptr(steps), stream), "bsp_panel_fill")
        cost = n_steps + BLOCK_COST * width * n_panels
        heaviest = max_panel_steps + BLOCK_COST * width
        # static round-robin: a unit is several times the heaviest panel, so that indivisible
        # panels cannot unbalance the CTAs; dynamic hand-out needs no such margin
        if SCHEDULE == "dynamic":
            target = UNIT_COST_DYNAMIC.get(bs, 24)
            # a whole number of units per CTA: equally fast CTAs then finish together
            # no floor at the heaviest panel: a panel heavier than a unit just leaves a few units empty,
            # while larger units would widen the window of output the CTAs work in beyond what L2 holds
            per_cta = max(1, min(MAX_UNITS_PER_CTA_DYNAMIC, round(cost / (max(n_ctas, 1) * max(target, 1)))))
            n_units = max(1, n_ctas * per_cta)
        else:
            unit_cost = max(UNIT_COST, 4 * heaviest)
            per_cta = max(1, min(MAX_UNITS_PER_CTA, round(cost / (max(n_ctas, 1) * unit_cost))))
            n_units = max(1, n_ctas * per_cta)
        unit_panel = torch.empty(n_units + 1, dtype=torch.int32, device=device)
        _cabi.check(lib.bsp_plan_schedule(_cabi.ptr(offsets), n_panels, BLOCK_COST * width, n_units,
                                          _cabi.ptr(unit_panel), stream), "bsp_plan_schedule")
        unit_step = offsets[unit_panel.long()].contiguous()
        plan = StepPlan(op, n_out, n_panels, n_steps, width, counted.panel_first, offsets, steps, counted.touched,
                        unit_panel, unit_step, n_units, SCHEDULE == "dynamic")
        plan.__dict__["_sched_pool"] = torch.zeros(2 * SCHED_POOL_PAIRS, dtype=torch.int32, device=device)
    return plan


def build_step_plan(op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor, R: int, K: int, C: int,
                    width: int, n_ctas: int, bs: int = 64) -> StepPlan:
    """Counts, reads (one device->host read: the total step count and the largest panel) and lists the
    steps of one product for panels of ``width`` blocks."""
    counted = count_steps(op, lut_out, packed_a, packed_b, R, K, C, width)
    resolve_counts([counted])
    return finish_step_plan(op, lut_out.size(0), counted, n_ctas, bs)


_status_words: dict[torch.device, Tensor] = {}


def read_with_status(values: Tensor, device: torch.device) -> list[int]:
    """Reads int64 device values to the host together with the device status word (one copy, one
    sync): wherever the host has to wait for the device anyway, a problem an earlier kernel recorded
    (``BSP_ERR_DEVICE_RANGE``, ``BSP_ERR_DEVICE_TIMEOUT``) surfaces as an exception."""
    word = status_word(device)
    *out, code = torch.cat([values.reshape(-1).to(torch.int64), word.to(torch.int64)]).tolist()
    if code != 0:
        word.zero_()
        raise _cabi.NativeError(int(code), "device status word (set by an earlier kernel)")
    return [int(v) for v in out]


def status_word(device: torch.device) -> Tensor:
    """Per-device int32 word the kernels write BSP_ERR_DEVICE_* codes into (never cleared by them)."""
    word = _status_words.get(device)
    if word is None:
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


def run_pair_plan(plan: PairPlan, a: Tensor, b: Tensor, bs: int) -> Tensor:
    """One block-sparse product with the mma.sync kernel; returns the compressed result ``(n_out, bs, bs)``."""
    device = a.device
    out = torch.empty((plan.n_out, bs, bs), dtype=a.dtype, device=device)
    if plan.n_out == 0:
        return out
    with _cabi.device_guard(device):
        status = _cabi.lib().bsp_matmul_mma(
            a.data_ptr(), a.size(0), b.data_ptr(), b.size(0), out.data_ptr(), plan.n_out,
            plan.offsets.data_ptr(), plan.pairs.data_ptr(), bs, _cabi.DATA_DTYPE_CODES[a.dtype], plan.op,
            status_word(device).data_ptr(), _cabi.stream_handle(device))
    if status:
        _cabi.check(status, "bsp_matmul_mma")
    return out


def run_step_plan(plan: StepPlan, a: Tensor, b: Tensor, bs: int, bias: Tensor | None = None,
                  lut_out: Tensor | None = None) -> Tensor:
    """One block-sparse product with the tcgen05 kernel; ``bias`` (one element per output column, with
    the output LUT) is added in the kernel's epilogue."""
    device = a.device
    out = torch.empty((plan.n_out, bs, bs), dtype=a.dtype, device=device)
    if plan.n_out == 0:
        return out
    with _cabi.device_guard(device):
        stream = _cabi.stream_handle(device)
        status = _cabi.lib().bsp_matmul_umma(
            a.data_ptr(), a.size(0), b.data_ptr(), b.size(0), out.data_ptr(), plan.n_out,
            None if bias is None else bias.data_ptr(), None if bias is None else lut_out.data_ptr(),
            *plan.launch_args(), plan.sched_ptr(stream), plan.width, bs, _cabi.DATA_DTYPE_CODES[a.dtype], plan.op,
            status_word(device).data_ptr(), stream)
    if status:
        _cabi.check(status, "bsp_matmul_umma")
    return out


class Product:
    """One block-sparse product (forward, dX or dY) of a layout triple.  Its plans are built when a
    launch first needs them: the pair plan for the mma.sync kernels, step plans for the tcgen05
    kernel (block size 64 / 128).  Building is split into a counting half without device->host read
    and a listing half that needs the totals, so that everything a call needs — of all three products
    of a training step — is read in one copy (``prepare_products``)."""

    def __init__(self, op: int, lut_out: Tensor, packed_a: Tensor, packed_b: Tensor, R: int, K: int, C: int):
        self.op, self.dims = op, (R, K, C)
        self.lut_out, self.packed_a, self.packed_b = lut_out, packed_a, packed_b
        self.n_out = lut_out.size(0)
        self._counted: dict[int, _Counted] = {}     # 0 = pair plan, 1 / 2 = step plan of that width
        self._pair: PairPlan | None = None
        self._steps: dict[tuple[int, int], StepPlan] = {}

    def _count(self, widths) -> list[_Counted]:
        """Launches the counting half of the plans in ``widths`` that are not counted yet; returns
        those whose totals still have to be read."""
        for w in widths:
            if w not in self._counted:
                args = (self.op, self.lut_out, self.packed_a, self.packed_b, *self.dims)
                self._counted[w] = count_pairs(*args) if w == 0 else count_steps(*args, w)
        return [self._counted[w] for w in widths if self._counted[w].total is None]

    def _needed(self, bs: int, dtype: torch.dtype, n_a: int, n_b: int) -> tuple[int, ...]:
        """Which plans a launch may consult under the current kernel selection."""
        if (_kernel_choice == "mma" or bs not in (64, 128) or n_a == 0 or n_b == 0 or self.n_out == 0
                or dtype not in (torch.float16, torch.bfloat16, torch.float32)):
            return (0,)
        if _kernel_choice == "umma":
            return (1,)
        if _kernel_choice == "panel":
            return (2,)
        # automatic: the two-block panels are counted first; their walk also yields the pair count the
        # choice needs (``choose`` counts the single-block plan only when it picks that one)
        return (2,) if bs in PANEL_AUTO_BLOCK_SIZES else (1,)

    @property
    def pair(self) -> PairPlan:
        if self._pair is None:
            resolve_counts(self._count((0,)))
            self._pair = finish_pair_plan(self.op, self._counted[0])
        return self._pair

    def step_plan(self, bs: int, dtype: torch.dtype, width: int) -> StepPlan:
        key = (bs, width)
        if key not in self._steps:
            resolve_counts(self._count((width,)))
            n_ctas = _cabi.lib().bsp_umma_num_ctas(_cabi.DATA_DTYPE_CODES[dtype], bs, width)
            self._steps[key] = finish_step_plan(self.op, self.n_out, self._counted[width], n_ctas, bs)
        return self._steps[key]

    def choose(self, bs: int, dtype: torch.dtype, n_a: int, n_b: int) -> tuple[str, int]:
        """(kernel, panel width) for a launch under the current kernel selection."""
        needed = self._needed(bs, dtype, n_a, n_b)
        if needed == (0,):
            return "mma", 0  # also: without operand blocks only zero blocks are written
        resolve_counts(self._count(needed))
        counted = self._counted[needed[0]]
        if counted.total == 0:
            return "mma", 0  # no pair anywhere: only zero blocks are written
        if _kernel_choice != "auto" or needed[0] == 1:
            return "umma", needed[0]
        if counted.total <= PANEL_STEP_RATIO * counted.pairs:
            return "umma", 2
        if 1 not in self._counted:
            # the single-block plan's counts come out of the walk just read
            self._counted[1] = single_block_counts(self.op, self.lut_out, self.packed_a, self.packed_b, *self.dims,
                                                   counted)
        return "umma", 1

    def prepare(self, bs: int, dtype: torch.dtype, n_a: int, n_b: int) -> None:
        """Builds the plan a launch with these arguments will use."""
        kernel, width = self.choose(bs, dtype, n_a, n_b)
        if kernel == "mma":
            self.pair
        else:
            self.step_plan(bs, dtype, width)

    def run(self, a: Tensor, b: Tensor, bs: int, bias: Tensor | None = None) -> Tensor:
        """The product; with ``bias`` (data dtype, one element per output column) every output row
        additionally gets the bias: fused into the tcgen05 kernel's epilogue, a second in-place pass
        (``bsp_bias_add``) behind the mma.sync kernel."""
        kernel, width = self.choose(bs, a.dtype, a.size(0), b.size(0))
        a, b = _cabi.aligned(a), _cabi.aligned(b)
        if bias is not None:
            bias = _cabi.aligned(bias)
        if kernel == "mma":
            out = run_pair_plan(self.pair, a, b, bs)
            if bias is not None and out.size(0):
                with torch.cuda.device(out.device):
                    _cabi.check(_cabi.lib().bsp_bias_add(
                        _cabi.ptr(out), _cabi.ptr(self.lut_out), out.size(0), bs, _cabi.ptr(bias), bias.numel(),
                        _cabi.DATA_DTYPE_CODES[out.dtype], _cabi.ptr(out), _cabi.stream_handle(out.device)),
                        "bsp_bias_add")
            return out
        return run_step_plan(self.step_plan(bs, a.dtype, width), a, b, bs, bias, self.lut_out)


def prepare_products(requests: list[tuple[Product, int, torch.dtype, int, int]]) -> None:
    """Builds the plans the launches ``(product, block size, dtype, n_a, n_b)`` will use, with the
    totals of all of them read from the device in one copy."""
    pending: list[_Counted] = []
    for product, bs, dtype, n_a, n_b in requests:
        pending += product._count(product._needed(bs, dtype, n_a, n_b))
    resolve_counts(pending)
    for product, bs, dtype, n_a, n_b in requests:
        product.prepare(bs, dtype, n_a, n_b)
