"""The kernels' own range checks of plan indices, exercised through the C ABI with a host-corrupted plan.

Both matmul kernels compare every operand block index they take from a plan with the operand's block
count before they use it (the reference guards its loads with masks, blksprs/ops/matmul.py:204-209,
230-231; invalid metadata must never become an out-of-range access).  A bad index makes the kernel
write ``BSP_ERR_DEVICE_RANGE`` into the status word and use block 0 in place of the bad index (the
mma.sync tile kernel for larger blocks skips the pair).  Here one index of an otherwise valid plan is
replaced by ``n`` (one past the end) or by ``-2``; the operand buffers are allocated with a few blocks of slack, so that even a
wrong guard could not leave the allocation.  Expected: the status word holds the range code, every
output block that does not depend on the corrupted entry equals the clean run bit for bit, and the
device keeps working.
"""
import pytest
import torch

from gpu_util import DEV, make_case

pytestmark = pytest.mark.gpu


def _setup(bs, dtype):
    from blksprs_b200.ops.matmul import matmul_build_layout_cache, _PLANS
    case = make_case(2, 4 * bs, 5 * bs, 3 * bs, bs, 0.6, dtype, seed=5, out_layout="ones")
    lx, ly, lo = (case[k].to(DEV) for k in ("lx", "ly", "lo"))
    n_x, n_y = case["x"].size(0), case["y"].size(0)
    slack = 4
    # operands with slack blocks behind the ones the layouts know about
    x = torch.zeros((n_x + slack, bs, bs), dtype=dtype, device=DEV)
    y = torch.zeros((n_y + slack, bs, bs), dtype=dtype, device=DEV)
    x[:n_x] = case["x"].to(DEV)
    y[:n_y] = case["y"].to(DEV)
    cache = matmul_build_layout_cache(None, lx, ly, lo)
    return cache[_PLANS].forward, x, y, n_x, n_y


def _status():
    from blksprs_b200 import plan
    word = plan.status_word(torch.device(DEV))
    code = int(word.item())
    word.zero_()
    return code


def _run_mma(product, pairs, x, y, n_x, n_y, bs):
    from blksprs_b200 import _cabi, plan
    p = product.pair
    out = torch.full((p.n_out, bs, bs), float("nan"), dtype=x.dtype, device=x.device)
    _cabi.check(_cabi.lib().bsp_matmul_mma(
        x.data_ptr(), n_x, y.data_ptr(), n_y, out.data_ptr(), p.n_out, p.offsets.data_ptr(), pairs.data_ptr(), bs,
        _cabi.DATA_DTYPE_CODES[x.dtype], p.op, plan.status_word(x.device).data_ptr(),
        _cabi.stream_handle(x.device)), "bsp_matmul_mma")
    torch.cuda.synchronize()
    return out


def _run_umma(product, sp, steps, x, y, n_x, n_y, bs):
    from blksprs_b200 import _cabi, plan
    out = torch.full((sp.n_out, bs, bs), float("nan"), dtype=x.dtype, device=x.device)
    _cabi.check(_cabi.lib().bsp_matmul_umma(
        x.data_ptr(), n_x, y.data_ptr(), n_y, out.data_ptr(), sp.n_out, None, None,
        sp.panel_first.data_ptr(), sp.n_panels, sp.step_offsets.data_ptr(), steps.data_ptr(), sp.touched.data_ptr(),
        sp.unit_panel.data_ptr(), sp.unit_step.data_ptr(), sp.n_units, None, sp.width, bs,
        _cabi.DATA_DTYPE_CODES[x.dtype], sp.op, plan.status_word(x.device).data_ptr(),
        _cabi.stream_handle(x.device)), "bsp_matmul_umma")
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("bad", ["past_end", "minus_two"])
@pytest.mark.parametrize("operand", ["a", "b"])
def test_mma_kernel_flags_bad_pair(bad, operand):
    from blksprs_b200 import _cabi
    bs = 32
    product, x, y, n_x, n_y = _setup(bs, torch.float16)
    assert _status() == 0
    clean = _run_mma(product, product.pair.pairs, x, y, n_x, n_y, bs)
    assert _status() == 0
    pairs = product.pair.pairs.clone()
    victim = product.pair.n_pairs // 2
    col = 0 if operand == "a" else 1
    n = n_x if operand == "a" else n_y
    pairs[victim, col] = n if bad == "past_end" else -2
    got = _run_mma(product, pairs, x, y, n_x, n_y, bs)
    assert _status() == _cabi.ERR_DEVICE_RANGE
    offsets = product.pair.offsets.cpu()
    hit = int(torch.searchsorted(offsets, torch.tensor(victim), right=True)) - 1  # the output block of that pair
    keep = torch.ones(clean.size(0), dtype=torch.bool)
    keep[hit] = False
    assert torch.equal(got[keep.to(DEV)], clean[keep.to(DEV)])
    assert not torch.isnan(got.float()).any()
    # the device is still usable and the clean plan still gives the clean result
    assert torch.equal(_run_mma(product, product.pair.pairs, x, y, n_x, n_y, bs), clean)
    assert _status() == 0


@pytest.mark.parametrize("width", [1, 2])
@pytest.mark.parametrize("bad", ["past_end", "minus_two"])
@pytest.mark.parametrize("operand", ["a", "b"])
def test_tcgen05_kernel_flags_bad_step(bad, operand, width):
    from blksprs_b200 import _cabi
    bs = 64
    product, x, y, n_x, n_y = _setup(bs, torch.bfloat16)
    sp = product.step_plan(bs, torch.bfloat16, width)
    assert _status() == 0
    clean = _run_umma(product, sp, sp.steps, x, y, n_x, n_y, bs)
    assert _status() == 0
    steps = sp.steps.clone()
    victim = sp.n_steps // 2
    rec = steps[victim].tolist()
    if operand == "a":
        col, n = 0, n_x
    else:
        col = 1 + [q for q in range(4) if (rec[5] >> q) & 1][0]   # a column the step really uses
        n = n_y
    steps[victim, col] = n if bad == "past_end" else -2
    got = _run_umma(product, sp, steps, x, y, n_x, n_y, bs)
    assert _status() == _cabi.ERR_DEVICE_RANGE
    # the panel of that step holds the only output blocks that may differ
    step_off = sp.step_offsets.cpu()
    panel = int(torch.searchsorted(step_off, torch.tensor(victim), right=True)) - 1
    first = sp.panel_first.cpu()
    keep = torch.ones(clean.size(0), dtype=torch.bool)
    keep[int(first[panel]):int(first[panel + 1])] = False
    assert torch.equal(got[keep.to(DEV)], clean[keep.to(DEV)])
    assert not torch.isnan(got.float()).any()
    assert torch.equal(_run_umma(product, sp, sp.steps, x, y, n_x, n_y, bs), clean)
    assert _status() == 0
