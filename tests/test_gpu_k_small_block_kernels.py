"""The mma.sync kernels for block sizes 16 and 32 (operands streamed into registers; fp32 blocks of 32
through a ring of copy stages) on problems large enough that a warp takes chunks of many consecutive
output blocks: the pair stream then crosses output-block boundaries (including blocks without any
pair, which must come out as zeros), crosses the 32-record windows in which the pair list is fetched,
passes from one chunk to the next with the next chunk's first pairs already requested, and wraps the
slots (ring stages) many times.  Forward and both backward products against the CPU oracle; the small
shapes of the reference's test matrix (one block per warp) are covered by the general matmul tests."""
import pytest
import torch

from gpu_util import check_case, make_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("bs,batch,kept", [(16, 80, 0.5), (16, 24, 0.15), (32, 40, 0.5)],
                         ids=["bs16-chunk32", "bs16-sparse", "bs32"])
def test_chunked_pair_stream_matches_oracle(bs, batch, kept, dtype):
    # 64 x 64 output blocks per batch on an all-ones output layout: with few operand blocks many
    # output blocks have no pair at all
    case = make_case(batch, 64 * bs, 64 * bs, 32 * bs, bs, kept, dtype, seed=3, out_layout="ones")
    check_case(case)


def test_run_to_run_bit_equal():
    """No atomics and a fixed summation order per output block: two runs give identical bits."""
    import blksprs_b200 as bsp
    case = make_case(24, 1024, 1024, 512, 16, 0.4, torch.float16, seed=9, out_layout="ones")
    dev = "cuda:0"
    args = (case["x"].to(dev), case["lx"].to(dev), case["y"].to(dev), case["ly"].to(dev), case["lo"].to(dev), 16)
    first = bsp.ops.matmul(*args)
    second = bsp.ops.matmul(*args)
    assert torch.equal(first, second)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
@pytest.mark.parametrize("bs", [16, 32])
def test_every_pair_count_per_chunk(bs, dtype):
    """Few output blocks, so that a warp's chunk is a single block, and block r of an output column has
    exactly r pairs (row r of X holds its first r blocks, Y is full): the per-chunk pair streams have
    every length from 0 to 71 (shorter than the slots in flight, equal to them, one record window, a
    window and a bit, more than two windows), and a chunk without pairs sits before and between
    chunks with pairs.  The backward products see the transposed pattern (many pairs per block of X's
    gradient for the long rows, none for blocks of Y's gradient that no row reaches)."""
    rows, cols = 72, 2
    lx = torch.zeros((1, rows, rows), dtype=torch.bool)
    for r in range(rows):
        lx[0, r, :r] = True
    ly = torch.ones((1, rows, cols), dtype=torch.bool)
    lo = torch.ones((1, rows, cols), dtype=torch.bool)
    g = torch.Generator().manual_seed(21)
    case = dict(x=torch.randn((int(lx.sum()), bs, bs), generator=g).to(dtype), lx=lx,
                y=torch.randn((int(ly.sum()), bs, bs), generator=g).to(dtype), ly=ly, lo=lo, bs=bs,
                grad=torch.randn((int(lo.sum()), bs, bs), generator=g).to(dtype))
    check_case(case, tol=4e-3 if dtype == torch.float32 else None)
