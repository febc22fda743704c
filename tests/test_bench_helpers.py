"""The benchmark's own checking machinery, on CPU: per-batch seeded data do not depend on the number of
shards, the sampled-block check accepts the oracle's result and rejects a corrupted one (all three
products), and the per-batch checksums are exact and shard-independent."""
import torch

import bench
from blksprs_b200.sharding import shard_bounds
from oracle import oracle


def _small(name="config5", batch=4):
    lx, ly, lo, bs, dtype = bench.workload_layouts(name, batch=batch)
    return lx, ly, lo, bs, dtype


def test_per_batch_values_do_not_depend_on_the_shard_count():
    lx, ly, lo, bs, dtype = _small()
    whole = bench.shard_values("config5", lx, ly, lo, bs, dtype, 0, "cpu", 0, 4)
    for world in (2, 4):
        parts = [bench.shard_values("config5", lx, ly, lo, bs, dtype, 0, "cpu", *shard_bounds(4, world, r))
                 for r in range(world)]
        for which in range(3):
            assert torch.equal(torch.cat([p[which] for p in parts]), whole[which])
    other_seed = bench.shard_values("config5", lx, ly, lo, bs, dtype, 1, "cpu", 0, 4)
    assert not torch.equal(other_seed[0], whole[0])


def test_sampled_block_check_accepts_the_oracle_and_sees_a_wrong_block():
    lx, ly, lo, bs, dtype = _small("config2", batch=1)
    bs_small = 16   # the layouts alone define the structure; small blocks keep the CPU products quick
    g = torch.Generator().manual_seed(3)
    x = torch.randn((int(lx.sum()), bs_small, bs_small), generator=g)
    y = torch.randn((int(ly.sum()), bs_small, bs_small), generator=g)
    grad = torch.randn((int(lo.sum()), bs_small, bs_small), generator=g)
    out = oracle.matmul_forward(x, lx, y, ly, lo, bs_small)
    gx, gy = oracle.matmul_backward(grad, x, lx, y, ly, lo, bs_small)
    assert bench.sampled_block_check(x, lx, y, ly, lo, out, bs_small, "nn", 24)["max_rel_err"] < 1e-5
    assert bench.sampled_block_check(grad, lo, y, ly, lx, gx, bs_small, "nt", 24)["max_rel_err"] < 1e-5
    assert bench.sampled_block_check(x, lx, grad, lo, ly, gy, bs_small, "tn", 24)["max_rel_err"] < 1e-5
    bad = out.clone()
    bad[0] += 1.0   # block 0 is always among the sampled ones
    assert bench.sampled_block_check(x, lx, y, ly, lo, bad, bs_small, "nn", 24)["max_rel_err"] > 1e-2
    # a result that is not a number must not slip through (NaN compares false with everything)
    for poison in (float("nan"), float("inf")):
        bad = out.clone()
        bad[0, 3, 5] = poison
        err = bench.sampled_block_check(x, lx, y, ly, lo, bad, bs_small, "nn", 24)["max_rel_err"]
        assert not (err <= 1e-2), err
        bad = out.clone()
        bad[-1] = poison   # the last block is sampled as well; later finite blocks must not reset the verdict
        err = bench.sampled_block_check(x, lx, y, ly, lo, bad, bs_small, "nn", 24)["max_rel_err"]
        assert not (err <= 1e-2), err


def test_batch_checksums_are_exact_and_per_batch():
    lx, ly, lo, bs, dtype = _small()
    out = bench.shard_values("config5", lx, ly, lo, bs, dtype, 0, "cpu", 0, 4)[2]
    sums = bench.batch_checksums(out, lo)
    assert sums.shape == (4,) and sums.dtype == torch.int64
    off = bench.batch_block_offsets(lo).tolist()
    # a shard's checksums equal the same batches' checksums of the whole
    part = bench.batch_checksums(out[off[2]:off[4]], lo[2:4])
    assert torch.equal(part, sums[2:4])
    flipped = out.clone()
    flipped[off[1]] = -flipped[off[1]]   # changes the bit patterns of one block of batch 1
    assert not torch.equal(bench.batch_checksums(flipped, lo)[1], sums[1])
    assert torch.equal(bench.batch_checksums(flipped, lo)[[0, 2, 3]], sums[[0, 2, 3]])
