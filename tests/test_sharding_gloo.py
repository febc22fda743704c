"""Batch sharding across ranks (gloo, world size 2, CPU): shards are independent, and gathering the
per-rank results reproduces the unsharded result.  The per-rank product is the CPU oracle here; on
GPUs it is the CUDA path (tests/test_gpu_c_multi.py)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, result_queue):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from blksprs_b200.sharding import batch_shard
    from oracle import oracle
    import cases
    bs = 16
    lx = cases.bernoulli_layout((5, 4, 6), 0.5, 70)   # 5 batches over 2 ranks: uneven split
    ly = cases.bernoulli_layout((5, 6, 3), 0.5, 71)
    lo = torch.from_numpy(oracle.layout_matmul(lx, ly))
    g = torch.Generator().manual_seed(72)
    x = torch.randn((int(lx.sum()), bs, bs), generator=g)
    y = torch.randn((int(ly.sum()), bs, bs), generator=g)
    xs, lxs = batch_shard(x, lx, world, rank)
    ys, lys = batch_shard(y, ly, world, rank)
    _, los = batch_shard(torch.empty((int(lo.sum()), 0)), lo, world, rank)
    assert xs.data_ptr() == x[xs.storage_offset() // (bs * bs)].data_ptr()  # a view, not a copy
    # per-shard LUTs restart at zero
    assert oracle.packed_indices(lxs).max() == xs.size(0) - 1
    out = oracle.matmul_forward(xs, lxs, ys, lys, los, bs)
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        full = oracle.matmul_forward(x, lx, y, ly, lo, bs)
        result_queue.put(bool(torch.equal(torch.cat(gathered), full)))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds_cover_all_batches():
    from blksprs_b200.sharding import shard_bounds
    for n in (0, 1, 5, 16, 256):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_two_rank_sharded_product_equals_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok
