"""Two ranks on two GPUs: each runs the CUDA matmul on its batch shard with its own LUTs; NCCL gathers
the results, which must equal the single-GPU result bit for bit (no collective on the data path)."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import blksprs_b200 as bs
    from blksprs_b200.sharding import batch_shard
    from gpu_util import make_case
    bsz = 64
    case = make_case(6, 256, 192, 320, bsz, 0.5, torch.bfloat16, seed=21, out_layout="exact")
    x, lx, y, ly, lo = (case[k] for k in ("x", "lx", "y", "ly", "lo"))
    xs, lxs = batch_shard(x, lx, world, rank)
    ys, lys = batch_shard(y, ly, world, rank)
    _, los = batch_shard(torch.empty((int(lo.sum()), 0)), lo, world, rank)
    out = bs.ops.matmul(xs.to(dev), lxs.to(dev), ys.to(dev), lys.to(dev), los.to(dev), bsz)
    counts = torch.tensor([out.size(0)], device=dev)
    all_counts = [torch.zeros_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts)
    cap = int(max(c.item() for c in all_counts))
    padded = torch.zeros((cap, bsz, bsz), dtype=out.dtype, device=dev)
    padded[:out.size(0)] = out
    gathered = [torch.zeros_like(padded) for _ in range(world)]
    dist.all_gather(gathered, padded)
    if rank == 0:
        joined = torch.cat([g[:int(c.item())] for g, c in zip(gathered, all_counts)])
        full = bs.ops.matmul(x.to(dev), lx.to(dev), y.to(dev), ly.to(dev), lo.to(dev), bsz)
        q.put(bool(torch.equal(joined, torch.Tensor(full))))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_batch_shards_equal_single_gpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert ok
