"""Batch sharding of compressed tensors for multi-GPU runs.

The block-sparse matmul has no exchange step: every output block depends only on blocks of the
same batch index (blksprs/ops/matmul.py:201-215 index both reverse LUTs by the output block's
batch).  Compressed tensors are ordered batch-major (blksprs/utils/tools.py:33-35), so the blocks
of a contiguous batch range are a contiguous row range of the compressed tensor: a shard is a
zero-copy view, and each rank builds its own LUTs from its layout slice (indices restart at 0,
exactly as if the reference ran on the slice).
"""
from __future__ import annotations

import torch
from torch import Tensor


def shard_bounds(n_batches: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous batch range ``[begin, end)`` of ``rank``; sizes differ by at most one."""
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    base, extra = divmod(n_batches, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def block_offsets(sparsity_layout: Tensor) -> Tensor:
    """int64 ``(B + 1)``: index of the first compressed block of every batch (host tensor)."""
    per_batch = (sparsity_layout.reshape(sparsity_layout.size(0), -1) != 0).sum(dim=1).to(torch.int64).cpu()
    out = torch.zeros(per_batch.numel() + 1, dtype=torch.int64)
    out[1:] = torch.cumsum(per_batch, 0)
    return out


def batch_shard(compressed: Tensor, sparsity_layout: Tensor, world_size: int, rank: int,
                offsets: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """The rank's slice of a compressed tensor and of its layout (views, nothing is copied)."""
    begin, end = shard_bounds(sparsity_layout.size(0), world_size, rank)
    if offsets is None:
        offsets = block_offsets(sparsity_layout)
    lo, hi = int(offsets[begin]), int(offsets[end])
    return compressed[lo:hi], sparsity_layout[begin:end]
