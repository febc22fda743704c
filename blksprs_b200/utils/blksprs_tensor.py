"""Marker type for compressed block-sparse tensors.

Mirrors ``BlksprsTensor`` of the reference (blksprs/utils/blksprs_tensor.py:7-25):
a ``torch.Tensor`` subclass that only changes ``repr``; ``wrap`` leaves the
tensor untouched while Dynamo traces.
"""
import torch
from torch import Tensor


class BlksprsTensor(Tensor):
    """A compressed block-sparse tensor ``(n_sparse_blocks, bs, bs)``."""

    def __repr__(self, *, tensor_contents=None):
        inner = Tensor.__repr__(Tensor(self), tensor_contents=tensor_contents)
        return f"BlksprsTensor({inner})"

    @staticmethod
    def wrap(tensor: Tensor) -> "BlksprsTensor":
        """Marks ``tensor`` as compressed (a no-op inside a Dynamo-traced region)."""
        if torch._dynamo.is_compiling():
            return tensor  # type: ignore[return-value]
        return BlksprsTensor(tensor)
