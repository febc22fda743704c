"""Operations on compressed block-sparse tensors (the matmul path and the ops around it)."""
from .conversion import from_blksprs, to_blksprs, to_dense, to_dense_shaped, to_sparse, to_sparse_shaped
from .matmul import matmul
from .matmul_softmax import matmul_softmax
from .softmax import softmax, softmax_fused, softmax_regular
from .transpose import transpose

__all__ = ["from_blksprs", "matmul", "matmul_softmax", "softmax", "softmax_fused", "softmax_regular", "to_blksprs", "to_dense", "to_dense_shaped", "to_sparse", "to_sparse_shaped",
           "transpose"]
