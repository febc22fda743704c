"""Operations on compressed block-sparse tensors (the matmul path)."""
from .matmul import matmul
from .transpose import transpose

__all__ = ["matmul", "transpose"]
