"""Sparsity-layout helpers of the matmul path."""
from .sparsity_layout import (
    build_sparsity_layout_full,
    build_sparsity_layout_matmul,
    build_sparsity_layout_matmul_fast,
    build_sparsity_layout_matmul_outer,
)

__all__ = [
    "build_sparsity_layout_full",
    "build_sparsity_layout_matmul",
    "build_sparsity_layout_matmul_fast",
    "build_sparsity_layout_matmul_outer",
]
