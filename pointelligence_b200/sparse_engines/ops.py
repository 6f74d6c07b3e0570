"""Operator facade (mirror of ``sparse_engines/ops.py:1-6`` for the two
convolution primitives)."""
from .mvmr import sparse_matrix_vector_multiplication_reduction
from .vvor import sparse_vector_vector_outer_product_reduction

__all__ = ["sparse_matrix_vector_multiplication_reduction",
           "sparse_vector_vector_outer_product_reduction"]
