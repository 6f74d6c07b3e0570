"""Operator facade (mirror of ``sparse_engines/ops.py:1-6``)."""
from .mvmr import sparse_matrix_vector_multiplication_reduction
from .segment_reduce import indexed_segment_reduce, large_segment_reduce
from .vvor import sparse_vector_vector_outer_product_reduction

__all__ = ["sparse_matrix_vector_multiplication_reduction",
           "sparse_vector_vector_outer_product_reduction",
           "large_segment_reduce", "indexed_segment_reduce"]
