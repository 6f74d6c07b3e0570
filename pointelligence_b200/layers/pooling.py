"""Global and local pooling over ragged point features.

Mirror of the reference's ``layers/pooling.py:20-47``: ``GlobalPool`` reduces
every sample of the batch to one row, ``max_pool3d`` takes the maximum over
each output point's neighbourhood after an optional strided down-sampling.
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from ..sparse_engines.segment_reduce import indexed_segment_reduce, large_segment_reduce
from .metadata import MetaData
from .triplets import handle_stride_and_build_triplets

__all__ = ["GlobalPool", "max_pool3d"]


class GlobalPool(torch.nn.Module):
    def __init__(self, method="mean"):
        super().__init__()
        assert method in ["max", "min", "mean"]
        self.method = method

    def forward(self, x: Tensor, sample_sizes: Tensor) -> Tensor:
        return large_segment_reduce(x, reduce=self.method, lengths=sample_sizes)

    def extra_repr(self) -> str:
        return f"method: {self.method}"


def max_pool3d(x: Tensor, m: MetaData, kernel_size: int, stride: float) -> Tuple[Tensor, MetaData]:
    # triplets ordered by output point: the neighbours of output i are the
    # num_neighbors[i] consecutive entries of j
    m = handle_stride_and_build_triplets(m, stride, kernel_size, sort_by="i", return_num_neighbors=True)
    out = indexed_segment_reduce(x, reduce="max", indices=m.j, lengths=m.num_neighbors)
    return out, m
