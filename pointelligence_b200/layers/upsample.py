"""Up-sampling convolution (mirror of ``layers/upsample.py:19-247``): every
point of the parent (fine) cloud gathers features from nearby points of the
down-sampled cloud through a ``PointConv3d``.  The rulebook is either a fresh
radius search (coarse points as sources, fine points as queries) or the edges
the strided convolution cached on the parent (``straight_recover``)."""
from __future__ import annotations

import math
import warnings
from functools import partial
from typing import Tuple

import torch
from torch import Tensor

from ..sparse_engines._seg_offs import kernel_offset_segments
from .contract import TripletContract
from .conv import PointConv3d
from .metadata import MetaData
from .triplets import (build_triplets, build_triplets_segmented, radius_scaler_for_kernel_size,
                       should_use_direct_segmented_triplets, voxelize_3d)


def recompute_cached_upsample_k(m_low: MetaData, kernel_size: int) -> Tensor:
    """Taps of the cached up-sampling edges for another kernel size: the edge
    graph does not depend on the kernel, only the quantisation of the
    source-minus-query offset (on the fine grid) does."""
    with torch.no_grad():
        offset = m_low.points[m_low.parent.j_upsample.long()] - m_low.parent.points[m_low.parent.i_upsample.long()]
        return voxelize_3d(kernel_size, offset, grid_size=m_low.parent.grid_size)


class Upsample(torch.nn.Module):
    """``output[i_high] += input[j_low] @ W[k]`` from the coarse cloud ``m_low`` to its parent."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, bias: bool = True,
                 receptive_field_scaler: float = 1.0, distance_type: str = "ball",
                 straight_recover: bool = False, recompute_k: bool = False):
        super().__init__()
        self.conv = PointConv3d(in_channels=in_channels, out_channels=out_channels, kernel_size=kernel_size, bias=bias)
        self.receptive_field_scaler = receptive_field_scaler
        self.distance_type = distance_type
        self.kernel_size = kernel_size
        self.straight_recover = straight_recover
        self.recompute_k = recompute_k

    def forward(self, x_low: Tensor, m_low: MetaData) -> Tuple[Tensor, MetaData]:
        if m_low.parent is None:
            raise ValueError("Parent information is required for upsampling. "
                             "Make sure to use conv_with_stride with stride > 1 to save parent info.")
        hi = m_low.parent
        cached = self.straight_recover and hi.i_upsample is not None and hi.j_upsample is not None and (
            self.recompute_k or hi.k_upsample is not None)
        if cached and self.recompute_k:
            k, order = torch.sort(recompute_cached_upsample_k(m_low, self.kernel_size), stable=True)
            i_high, j_low = hi.i_upsample[order], hi.j_upsample[order]
            seg_offs = kernel_offset_segments(k, self.kernel_size ** 3)
        elif cached:
            i_high, j_low, k, seg_offs = hi.i_upsample, hi.j_upsample, hi.k_upsample, hi.seg_offs_upsample
        else:
            scaler = radius_scaler_for_kernel_size(self.kernel_size, self.receptive_field_scaler, self.distance_type)
            radius = m_low.grid_size * scaler
            if radius < m_low.grid_size * math.sqrt(3):
                warnings.warn(f"Upsample search radius ({radius:.4f}) is smaller than the worst-case voxel diagonal "
                              f"({m_low.grid_size * math.sqrt(3):.4f} = grid_size_low * sqrt(3)). Some high-res points "
                              "in isolated voxels may find zero neighbors. Increase receptive_field_scaler "
                              f"(currently {self.receptive_field_scaler}).")
            common = dict(points=m_low.points, sample_inds=m_low.sample_inds, sample_sizes=m_low.sample_sizes,
                          neighbor_radius=radius, query_points=hi.points, query_sample_inds=hi.sample_inds,
                          query_sample_sizes=hi.sample_sizes, return_num_neighbors=False, radius_scaler=scaler)
            if self.distance_type == "ball" and should_use_direct_segmented_triplets(self.kernel_size):
                i_high, j_low, k, seg_offs, _ = build_triplets_segmented(kernel_size=self.kernel_size, **common)
            else:
                i_high, j_low, k, _ = build_triplets(
                    kernel_indexer=partial(voxelize_3d, kernel_size=self.kernel_size), sort_by="k", **common)
                seg_offs = kernel_offset_segments(k, self.kernel_size ** 3)
        x_high = self.conv(x_low, i_high, j_low, k, hi.points.shape[0], contract=TripletContract.submanifold(),
                           seg_offs=seg_offs)
        m_high = MetaData(points=hi.points, sample_inds=hi.sample_inds, sample_sizes=hi.sample_sizes,
                          grid_size=hi.grid_size, i=i_high, j=j_low, k=k, seg_offs=seg_offs, parent=hi.parent)
        return x_high, m_high
