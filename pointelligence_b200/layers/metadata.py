"""Spatial bookkeeping that travels with the features (mirror of
``layers/metadata.py:20-158``)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from functools import partial
from typing import Callable, Optional, Tuple

from torch import Tensor
from torch.nn.modules.utils import _triple

from .contract import TripletContract


@dataclass(kw_only=True)
class MetaData:
    points: Tensor
    sample_inds: Tensor
    sample_sizes: Tensor
    grid_size: float
    i: Tensor = None
    j: Tensor = None
    k: Tensor = None
    seg_offs: Tensor = None
    num_neighbors: Tensor = None
    downsample_indices: Tensor = None
    contract: Optional[TripletContract] = None
    i_upsample: Tensor = None
    j_upsample: Tensor = None
    k_upsample: Tensor = None
    seg_offs_upsample: Tensor = None
    parent: Optional["MetaData"] = None
    kernel_size: Optional[Tuple[int, int, int]] = None
    receptive_field_scaler: float = 1.0
    sort_by: str = "k"
    return_num_neighbors: bool = False
    query_points: Optional[Tensor] = None
    query_sample_inds: Optional[Tensor] = None
    query_sample_sizes: Optional[Tensor] = None
    distance_type: str = "ball"
    auto_build_triplets: bool = True

    def __post_init__(self):
        if self.auto_build_triplets and self.kernel_size is not None and self.empty_triplets():
            self.build_triplets()

    def build_triplets(self, kernel_size=None, neighbor_radius: Optional[float] = None,
                       kernel_indexer: Optional[Callable] = None, **kwargs):
        from ..sparse_engines._seg_offs import kernel_offset_segments
        from .triplets import (build_triplets, build_triplets_segmented, radius_scaler_for_kernel_size,
                               should_use_direct_segmented_triplets, voxelize_3d)

        kernel_size = kernel_size or self.kernel_size
        if kernel_size is None:
            raise ValueError("kernel_size must be provided either in __init__ or build_triplets()")
        opt = lambda name: kwargs.get(name, getattr(self, name))
        sort_by, distance_type = opt("sort_by"), opt("distance_type")
        radius_scaler = radius_scaler_for_kernel_size(kernel_size, opt("receptive_field_scaler"), distance_type)
        if neighbor_radius is None:
            neighbor_radius = self.grid_size * radius_scaler
        common = dict(points=self.points, sample_inds=self.sample_inds, sample_sizes=self.sample_sizes,
                      neighbor_radius=neighbor_radius, query_points=opt("query_points"),
                      query_sample_inds=opt("query_sample_inds"),
                      query_sample_sizes=opt("query_sample_sizes"),
                      return_num_neighbors=opt("return_num_neighbors"), radius_scaler=radius_scaler)
        if (kernel_indexer is None and sort_by == "k" and distance_type == "ball"
                and should_use_direct_segmented_triplets(kernel_size)):
            i, j, k, seg_offs, num_neighbors = build_triplets_segmented(kernel_size=kernel_size, **common)
        else:
            indexer = kernel_indexer or partial(voxelize_3d, kernel_size=kernel_size)
            i, j, k, num_neighbors = build_triplets(kernel_indexer=indexer, sort_by=sort_by, **common)
            seg_offs = (kernel_offset_segments(k, math.prod(_triple(kernel_size)))
                        if sort_by == "k" else None)
        self.i, self.j, self.k, self.seg_offs, self.num_neighbors = i, j, k, seg_offs, num_neighbors
        self.contract = TripletContract(k_sorted=(sort_by == "k"))

    def dirty_triplets(self):
        self.i = self.j = self.k = self.seg_offs = self.contract = None

    def empty_triplets(self):
        if self.i is None or self.j is None or self.k is None:
            assert self.i is None and self.j is None and self.k is None
            return True
        return False

    def num_points(self):
        return self.points.shape[0]
