"""Point convolution as a two-phase op (interface of ``layers/two_phase_conv.py:20-46``).

``build_indices`` does what ``conv_with_stride`` does before it touches the features -- the
down-sampling and the triplet build of ``handle_stride_and_build_triplets`` with the operator's
expanded kernel size -- and, beyond the reference, prepares what the first feature pass would
otherwise prepare lazily behind a host hand-over (the output-stationary MVMR plan of a layer the
engine policy sends there).  ``apply`` is then the convolution alone: kernels only, so a chain of
them can be captured into a CUDA graph.

``handle_stride_and_build_triplets`` updates the geometry object in place, and a model marks the
triplets of a strided convolution dirty before the next layer.  With every build hoisted in front
of every ``apply`` neither can be left to the caller, so the bundle keeps a snapshot of the
geometry as this convolution needs it, and after a strided convolution the geometry handed to the
next op has its triplets marked dirty (the next stride-1 op builds the rulebook of the new level;
consecutive stride-1 ops share one rulebook, as in a serial model).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

import torch

from .metadata import MetaData
from .triplets import handle_stride_and_build_triplets


@dataclass
class ConvBundle:
    meta: MetaData        # i, j, k, seg_offs, contract and the output point count
    next_geom: MetaData   # geometry after the (possibly strided) convolution


class ConvOp:
    separable = True

    def __init__(self, conv_op, stride: float, receptive_field_scaler: float = 1.0, distance_type: str = "ball"):
        self.conv_op = conv_op
        self.stride = float(stride)
        self.rf = float(receptive_field_scaler)
        self.distance_type = distance_type

    def build_indices(self, geom: MetaData) -> ConvBundle:
        m = handle_stride_and_build_triplets(geom, self.stride, self.conv_op.kernel_size_3, self.rf,
                                             distance_type=self.distance_type)
        self._prepare_engine(m)
        snapshot = copy.copy(m)
        if self.stride != 1:
            m.dirty_triplets()
        return ConvBundle(meta=snapshot, next_geom=m)

    def _prepare_engine(self, m: MetaData) -> None:
        """Build the forward MVMR plan now if the engine policy will ask for it."""
        from .. import _cabi

        weight = getattr(self.conv_op, "weight", None)
        if weight is not None and weight.dim() == 4 and m.i is not None and m.i.is_cuda and m.seg_offs is not None:
            _cabi.prepare_mvmr(weight, m.j, m.i, m.seg_offs, m.num_points())

    def apply(self, x: torch.Tensor, b: ConvBundle) -> torch.Tensor:
        m = b.meta
        return self.conv_op(x, m.i, m.j, m.k, m.num_points(), contract=m.contract, seg_offs=m.seg_offs)
