"""Grid down-sampling (mirror of ``internals/grid_sample.py:42-121``).

``center_nearest`` -- the reduction the convolution path uses -- runs entirely
in the CUDA library: binning (Python-style floor division), 64-bit cell keys,
radix sort, segment heads and the per-cell arg-min with the reference's fp32
arithmetic and lowest-index tie break.  The other reductions reuse its cell
assignment and finish with a handful of torch calls.
"""
from __future__ import annotations

import torch

from .. import _cabi


@_cabi.on_geometry_stream
def grid_sample_filter(points, grid_size, sample_inds=None, reduction="center_nearest",
                       return_mapping=False, center_nearest_impl="auto"):
    """Returns ``(points_f (S,3), sample_inds_f (S,) or None, indices (S,) int64, mapping or None)``.

    Cells are emitted in ascending (sample, z, y, x) order.  ``center_nearest_impl``
    is accepted for source compatibility; there is one implementation.
    """
    reductions = ["center", "center_nearest", "random", "mean"]
    assert reduction in reductions, "reduction should be in one of %s!" % " ".join(reductions)
    if center_nearest_impl not in ("auto", "torch", "triton"):
        raise ValueError("center_nearest_impl must be one of: auto, torch, triton")
    _cabi.require_cuda(points, sample_inds)
    if points.dim() != 2 or points.shape[1] != 3:
        raise ValueError(f"points must have shape [N, 3], got {tuple(points.shape)}")
    dev = points.device
    if points.shape[0] == 0:
        idx = torch.empty(0, dtype=torch.int64, device=dev)
        si = None if sample_inds is None else sample_inds[idx]
        return points[idx], si, idx, (idx.clone() if return_mapping else None)

    if points.dtype != torch.float32:
        # The reference bins half-precision clouds in their own precision; the
        # convolution path only ever passes fp32 coordinates.
        raise NotImplementedError("grid_sample_filter expects float32 points")
    pts32 = points
    need_map = return_mapping or reduction == "mean"
    indices, out_pts, out_smp, mapping = _cabi.grid_sample_center_nearest(
        pts32, float(grid_size), sample_inds, need_map)
    sample_f = None if sample_inds is None else sample_inds[indices]
    if reduction in ("center_nearest", "random"):
        points_f = out_pts
    elif reduction == "center":
        cells = points[indices].div(grid_size, rounding_mode="floor")
        points_f = (cells + 0.5).mul_(grid_size)
    else:  # mean
        points_f = torch.zeros((indices.numel(), 3), dtype=points.dtype, device=dev)
        points_f.index_reduce_(0, mapping, points, reduce="mean", include_self=False)
    return points_f, sample_f, indices, (mapping if return_mapping else None)
