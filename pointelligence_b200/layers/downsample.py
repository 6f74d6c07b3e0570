"""Voxel down-sampling of a ragged point batch (mirror of
``layers/downsample.py:15-42``)."""
import torch

from .. import _cabi
from ..internals.grid_sample import grid_sample_filter


@torch.compiler.disable
@_cabi.on_geometry_stream
def downsample(points, sample_inds, grid_size, stride):
    """Returns ``(points_, sample_inds_, grid_size * stride, indices)``."""
    with torch.no_grad():
        grid_size = grid_size * stride
        points_, sample_inds_, indices, _ = grid_sample_filter(
            points=points, grid_size=grid_size, sample_inds=sample_inds,
            reduction="center_nearest", return_mapping=False)
        return points_, sample_inds_, grid_size, indices
