"""Grid-cell indices and collision-free keys (mirror of
``internals/grid_indexing.py:20-111``).  Host-side torch code used by the
generic rulebook builders; the down-sampling hot path bins and sorts inside
the CUDA library instead."""
from __future__ import annotations

import torch


def compute_grid_indices(points, grid_size, sample_inds=None, dtype=torch.int32):
    """Cell of every point (Python-style floor division), optional sample column."""
    grid = points.div(grid_size, rounding_mode="floor").to(dtype)
    if sample_inds is not None:
        grid = torch.cat((grid, sample_inds.unsqueeze(-1).to(dtype)), dim=1)
    return grid.contiguous()


def reduce_indices_to_1d(inds, inds_min=None, inds_stride=None, dtype=None):
    """Mixed-radix key: first column fastest, last column slowest."""
    assert inds.dtype is not torch.float16
    if inds_min is None:
        inds_min = torch.amin(inds, dim=0, keepdim=True)
    if inds_stride is None:
        step = torch.amax(inds, dim=0, keepdim=True) + 1 - inds_min
        cum = step.cumprod(dim=-1, dtype=torch.int64)
        dtype = torch.int64
        inds_stride = cum.roll(1, dims=-1)
        inds_stride[0, 0] = 1
    keys = ((inds - inds_min).to(dtype) * inds_stride.to(dtype)).sum(dim=-1)
    return keys, inds_min, inds_stride, dtype


def reduction_params_from_indices(*indices):
    if not indices:
        raise ValueError("at least one index tensor is required")
    lo = torch.stack([x.amin(dim=0) for x in indices]).amin(dim=0, keepdim=True)
    hi = torch.stack([x.amax(dim=0) for x in indices]).amax(dim=0, keepdim=True)
    cum = (hi - lo + 1).cumprod(dim=-1, dtype=torch.int64)
    stride = cum.roll(1, dims=-1)
    stride[0, 0] = 1
    return lo, stride, torch.int64


def build_sorted_grid_segments(grid_inds, *, return_inverse=False):
    """(sorter, segment lengths, optional segment id per input row)."""
    keys, _, _, _ = reduce_indices_to_1d(grid_inds)
    sorted_keys, sorter = torch.sort(keys, stable=True)
    if return_inverse:
        _, inv_sorted, counts = torch.unique_consecutive(sorted_keys, return_inverse=True, return_counts=True)
        inverse = torch.empty_like(inv_sorted)
        inverse.index_copy_(0, sorter, inv_sorted)
    else:
        _, counts = torch.unique_consecutive(sorted_keys, return_counts=True)
        inverse = None
    return sorter, counts, inverse
