"""Ragged index helpers (mirror of ``internals/indexing.py:19-90``)."""
from __future__ import annotations

import torch


def cumsum_exclusive(x, return_sum=False):
    """Exclusive prefix sum along dim 0 (and optionally the total as a 0-d tensor)."""
    inc = torch.cumsum(x, dim=0)
    exc = inc - x
    if return_sum:
        total = inc[-1] if x.numel() else x.new_zeros(())
        return exc, total
    return exc


def repeat_interleave_indices(repeats_cumsum, output_size, may_contain_zero_repeats=False):
    """``out[p]`` = index of the segment that position ``p`` falls in, given the
    exclusive prefix sum of the segment lengths."""
    output_size = int(output_size)
    pos = torch.arange(output_size, device=repeats_cumsum.device, dtype=repeats_cumsum.dtype)
    return torch.searchsorted(repeats_cumsum, pos, right=True) - 1
