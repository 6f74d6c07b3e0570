"""Public MVMR operator.

Stands in for ``sparse_engines/mvmr_triton.py:148-254`` (the operator behind
``sparse_engines.ops.sparse_matrix_vector_multiplication_reduction``): same
argument order, same promotion of mixed dtypes, same output shape and dtype,
same autograd duals (weight gradient = VVOR, input gradient = MVMR with the
weight used transposed).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ._dispatch_override import current_engine, current_mode, warn_pt_fallback
from ._ops import mvmr_op
from ._seg_offs import is_sorted_cached, kernel_offset_segments


def _segments_or_taps(sort_key, num_bins, seg_offs, site, **ctx):
    """(seg_offs, tap_idx) for the C ABI: segment offsets when the key is
    sorted (given, or proven once per tensor), the raw key otherwise."""
    if seg_offs is not None:
        return seg_offs, None
    if sort_key.numel() == 0 or is_sorted_cached(sort_key):
        return kernel_offset_segments(sort_key, num_bins), None
    if current_mode() == "auto":
        warn_pt_fallback(site, "index is not sorted", **ctx)
    return None, sort_key


def sparse_matrix_vector_multiplication_reduction(
        a: Tensor, a_idx: Tensor, b: Tensor, b_idx: Tensor, o_idx: Tensor, n_o: int,
        seg_offs: Optional[Tensor] = None) -> Tensor:
    """``o[o_idx[t], g, :] += b[b_idx[t], g, :] @ a[a_idx[t], g, :, :]``.

    a (K,G,C,M); b (N_b,G,C); returns (n_o,G,M) in ``promote_types(a, b)``.
    """
    if a.dtype != b.dtype:
        promoted = torch.promote_types(a.dtype, b.dtype)
        a, b = a.to(promoted), b.to(promoted)
    K, G, C, M = a.shape
    seg, taps = _segments_or_taps(a_idx, K, seg_offs, "mvmr", K=K, G=G, C=C, M=M)
    out = mvmr_op(a.contiguous(), b.reshape(b.shape[0], G * C), b_idx, o_idx, seg, taps, int(n_o),
                  False, current_engine())
    return out.view(int(n_o), G, M)
