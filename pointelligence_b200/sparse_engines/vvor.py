"""Public VVOR operator.

Stands in for ``sparse_engines/vvor_triton.py:116-223`` (the operator behind
``sparse_engines.ops.sparse_vector_vector_outer_product_reduction``).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ._dispatch_override import current_engine
from ._ops import vvor_op
from .mvmr import _segments_or_taps


def sparse_vector_vector_outer_product_reduction(
        a: Tensor, a_idx: Tensor, b: Tensor, b_idx: Tensor, o_idx: Tensor, n_o: int,
        seg_offs: Optional[Tensor] = None) -> Tensor:
    """``o[o_idx[t], g, m, c] += a[a_idx[t], g, m] * b[b_idx[t], g, c]``.

    a (N_a,G,M); b (N_b,G,C); returns (n_o,G,M,C) in ``promote_types(a, b)``.
    """
    if a.dtype != b.dtype:
        promoted = torch.promote_types(a.dtype, b.dtype)
        a, b = a.to(promoted), b.to(promoted)
    seg, taps = _segments_or_taps(o_idx, int(n_o), seg_offs, "vvor", K=int(n_o), G=a.shape[1],
                                  C=b.shape[2], M=a.shape[2])
    return vvor_op(a.contiguous(), a_idx, b.contiguous(), b_idx, seg, taps, int(n_o), current_engine())
