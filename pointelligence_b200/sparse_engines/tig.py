"""Tap-sorted convolution engine interface.

Mirror of the reference's production engine module ``sparse_engines/tig.py``:
``TigIndex`` (:772-935), ``tig_forward`` (:1090-1206), ``tig_grad_input``
(:1220-1309), ``tig_grad_weight`` (:1390-1465) and the differentiable
``tig_mvmr`` (:1566-1600) with its 12-argument operator schema (:1508-1563).
The index object carries the same attributes the reference's callers read
(``flat_i``, ``flat_j``, ``flat_seg``, ``N``, ``N_in``, ``K``, ``T``,
``exact_cover_*``, ``uniform_seg_len``); only the flat, tap-sorted orientation
exists here (the reference's hybrid orientation is a bench-only mode).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import _cabi
from ._dispatch_override import current_engine, resolve_input_precision
from ._ops import mvmr_op, vvor_op
from ._seg_offs import kernel_offset_segments

__all__ = ["TigIndex", "tig_forward", "tig_grad_input", "tig_grad_weight", "tig_mvmr"]


def _maybe_int(x):
    return x if isinstance(x, torch.SymInt) else int(x)


class TigIndex:
    """Tap-sorted triplet index: ``out[flat_i[t]] += feat[flat_j[t]] @ W[tap(t)]``."""

    def __init__(self, i, j, k, n_out, num_kernel_offsets=27, build_hybrid=False,
                 assume_sorted=False, n_in=None, exact_cover_out=False, exact_cover_in=False,
                 uniform_seg_len=None):
        self.exact_cover_out = bool(exact_cover_out)
        self.exact_cover_in = bool(exact_cover_in)
        self.N = _maybe_int(n_out)
        self.N_in = _maybe_int(n_in) if n_in is not None else self.N
        self.K = int(num_kernel_offsets)
        self.T = _maybe_int(i.numel())
        if self.T and not assume_sorted and not bool((k[1:] >= k[:-1]).all()):
            order = torch.argsort(k, stable=True)
            i, j, k = i[order], j[order], k[order]
        self.flat_i, self.flat_j = i, j
        self.uniform_seg_len = int(uniform_seg_len) if uniform_seg_len is not None else None
        if self.uniform_seg_len is not None:
            assert self.uniform_seg_len * self.K == self.T
            self.flat_seg = torch.arange(self.K + 1, device=i.device, dtype=torch.int64) * self.uniform_seg_len
        else:
            self.flat_seg = kernel_offset_segments(k, self.K)
        self.has_hybrid = False

    @classmethod
    def from_flat(cls, flat_i, flat_j, flat_seg, n_out, n_in, num_kernel_offsets,
                  exact_cover_out=False, exact_cover_in=False, uniform_seg_len=-1):
        self = cls.__new__(cls)
        self.flat_i, self.flat_j, self.flat_seg = flat_i, flat_j, flat_seg
        self.N, self.N_in = _maybe_int(n_out), _maybe_int(n_in)
        self.K = int(num_kernel_offsets)
        self.T = _maybe_int(flat_i.numel())
        self.exact_cover_out, self.exact_cover_in = bool(exact_cover_out), bool(exact_cover_in)
        self.uniform_seg_len = int(uniform_seg_len) if uniform_seg_len >= 0 else None
        self.has_hybrid = False
        return self


def _w4(weight):
    return weight if weight.dim() == 4 else weight.unsqueeze(1)


def _match(weight, feat):
    if weight.dtype != feat.dtype:
        promoted = torch.promote_types(weight.dtype, feat.dtype)
        weight, feat = weight.to(promoted), feat.to(promoted)
    return weight.contiguous(), feat.contiguous()


def tig_forward(weight, feat, index, mode="auto", input_precision=None, flat_cfg=None, l0_cfg=None):
    """``out[i] += feat[j] @ W[k]``; feat (N_in, G*C) -> (N, G*M) in feat.dtype."""
    w = _w4(weight)
    assert w.shape[0] == index.K and feat.size(1) == w.shape[1] * w.shape[2]
    assert feat.size(0) == index.N_in, f"feat rows {feat.size(0)} != index.N_in {index.N_in}"
    out_dtype = feat.dtype
    w, feat = _match(w, feat)
    engine = current_engine()
    if index.exact_cover_out and index.T == index.N:
        engine |= _cabi.ENGINE_FLAG_FAN_IN_ONE    # every output row has one triplet: rows are stored, not reduced
    out = mvmr_op(w, feat, index.flat_j, index.flat_i, index.flat_seg, None, index.N, False, engine)
    return out.to(out_dtype)


def tig_grad_input(weight, grad_out, index, input_precision=None, flat_cfg=None):
    """``grad_feat[j] += grad_out[i] @ W[k]^T`` -- same kernel, roles swapped."""
    w = _w4(weight)
    assert grad_out.size(0) == index.N, f"grad_out rows {grad_out.size(0)} != index.N {index.N}"
    out_dtype = grad_out.dtype
    w, grad_out = _match(w, grad_out)
    if index.N == index.N_in and _cabi.is_symmetric(index.flat_i, index.flat_j):
        # a self-search rulebook holds (j, i, K - 1 - k) with every (i, j, k): the input gradient is
        # the forward schedule over the same rulebook (and the same plan) with the taps reversed
        out = mvmr_op(w.flip(0), grad_out, index.flat_j, index.flat_i, index.flat_seg, None, index.N_in, True,
                      current_engine())
        return out.to(out_dtype)
    engine = current_engine()
    if index.exact_cover_in and index.T == index.N_in:
        engine |= _cabi.ENGINE_FLAG_FAN_IN_ONE    # every input row has one triplet: its gradient row is stored
    out = mvmr_op(w, grad_out, index.flat_i, index.flat_j, index.flat_seg, None, index.N_in, True, engine)
    return out.to(out_dtype)


def tig_grad_weight(feat, grad_out, index, weight_shape, input_precision=None, wgrad_cfg=None):
    """``grad_W[k] += feat[j]^T (outer) grad_out[i]``; returned in feat.dtype."""
    G = weight_shape[1] if len(weight_shape) == 4 else 1
    out_dtype = feat.dtype
    feat, grad_out = _match(feat, grad_out)
    gw = vvor_op(feat.view(feat.shape[0], G, -1), index.flat_j, grad_out.view(grad_out.shape[0], G, -1),
                 index.flat_i, index.flat_seg, None, index.K, current_engine())
    return gw.to(out_dtype).view(tuple(weight_shape))


@torch.library.custom_op("pointelligence_b200::tig_mvmr", mutates_args=())
def _tig_mvmr_op(weight: Tensor, feat: Tensor, flat_i: Tensor, flat_j: Tensor, flat_seg: Tensor,
                 n_out: int, n_in: int, num_kernel_offsets: int, exact_cover_out: bool,
                 exact_cover_in: bool, uniform_seg_len: int, input_precision: str) -> Tensor:
    index = TigIndex.from_flat(flat_i, flat_j, flat_seg, n_out, n_in, num_kernel_offsets,
                               exact_cover_out, exact_cover_in, uniform_seg_len)
    return tig_forward(weight, feat, index)


@_tig_mvmr_op.register_fake
def _(weight, feat, flat_i, flat_j, flat_seg, n_out, n_in, num_kernel_offsets, exact_cover_out,
      exact_cover_in, uniform_seg_len, input_precision):
    G = weight.shape[1] if weight.dim() == 4 else 1
    return feat.new_empty((n_out, G * weight.shape[-1]))


def _tig_setup(ctx, inputs, output):
    (weight, feat, flat_i, flat_j, flat_seg, n_out, n_in, K, eco, eci, usl, prec) = inputs
    ctx.save_for_backward(weight, feat, flat_i, flat_j, flat_seg)
    ctx.meta = (n_out, n_in, K, eco, eci, usl)


def _tig_backward(ctx, grad_out):
    weight, feat, flat_i, flat_j, flat_seg = ctx.saved_tensors
    index = TigIndex.from_flat(flat_i, flat_j, flat_seg, *ctx.meta)
    gw = gf = None
    if ctx.needs_input_grad[0]:
        gw = tig_grad_weight(feat, grad_out, index, weight.shape).to(weight.dtype)
    if ctx.needs_input_grad[1]:
        gf = tig_grad_input(weight, grad_out, index).to(feat.dtype)
    return (gw, gf) + (None,) * 10


_tig_mvmr_op.register_autograd(_tig_backward, setup_context=_tig_setup)


def tig_mvmr(weight, feat, index, mode="auto", input_precision: Optional[str] = None):
    """Differentiable tap-sorted convolution: one autograd node, three kernel
    families (forward MVMR, transposed MVMR, VVOR)."""
    if input_precision is None:
        input_precision = resolve_input_precision(feat.dtype)
    return _tig_mvmr_op(weight, feat, index.flat_i, index.flat_j, index.flat_seg, index.N, index.N_in,
                        index.K, index.exact_cover_out, index.exact_cover_in,
                        index.uniform_seg_len if index.uniform_seg_len is not None else -1,
                        input_precision)
