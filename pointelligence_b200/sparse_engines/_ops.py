"""The two differentiable device primitives every public operator is built on.

``mvmr_op``   out[scatter[t]] += feat[gather[t]] @ W[tap(t)]        (or W^T)
``vvor_op``   out[o[t], g, m, c] += a[a_idx[t], g, m] * b[b_idx[t], g, c]

Both are ``torch.library`` custom operators (shape-only fake kernels, so they
are opaque leaves for ``torch.compile``) whose backward passes are expressed
with each other -- the duality the reference wires up in
``sparse_engines/mvmr_triton.py:272-329`` and ``vvor_triton.py:239-294``.
The CUDA work happens in the C-ABI library; nothing here computes on the host.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import _cabi

_NS = "pointelligence_b200"


@torch.library.custom_op(f"{_NS}::mvmr", mutates_args=())
def mvmr_op(weight: Tensor, feat: Tensor, gather: Tensor, scatter: Tensor,
            seg_offs: Optional[Tensor], tap_idx: Optional[Tensor], n_out: int,
            transpose: bool, engine: int) -> Tensor:
    return _cabi.mvmr(weight, feat, gather, scatter, seg_offs, tap_idx, n_out, transpose, engine)


@mvmr_op.register_fake
def _(weight, feat, gather, scatter, seg_offs, tap_idx, n_out, transpose, engine):
    K, G, C, M = weight.shape
    return feat.new_empty((n_out, G * (C if transpose else M)))


@torch.library.custom_op(f"{_NS}::vvor", mutates_args=())
def vvor_op(a: Tensor, a_idx: Tensor, b: Tensor, b_idx: Tensor, seg_offs: Optional[Tensor],
            o_idx: Optional[Tensor], n_o: int, engine: int) -> Tensor:
    return _cabi.vvor(a, a_idx, b, b_idx, seg_offs, o_idx, n_o, engine)


@vvor_op.register_fake
def _(a, a_idx, b, b_idx, seg_offs, o_idx, n_o, engine):
    return a.new_empty((n_o, a.shape[1], a.shape[2], b.shape[2]))


def _mvmr_setup(ctx, inputs, output):
    weight, feat, gather, scatter, seg_offs, tap_idx, n_out, transpose, engine = inputs
    ctx.save_for_backward(weight, feat, gather, scatter, seg_offs, tap_idx)
    ctx.transpose, ctx.engine = transpose, engine & 0xff   # a fan-in-1 promise holds for this direction only


def _mvmr_backward(ctx, grad):
    weight, feat, gather, scatter, seg_offs, tap_idx = ctx.saved_tensors
    K, G, C, M = weight.shape
    grad = grad.contiguous()
    gw = gf = None
    if ctx.needs_input_grad[0]:
        f3 = feat.reshape(feat.shape[0], G, -1)
        g3 = grad.reshape(grad.shape[0], G, -1)
        if ctx.transpose:   # dW[k][c][m] += grad[s][c] * feat[g][m]
            gw = vvor_op(g3, scatter, f3, gather, seg_offs, tap_idx, K, ctx.engine)
        else:               # dW[k][c][m] += feat[g][c] * grad[s][m]
            gw = vvor_op(f3, gather, g3, scatter, seg_offs, tap_idx, K, ctx.engine)
    if ctx.needs_input_grad[1]:
        gf = mvmr_op(weight, grad, scatter, gather, seg_offs, tap_idx, feat.shape[0],
                     not ctx.transpose, ctx.engine)
    return gw, gf, None, None, None, None, None, None, None


mvmr_op.register_autograd(_mvmr_backward, setup_context=_mvmr_setup)


def _vvor_setup(ctx, inputs, output):
    a, a_idx, b, b_idx, seg_offs, o_idx, n_o, engine = inputs
    ctx.save_for_backward(a, a_idx, b, b_idx, seg_offs, o_idx)
    ctx.engine = engine


def _vvor_backward(ctx, grad):
    a, a_idx, b, b_idx, seg_offs, o_idx = ctx.saved_tensors
    grad = grad.contiguous()   # (n_o, G, Ma, Cb) acts as a weight bank
    ga = gb = None
    if ctx.needs_input_grad[0]:   # ga[ai] += b[bi] @ grad[o]^T
        ga = mvmr_op(grad, b.reshape(b.shape[0], -1), b_idx, a_idx, seg_offs, o_idx, a.shape[0],
                     True, ctx.engine).reshape(a.shape)
    if ctx.needs_input_grad[2]:   # gb[bi] += a[ai] @ grad[o]
        gb = mvmr_op(grad, a.reshape(a.shape[0], -1), a_idx, b_idx, seg_offs, o_idx, b.shape[0],
                     False, ctx.engine).reshape(b.shape)
    return ga, None, gb, None, None, None, None, None


vvor_op.register_autograd(_vvor_backward, setup_context=_vvor_setup)
