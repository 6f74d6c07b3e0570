"""Segment reductions over ragged batches.

Stand in for the reference's ``sparse_engines/large_segment_reduce_triton.py``
(``large_segment_reduce``, :180-188) and
``sparse_engines/indexed_segment_reduce_triton.py`` (``indexed_segment_reduce``,
:147-173): same call signatures, same results for empty segments, same
gradient rules (broadcast for sum / mean, value match for max / min).  Both are
``torch.library`` custom operators backed by the C-ABI library; accumulation is
fp32 for every input type and the result is rounded once.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _cabi

_NS = "pointelligence_b200"


def _op_code(reduce):
    if reduce not in _cabi.REDUCE_OPS:
        raise ValueError(f"Mode must be one of {list(_cabi.REDUCE_OPS.keys())}")
    return _cabi.REDUCE_OPS[reduce]


@torch.library.custom_op(f"{_NS}::large_segment_reduce", mutates_args=())
def _large_op(x: Tensor, lengths: Tensor, op: int) -> Tensor:
    return _cabi.segment_reduce(x, lengths, op)


@_large_op.register_fake
def _(x, lengths, op):
    return x.new_empty((lengths.shape[0], x.shape[1]))


@torch.library.custom_op(f"{_NS}::large_segment_reduce_backward", mutates_args=())
def _large_bwd_op(grad_out: Tensor, x: Tensor, out: Tensor, lengths: Tensor, op: int, n_rows: int) -> Tensor:
    return _cabi.segment_reduce_backward(grad_out, x, out, lengths, op, n_rows)


@_large_bwd_op.register_fake
def _(grad_out, x, out, lengths, op, n_rows):
    return grad_out.new_empty((n_rows, grad_out.shape[1]))


def _large_setup(ctx, inputs, output):
    x, lengths, op = inputs
    ctx.op, ctx.n_rows = op, x.shape[0]
    if op >= 2:
        ctx.save_for_backward(lengths, x, output)
    else:
        ctx.save_for_backward(lengths)


def _large_backward(ctx, grad_out):
    if ctx.op >= 2:
        lengths, x, out = ctx.saved_tensors
    else:
        (lengths,) = ctx.saved_tensors
        x = out = grad_out   # not read for sum / mean
    return _large_bwd_op(grad_out.contiguous(), x, out, lengths, ctx.op, ctx.n_rows), None, None


_large_op.register_autograd(_large_backward, setup_context=_large_setup)


def large_segment_reduce(x, reduce, *, lengths):
    """``out[s] = reduce`` of the ``lengths[s]`` consecutive rows of ``x`` (N, C) -> (S, C) in ``x.dtype``."""
    # contiguous here, not inside the operator: the tensor saved for the max / min gradient must be
    # the one the kernel read (a column slice or a transposed view has another memory layout)
    return _large_op(x.contiguous(), lengths, _op_code(reduce))


@torch.library.custom_op(f"{_NS}::indexed_segment_reduce", mutates_args=())
def _indexed_op(x: Tensor, indices: Tensor, lengths: Tensor, op: int) -> Tensor:
    return _cabi.indexed_segment_reduce(x, indices, lengths, op)


@_indexed_op.register_fake
def _(x, indices, lengths, op):
    return x.new_empty((lengths.shape[0], x.shape[1]))


@torch.library.custom_op(f"{_NS}::indexed_segment_reduce_backward", mutates_args=())
def _indexed_bwd_op(grad_y: Tensor, x: Tensor, y: Tensor, indices: Tensor, lengths: Tensor, op: int,
                    n_x: int) -> Tensor:
    return _cabi.indexed_segment_reduce_backward(grad_y, x, y, indices, lengths, op, n_x)


@_indexed_bwd_op.register_fake
def _(grad_y, x, y, indices, lengths, op, n_x):
    return grad_y.new_empty((n_x, grad_y.shape[1]))


def _indexed_setup(ctx, inputs, output):
    x, indices, lengths, op = inputs
    ctx.op, ctx.n_x = op, x.shape[0]
    if op >= 2:
        ctx.save_for_backward(indices, lengths, x, output)
    else:
        ctx.save_for_backward(indices, lengths)


def _indexed_backward(ctx, grad_y):
    if ctx.op >= 2:
        indices, lengths, x, y = ctx.saved_tensors
    else:
        indices, lengths = ctx.saved_tensors
        x = y = grad_y   # not read for sum / mean
    return _indexed_bwd_op(grad_y.contiguous(), x, y, indices, lengths, ctx.op, ctx.n_x), None, None, None


_indexed_op.register_autograd(_indexed_backward, setup_context=_indexed_setup)


def indexed_segment_reduce(x, reduce, indices, *, lengths):
    """``y[k] = reduce`` of ``x[indices[e]]`` over the ``lengths[k]`` consecutive entries of list k."""
    return _indexed_op(x.contiguous(), indices, lengths, _op_code(reduce))
