"""Normalisation layers for ragged batches (samples of different length stored
back to back).

Stand in for the reference's ``layers/norm.py:12-172``: ``RaggedNorm`` and its four wrappers
with the same constructor arguments and the same arithmetic (fp32, mean first, then the variance
of the centred values, cast back to the input type).  On CUDA the three per-sample norms run as
the library's fused kernels (layer norm with its residual / ReLU tail, group and instance norm as
one kernel family over (sample, channel group) statistics).  With a ``reduce_fn`` plugged in, or on
the CPU, they share one code path that treats layer / group / instance as the same computation
over (groups, width) views, with the per-sample sums done by the library's segment reduction
(the reference defaults to ``torch.segment_reduce`` and lets a caller plug ``large_segment_reduce``
in as ``reduce_fn``, :22-57; ``reduce_fn`` still overrides the library kernel here, and is called
with ``reduce="sum"``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import _cabi
from ..sparse_engines.segment_reduce import large_segment_reduce

__all__ = ["RaggedNorm", "RaggedBatchNorm", "RaggedInstanceNorm", "RaggedLayerNorm", "RaggedGroupNorm",
           "fused_layer_norm", "fused_group_norm"]


class _FusedLayerNorm(torch.autograd.Function):
    """One autograd node over the library's fused kernels (``pcx_ragged_layer_norm`` and its
    backward): statistics, affine, optional residual add and ReLU."""

    @staticmethod
    def forward(ctx, x, lengths, weight, bias, residual, eps, relu):
        y, mean, rstd = _cabi.ragged_layer_norm(x, lengths, weight, bias, residual, eps, relu)
        ctx.save_for_backward(x, y, lengths, weight, mean, rstd)
        ctx.relu, ctx.has_residual = bool(relu), residual is not None
        ctx.param_dtypes = (None if weight is None else weight.dtype, None if bias is None else bias.dtype)
        ctx.residual_dtype = None if residual is None else residual.dtype
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, y, lengths, weight, mean, rstd = ctx.saved_tensors
        want_affine = weight is not None and (ctx.needs_input_grad[2] or ctx.needs_input_grad[3])
        want_res = ctx.has_residual and ctx.needs_input_grad[4]
        gx, gw, gb, gres = _cabi.ragged_layer_norm_backward(grad_y, x, y, lengths, weight, mean, rstd, ctx.relu,
                                                            want_affine, want_res)
        if gw is not None:
            gw, gb = gw.to(ctx.param_dtypes[0]), gb.to(ctx.param_dtypes[1])
        if gres is not None:
            gres = gres.to(ctx.residual_dtype)
        return gx, None, gw, gb, gres, None, None


class _FusedGroupNorm(torch.autograd.Function):
    """Group / instance norm over the library's kernels (``pcx_ragged_group_norm`` and its backward)."""

    @staticmethod
    def forward(ctx, x, lengths, weight, bias, groups, eps):
        y, mean, rstd = _cabi.ragged_group_norm(x, lengths, weight, bias, groups, eps)
        ctx.save_for_backward(x, lengths, weight, mean, rstd)
        ctx.groups = int(groups)
        ctx.param_dtypes = (None if weight is None else weight.dtype, None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, lengths, weight, mean, rstd = ctx.saved_tensors
        want_affine = weight is not None and (ctx.needs_input_grad[2] or ctx.needs_input_grad[3])
        gx, gw, gb = _cabi.ragged_group_norm_backward(grad_y, x, lengths, weight, mean, rstd, ctx.groups, want_affine)
        if gw is not None:
            gw, gb = gw.to(ctx.param_dtypes[0]), gb.to(ctx.param_dtypes[1])
        return gx, None, gw, gb, None, None


def fused_group_norm(x, lengths, groups, weight=None, bias=None, eps=1e-5):
    """``RaggedGroupNorm`` (``groups == x.shape[1]``: ``RaggedInstanceNorm``) as two statistics passes and
    one normalising pass of the library (layers/norm.py:86-116 of the reference composes it from a dozen
    torch launches); CUDA tensors only."""
    return _FusedGroupNorm.apply(x, lengths, weight, bias, groups, eps)


def fused_layer_norm(x, lengths, weight=None, bias=None, eps=1e-5, residual=None, relu=False):
    """``relu?(RaggedLayerNorm(x) (+ residual))`` in one pass over the data (CUDA tensors only).

    Same arithmetic as ``RaggedLayerNorm`` (layers/norm.py:59-83,118-130 of the reference) followed by
    the ``out += identity; relu(out)`` tail of its residual blocks (models/resnet.py:129-130)."""
    return _FusedLayerNorm.apply(x, lengths, weight, bias, residual, eps, relu)


class RaggedNorm(nn.Module):
    def __init__(self, num_features, norm_type="batch", num_groups=1, eps=1e-5, affine=True, reduce_fn=None):
        super().__init__()
        self.norm_type = norm_type.lower()
        self.num_features = num_features
        self.num_groups = num_groups
        self.eps = eps
        self.affine = affine
        self.reduce_fn = reduce_fn
        if self.norm_type == "batch":
            self.bn = nn.BatchNorm1d(num_features, eps=eps, affine=affine)
        elif self.affine:
            self.weight = nn.Parameter(torch.ones(num_features))
            self.bias = nn.Parameter(torch.zeros(num_features))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def _segment_sum(self, x, lengths):
        fn = self.reduce_fn if self.reduce_fn is not None else large_segment_reduce
        return fn(x, reduce="sum", lengths=lengths)

    def _groups(self):
        """Statistics groups per sample: the three per-sample norms differ only in how the channels
        are pooled -- all of them (layer), ``num_groups`` blocks (group), or none (instance)."""
        if self.norm_type == "layer":
            return 1
        if self.norm_type == "group":
            return self.num_groups
        if self.norm_type == "instance":
            return self.num_features
        raise ValueError(f"Unknown norm_type: {self.norm_type}")

    def forward(self, x, lengths=None):
        input_dtype = x.dtype
        if self.norm_type == "batch":
            return self.bn(x.float()).to(input_dtype)
        groups = self._groups()
        if lengths is None:
            raise ValueError(f"lengths argument is required for {self.norm_type} norm")
        if self.reduce_fn is None and x.is_cuda:
            if self.norm_type == "layer":
                return fused_layer_norm(x, lengths, self.weight, self.bias, self.eps)
            if groups <= 4096 and self.num_features % groups == 0:
                return fused_group_norm(x, lengths, groups, self.weight, self.bias, self.eps)
        # fp32, two passes (mean, then variance of the centred values) as layers/norm.py:86-130 of
        # the reference; one code path for the three norms: rows are viewed as (groups, width),
        # every pass is a per-row sum over the width followed by one segment sum over the sample
        n, width = x.shape[0], self.num_features // groups
        rows = x.float().view(n, groups, width)
        sample = torch.repeat_interleave(torch.arange(lengths.numel(), device=x.device), lengths, output_size=n)
        count = (lengths.to(torch.float32) * width).clamp_min(1.0).unsqueeze(1)
        mean = self._segment_sum(rows.sum(dim=2), lengths) / count                     # (samples, groups)
        centred = rows - mean[sample].unsqueeze(2)
        var = self._segment_sum(centred.square().sum(dim=2), lengths) / count
        out = (centred * torch.rsqrt(var + self.eps)[sample].unsqueeze(2)).view(n, self.num_features)
        if self.affine:
            out = out * self.weight.float() + self.bias.float()
        return out.to(input_dtype)


class RaggedBatchNorm(RaggedNorm):
    def __init__(self, num_features, eps=1e-5, affine=True, reduce_fn=None):
        super().__init__(num_features, norm_type="batch", eps=eps, affine=affine, reduce_fn=reduce_fn)


class RaggedInstanceNorm(RaggedNorm):
    def __init__(self, num_features, eps=1e-5, affine=False, reduce_fn=None):
        super().__init__(num_features, norm_type="instance", eps=eps, affine=affine, reduce_fn=reduce_fn)


class RaggedLayerNorm(RaggedNorm):
    def __init__(self, num_features, eps=1e-5, affine=True, reduce_fn=None):
        super().__init__(num_features, norm_type="layer", eps=eps, affine=affine, reduce_fn=reduce_fn)


class RaggedGroupNorm(RaggedNorm):
    def __init__(self, num_groups, num_channels, eps=1e-5, affine=True, reduce_fn=None):
        if num_channels % num_groups != 0:
            raise ValueError("num_channels must be divisible by num_groups")
        super().__init__(num_channels, norm_type="group", num_groups=num_groups, eps=eps, affine=affine,
                         reduce_fn=reduce_fn)
