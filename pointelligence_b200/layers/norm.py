"""Normalisation layers for ragged batches (samples of different length stored
back to back).

Mirror of the reference's ``layers/norm.py:12-172``: ``RaggedNorm`` with its
four wrappers, the same constructor arguments, the same fp32 arithmetic with a
cast back to the input type, the same two-pass statistics (mean, then variance
of the centred values).  The per-sample reductions run through the library's
segment reduction (the reference defaults to ``torch.segment_reduce`` and lets
a caller plug ``large_segment_reduce`` in as ``reduce_fn``, :22-57; here the
library kernel is the default and ``reduce_fn`` still overrides it).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..sparse_engines.segment_reduce import large_segment_reduce

__all__ = ["RaggedNorm", "RaggedBatchNorm", "RaggedInstanceNorm", "RaggedLayerNorm", "RaggedGroupNorm"]


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

    def _reduce(self, x, reduce_op, lengths):
        fn = self.reduce_fn if self.reduce_fn is not None else large_segment_reduce
        return fn(x, reduce=reduce_op, lengths=lengths)

    def forward(self, x, lengths=None):
        input_dtype = x.dtype
        if self.norm_type == "batch":
            return self.bn(x.float()).to(input_dtype)
        if lengths is None:
            raise ValueError(f"lengths argument is required for {self.norm_type} norm")
        x = x.float()
        if self.norm_type == "instance":
            x_norm = self._instance_norm(x, lengths)
        elif self.norm_type == "group":
            x_norm = self._group_norm(x, lengths)
        elif self.norm_type == "layer":
            x_norm = self._layer_norm(x, lengths)
        else:
            raise ValueError(f"Unknown norm_type: {self.norm_type}")
        if self.affine:
            x_norm = x_norm * self.weight.float() + self.bias.float()
        return x_norm.to(input_dtype)

    def _expand(self, per_sample, lengths):
        return torch.repeat_interleave(per_sample, lengths, dim=0)

    def _instance_norm(self, x, lengths):
        centred = x - self._expand(self._reduce(x, "mean", lengths), lengths)
        var = self._reduce(centred.pow(2), "mean", lengths)
        return centred / self._expand((var + self.eps).sqrt(), lengths)

    def _group_norm(self, x, lengths):
        per_group = self.num_features // self.num_groups
        xg = x.view(x.size(0), self.num_groups, per_group)
        mean = self._reduce(xg.mean(dim=2), "mean", lengths)
        centred = xg - self._expand(mean, lengths).unsqueeze(2)
        var = self._reduce(centred.pow(2).mean(dim=2), "mean", lengths)
        std = self._expand((var + self.eps).sqrt(), lengths).unsqueeze(2)
        return (centred / std).view(x.size(0), self.num_features)

    def _layer_norm(self, x, lengths):
        mean = self._reduce(x.mean(dim=1, keepdim=True), "mean", lengths)
        centred = x - self._expand(mean, lengths)
        var = self._reduce(centred.pow(2).mean(dim=1, keepdim=True), "mean", lengths)
        return centred / self._expand((var + self.eps).sqrt(), lengths)


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
