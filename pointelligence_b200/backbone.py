"""Segmentation backbone used by the training-step benchmark (configs 4 and 5).

A residual U-Net over native points wired like the reference's Pointcept overlay
(``overlays/Pointcept/add/pointcept/models/sparse_unet/unet_pointcnnpp.py:40-125``
for the block, ``:183-246`` for the stages, ``:339-419`` for the forward pass):
a 5x5x5 stem, four encoder stages of ``BasicBlock``s (stride 2 from the second
stage on), three ``Upsample`` stages with skip concatenation, a decoder stage at
full resolution and a 1x1x1 classifier.  Differences, all stated by the benchmark
configuration: the norm is ``RaggedLayerNorm`` (per-sample statistics, so ranks
need no collective for it), activations and convolution operands are bf16 with
fp32 master weights, every norm -> (+ identity) -> ReLU tail runs as one fused
kernel (``layers.norm.fused_layer_norm``), the shortcut projection (with its row gather at a
stride) is a one-tap MVMR of the library instead of a ``Linear``, and every decoder stage rebuilds the submanifold triplets of its own
cloud instead of inheriting the up-sampling layer's.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import _cabi
from .internals.triplet_cache import triplet_cache_scope
from .layers import MetaData, PointConv3d, RaggedLayerNorm, Upsample
from .layers.norm import fused_layer_norm
from .layers.triplets import (build_triplets_segmented, handle_stride_and_build_triplets,
                              radius_scaler_for_kernel_size)

RFS = 2.5   # receptive_field_scaler of every convolution, as in the reference's model


def _pad_to(n, multiple=16):
    return (n + multiple - 1) // multiple * multiple


class Bf16PointConv3d(PointConv3d):
    """``PointConv3d`` with bf16 operands: the fp32 master weight is cast on the fly and the
    input is taken as bf16.  Channel counts that are not multiples of 16 (the 3-channel input,
    the class logits) are zero-padded so that they take the tensor-core engine as well; the
    padding carries no gradient."""

    def forward(self, input, i, j, k, n, contract=None, seg_offs=None):
        w = self.weight.to(torch.bfloat16)
        K, G, C, M = w.shape
        Cp, Mp = _pad_to(C), _pad_to(M)
        x = input.to(torch.bfloat16)
        if (Cp, Mp) != (C, M):
            w = F.pad(w, (0, Mp - M, 0, Cp - C))
            x = F.pad(x, (0, Cp - C))
        out = self._conv_forward(x, i, j, k, n, w, None, contract=contract, seg_offs=seg_offs)
        if Mp != M:
            out = out.view(n, -1)[:, :M]
        if self.bias is not None:
            out = out + self.bias.to(out.dtype)
        return out


def project_rows(x: Tensor, rows, weight: Tensor) -> Tensor:
    """``x[rows] @ weight.T`` (``rows`` None: every row) as one MVMR with a single tap: the gather
    of the strided shortcut and its projection run in the library's own tensor-core kernels, and
    so do both gradients (VVOR for the weight, transposed MVMR for the input).  The reference
    gathers and calls a ``Linear`` (models/resnet.py:119-130)."""
    from .sparse_engines._dispatch_override import current_engine
    from .sparse_engines._ops import mvmr_op

    n_out = x.shape[0] if rows is None else rows.shape[0]
    gather = (torch.arange(n_out, device=x.device, dtype=torch.int32) if rows is None
              else rows.to(torch.int32))
    scatter = torch.arange(n_out, device=x.device, dtype=torch.int32)
    seg = torch.tensor([0, n_out], device=x.device, dtype=torch.int64)
    w = weight.to(x.dtype).t().contiguous().view(1, 1, weight.shape[1], weight.shape[0])
    return mvmr_op(w, x.contiguous(), gather, scatter, seg, None, n_out, False, current_engine())


def _norm_act(norm: RaggedLayerNorm, x: Tensor, lengths: Tensor, residual=None, relu=True) -> Tensor:
    return fused_layer_norm(x, lengths, norm.weight, norm.bias, norm.eps, residual=residual, relu=relu)


class BasicBlock(nn.Module):
    def __init__(self, inplanes: int, planes: int, stride: float = 1.0):
        super().__init__()
        self.conv1 = Bf16PointConv3d(inplanes, planes, kernel_size=3, bias=False)
        self.bn1 = RaggedLayerNorm(planes)
        self.conv2 = Bf16PointConv3d(planes, planes, kernel_size=3, bias=False)
        self.bn2 = RaggedLayerNorm(planes)
        self.stride = stride
        self.shortcut = None
        if inplanes != planes:
            self.shortcut = nn.Linear(inplanes, planes, bias=False)
            self.shortcut_norm = RaggedLayerNorm(planes)

    def forward(self, x: Tensor, m: MetaData) -> Tuple[Tensor, MetaData]:
        identity = x
        x, m = self._strided(x, m)
        x = _norm_act(self.bn1, x, m.sample_sizes)
        if self.stride != 1.0:
            scaler = radius_scaler_for_kernel_size(kernel_size=3, receptive_field_scaler=RFS)
            m.i, m.j, m.k, m.seg_offs, _ = build_triplets_segmented(
                points=m.points, sample_inds=m.sample_inds, sample_sizes=m.sample_sizes,
                neighbor_radius=m.grid_size * scaler, kernel_size=3, radius_scaler=scaler)
        x = self.conv2(x, m.i, m.j, m.k, m.num_points(), seg_offs=m.seg_offs)
        rows = m.downsample_indices if self.stride != 1.0 else None
        if self.shortcut is not None:
            identity = project_rows(identity, rows, self.shortcut.weight)
            identity = _norm_act(self.shortcut_norm, identity, m.sample_sizes, relu=False)
        elif rows is not None:
            identity = identity[rows]
        return _norm_act(self.bn2, x, m.sample_sizes, residual=identity), m

    def _strided(self, x, m):
        m = handle_stride_and_build_triplets(m, self.stride, self.conv1.kernel_size_3, RFS)
        x = self.conv1(x, m.i, m.j, m.k, m.num_points(), contract=m.contract, seg_offs=m.seg_offs)
        return x, m


class UpsampleBf16(Upsample):
    """``Upsample`` whose convolution takes bf16 operands."""

    def __init__(self, in_channels, out_channels, **kwargs):
        super().__init__(in_channels, out_channels, **kwargs)
        self.conv = Bf16PointConv3d(in_channels, out_channels, kernel_size=kwargs.get("kernel_size", 3),
                                    bias=kwargs.get("bias", True))


class ResUNet(nn.Module):
    def __init__(self, in_channels=3, num_classes=20, base_channels=32, channels: Sequence[int] = (32, 64, 128, 256),
                 tr_channels: Sequence[int] = (96, 96, 128, 256), layers: Sequence[int] = (2,) * 8):
        super().__init__()
        C, TR, L = list(channels), list(tr_channels), list(layers)
        self.conv1 = Bf16PointConv3d(in_channels, base_channels, kernel_size=5, bias=False)
        self.norm1 = RaggedLayerNorm(base_channels)

        def stage(cin, cout, n, stride):
            return nn.ModuleList([BasicBlock(cin if b == 0 else cout, cout, stride if b == 0 else 1.0)
                                  for b in range(n)])

        self.block1 = stage(base_channels, C[0], L[0], 1.0)
        self.enc_block1 = stage(C[0], C[1], L[1], 2.0)
        self.enc_block2 = stage(C[1], C[2], L[2], 2.0)
        self.enc_block3 = stage(C[2], C[3], L[3], 2.0)
        self.upsample4 = UpsampleBf16(C[3], TR[3], kernel_size=3, bias=False, receptive_field_scaler=RFS)
        self.norm4_tr = RaggedLayerNorm(TR[3])
        self.block4_tr = stage(TR[3], TR[3], L[4], 1.0)
        self.upsample3 = UpsampleBf16(C[2] + TR[3], TR[2], kernel_size=3, bias=False, receptive_field_scaler=RFS)
        self.norm3_tr = RaggedLayerNorm(TR[2])
        self.block3_tr = stage(TR[2], TR[2], L[5], 1.0)
        self.upsample2 = UpsampleBf16(C[1] + TR[2], TR[1], kernel_size=3, bias=False, receptive_field_scaler=RFS)
        self.norm2_tr = RaggedLayerNorm(TR[1])
        self.block2_tr = stage(TR[1], TR[1], L[6], 1.0)
        self.block1_tr = stage(C[0] + TR[1], TR[0], L[7], 1.0)
        self.final_conv = Bf16PointConv3d(TR[0], num_classes, kernel_size=1, bias=True)
        for mod in self.modules():
            if isinstance(mod, (nn.Linear, PointConv3d)):
                nn.init.trunc_normal_(mod.weight, std=0.02)

    def forward(self, feat: Tensor, points: Tensor, sample_inds: Tensor, sample_sizes: Tensor,
                grid_size: float) -> Tensor:
        # one rulebook per (cloud, radius, kernel size) and forward pass: the decoder levels
        # find the encoder levels' submanifold triplets in the cache
        # and the geometry of a level is built on a stream of its own while the feature kernels of
        # the level before it are still running (every point cloud of the network derives from
        # the input cloud through the library's geometry calls alone)
        with triplet_cache_scope(), _cabi.geometry_overlap(points.device):
            return self._forward(feat, points, sample_inds, sample_sizes, grid_size)

    def _forward(self, feat, points, sample_inds, sample_sizes, grid_size):
        m = MetaData(points=points, sample_inds=sample_inds, sample_sizes=sample_sizes, grid_size=grid_size)
        m = handle_stride_and_build_triplets(m, 1.0, self.conv1.kernel_size_3, RFS)
        x = self.conv1(feat, m.i, m.j, m.k, m.num_points(), contract=m.contract, seg_offs=m.seg_offs)
        m.dirty_triplets()
        x = _norm_act(self.norm1, x, m.sample_sizes)
        for blk in self.block1:
            x, m = blk(x, m)
        skips: List[Tensor] = [x]
        for stage in (self.enc_block1, self.enc_block2, self.enc_block3):
            for blk in stage:
                x, m = blk(x, m)
            skips.append(x)
        # every decoder stage drops the up-sampling triplets it arrives with, so that its blocks
        # convolve over the submanifold neighbourhoods of their own cloud
        x, m = self.upsample4(skips[-1], m)
        m.dirty_triplets()
        x = _norm_act(self.norm4_tr, x, m.sample_sizes)
        for blk in self.block4_tr:
            x, m = blk(x, m)
        x, m = self.upsample3(torch.cat([skips[-2], x], dim=1), m)
        m.dirty_triplets()
        x = _norm_act(self.norm3_tr, x, m.sample_sizes)
        for blk in self.block3_tr:
            x, m = blk(x, m)
        x, m = self.upsample2(torch.cat([skips[-3], x], dim=1), m)
        m.dirty_triplets()
        x = _norm_act(self.norm2_tr, x, m.sample_sizes)
        for blk in self.block2_tr:
            x, m = blk(x, m)
        x = torch.cat([skips[0], x], dim=1)
        m.dirty_triplets()
        for blk in self.block1_tr:
            x, m = blk(x, m)
        scaler = radius_scaler_for_kernel_size(kernel_size=1, receptive_field_scaler=RFS)
        i, j, k, seg, _ = build_triplets_segmented(points=m.points, sample_inds=m.sample_inds,
                                                   sample_sizes=m.sample_sizes, neighbor_radius=m.grid_size * scaler,
                                                   kernel_size=1, radius_scaler=scaler)
        return self.final_conv(x, i, j, k, m.num_points(), seg_offs=seg)
