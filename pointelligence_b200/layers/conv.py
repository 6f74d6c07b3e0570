"""Point convolution layer (mirror of ``layers/conv.py``: ``GeneralConv``
:85-465, ``PointConv3d`` :468-510, ``conv_with_stride`` :513-546).

Parameters keep the reference layout ``(K, G, C_in/G, C_out/G)`` and
initialisation ``U(+-1/sqrt((C_out/G) * K))`` so checkpoints interchange; a
legacy ``(C_in, C_out/G, K)`` weight is converted on load.  The forward routes
tap-sorted triplets (the contract every builder here produces) to the
tap-sorted engine and anything else to the public per-triplet operator.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch
from torch import Tensor
from torch.nn import Module, init
from torch.nn.modules.utils import _triple
from torch.nn.parameter import Parameter

from ..sparse_engines._dispatch_override import current_mode, resolve_input_precision, warn_pt_fallback
from ..sparse_engines.ops import sparse_matrix_vector_multiplication_reduction
from ..sparse_engines.tig import TigIndex, tig_mvmr
from .contract import TripletContract
from .metadata import MetaData
from .triplets import (build_full_cover_strided_rulebook, handle_stride_and_build_triplets,
                       handle_stride_disjoint_and_build_triplets)


class GeneralConv(Module):
    __constants__ = ["groups", "in_channels", "out_channels", "kernel_size"]

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, groups: int, bias: bool,
                 device=None, dtype=None) -> None:
        super().__init__()
        if groups <= 0:
            raise ValueError("groups must be a positive integer")
        if in_channels % groups != 0:
            raise ValueError("in_channels must be divisible by groups")
        if out_channels % groups != 0:
            raise ValueError("out_channels must be divisible by groups")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.groups = kernel_size, groups
        kw = {"device": device, "dtype": dtype}
        self.weight = Parameter(torch.empty(
            (kernel_size, groups, in_channels // groups, out_channels // groups), **kw))
        if bias:
            self.bias = Parameter(torch.empty(out_channels, **kw))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        fan_in = (self.out_channels // self.groups) * self.kernel_size
        bound = 1.0 / math.sqrt(fan_in) if fan_in > 0 else 0.0
        init.uniform_(self.weight, -bound, bound)
        if self.bias is not None and fan_in != 0:
            init.uniform_(self.bias, -bound, bound)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        key = prefix + "weight"
        w = state_dict.get(key)
        legacy = (self.in_channels, self.out_channels // self.groups, self.kernel_size)
        if w is not None and tuple(w.shape) == legacy:
            state_dict[key] = (w.reshape(self.groups, self.in_channels // self.groups,
                                         self.out_channels // self.groups, self.kernel_size)
                               .permute(3, 0, 1, 2).contiguous())
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)

    def extra_repr(self):
        s = f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}"
        if self.groups != 1:
            s += f", groups={self.groups}"
        if self.bias is None:
            s += ", bias=False"
        return s

    def _conv_forward(self, input: Tensor, i: Tensor, j: Tensor, k: Tensor, n: int, weight: Tensor,
                      bias: Optional[Tensor], *, contract: Optional[TripletContract] = None,
                      seg_offs: Optional[Tensor] = None) -> Tensor:
        x3 = input.view(input.shape[0], self.groups, -1) if input.dim() == 2 else input
        x3 = x3.contiguous()
        if contract is None:
            contract = TripletContract.submanifold()
        mode = current_mode()
        if mode == "auto":
            use_sorted = contract.k_sorted
            if not use_sorted:
                warn_pt_fallback("PointConv3d", "triplets are not k-sorted (contract)",
                                 K=weight.shape[0], C=self.in_channels, M=self.out_channels, G=self.groups)
        else:
            use_sorted = mode != "force_pt" and contract.k_sorted
        if use_sorted:
            n_in, K = x3.shape[0], weight.shape[0]
            if seg_offs is not None:
                idx = TigIndex.from_flat(
                    i, j, seg_offs, n_out=n, n_in=n_in, num_kernel_offsets=K,
                    exact_cover_out=contract.exact_cover_out, exact_cover_in=contract.exact_cover_in,
                    uniform_seg_len=contract.uniform_seg_len if contract.uniform_seg_len is not None else -1)
            else:
                idx = TigIndex(i, j, k, n, K, build_hybrid=False, assume_sorted=True, n_in=n_in,
                               uniform_seg_len=contract.uniform_seg_len,
                               exact_cover_out=contract.exact_cover_out,
                               exact_cover_in=contract.exact_cover_in)
            cin = weight.shape[2]
            if self.groups == 1 and cin > 256 and cin % 32 == 0 and x3.dtype in (torch.float16, torch.bfloat16):
                # wider than the tensor-core engine's 256-channel contraction: split the input
                # channels into two halves (two tensor-core passes, partial outputs added in fp32)
                half = cin // 2
                flat = x3.view(n_in, -1)
                parts = [tig_mvmr(weight[:, :, lo:lo + half].contiguous(), flat[:, lo:lo + half].contiguous(), idx,
                                  input_precision=resolve_input_precision(x3.dtype)).float()
                         for lo in (0, half)]
                output = (parts[0] + parts[1]).to(x3.dtype)
            else:
                output = tig_mvmr(weight, x3.view(n_in, -1), idx,
                                  input_precision=resolve_input_precision(x3.dtype))
        else:
            output = sparse_matrix_vector_multiplication_reduction(weight, k, x3, j, i, n)
        output = output.reshape(-1, weight.shape[1] * weight.shape[3])
        if bias is not None:
            output = output + bias
        return output


class PointConv3d(GeneralConv):
    """Convolution on native points (PointCNN++): ``out[i] += x[j] @ W[k]``."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, groups: int = 1,
                 bias: bool = True, device=None, dtype=None) -> None:
        self.kernel_size_3 = _triple(kernel_size)
        super().__init__(in_channels, out_channels, math.prod(self.kernel_size_3), groups, bias,
                         device=device, dtype=dtype)

    def forward(self, input: Tensor, i: Tensor, j: Tensor, k: Tensor, n: int,
                contract: Optional[TripletContract] = None, seg_offs: Optional[Tensor] = None) -> Tensor:
        return self._conv_forward(input, i, j, k, n, self.weight, self.bias, contract=contract,
                                  seg_offs=seg_offs)


def conv_with_stride(conv_op: Callable, x: Tensor, m: MetaData, stride: float,
                     receptive_field_scaler=1.0, distance_type: str = "ball") -> Tuple[Tensor, MetaData]:
    """Strided convolution: down-sample ``m`` by ``stride``, build the triplets
    from the parent cloud to the down-sampled cloud, convolve."""
    m = handle_stride_and_build_triplets(m, stride, conv_op.kernel_size_3, receptive_field_scaler,
                                         distance_type=distance_type)
    x = conv_op(x, m.i, m.j, m.k, m.num_points(), contract=m.contract, seg_offs=m.seg_offs)
    return x, m


class GenerativePointConv3d(GeneralConv):
    """Convolution onto an invented, denser point set (``layers/conv.py:687-755`` of the reference):
    ``forward(input, m)`` returns the features of the generated points and their ``MetaData``
    (parent = ``m``).  The point set and its rulebook come from a ``CoordinateGenerator`` (default
    ``KernelStampGenerator(kernel_size, expansion)``; its tap count sizes the weight); ``sites`` lets
    sibling layers share one generated set."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size=3, expansion: float = 2.0, generator=None,
                 groups: int = 1, bias: bool = True, device=None, dtype=None) -> None:
        from .generative import KernelStampGenerator

        self.kernel_size_3 = _triple(kernel_size)
        self.expansion = expansion
        if generator is None:
            generator = KernelStampGenerator(self.kernel_size_3, expansion)
        super().__init__(in_channels, out_channels, generator.kernel_taps, groups, bias, device=device, dtype=dtype)
        self.generator = generator

    def forward(self, input: Tensor, m: MetaData, sites=None) -> Tuple[Tensor, MetaData]:
        if sites is None:
            sites = self.generator(m)
        sites.validate()
        x = self._conv_forward(input, sites.i, sites.j, sites.k, sites.n_out, self.weight, self.bias,
                               contract=sites.to_contract())
        return x, sites.to_metadata(parent=m)


def conv_with_stride_disjoint(conv_op: Callable, x: Tensor, m: MetaData, stride: float) -> Tuple[Tensor, MetaData]:
    """Strided convolution as a grid partition, the patchify operator (``layers/conv.py:636-700`` of
    the reference): every input point contributes to exactly one token, the cell centre of side
    ``stride * grid_size`` it lies in, through the weight of its sub-voxel slot (``K**3`` slots for
    ``conv_op``'s cubic kernel).  ``Upsample(straight_recover=True, recompute_k=False)`` on the
    returned geometry is the matching unpatchify."""
    m = handle_stride_disjoint_and_build_triplets(m, stride, conv_op.kernel_size_3)
    x = conv_op(x, m.i, m.j, m.k, m.num_points(), contract=m.contract, seg_offs=m.seg_offs)
    return x, m


def conv_with_stride_full_cover(conv_op: Callable, x: Tensor, m: MetaData, stride: float,
                                radius_margin: float = 1e-2, radius_backend: str = "auto") -> Tuple[Tensor, MetaData]:
    """Overlapping strided convolution with guaranteed input coverage (mirror of
    ``layers/conv.py:549-632``): output centres are observed input points chosen
    by ``build_full_cover_strided_rulebook``; the mirrored rulebook is cached on
    the parent for the matching up-sampling layer."""
    if stride <= 1:
        raise ValueError(f"conv_with_stride_full_cover requires stride > 1; got {stride}.")
    import math

    from ..sparse_engines._seg_offs import kernel_offset_segments

    with torch.no_grad():
        pm = m.parent
        if not (pm is not None and pm.points.shape == m.points.shape and pm.grid_size == m.grid_size
                and torch.equal(pm.points, m.points) and torch.equal(pm.sample_inds, m.sample_inds)):
            pm = MetaData(points=m.points, sample_inds=m.sample_inds, sample_sizes=m.sample_sizes,
                          grid_size=m.grid_size, parent=m.parent)
            m.parent = pm
        rb = build_full_cover_strided_rulebook(
            points=pm.points, sample_inds=pm.sample_inds, sample_sizes=pm.sample_sizes, stride=stride,
            input_grid_size=pm.grid_size, kernel_size=conv_op.kernel_size_3, radius_margin=radius_margin,
            radius_backend=radius_backend, return_num_neighbors=True)
        taps = math.prod(conv_op.kernel_size_3)
        m.points, m.sample_inds, m.sample_sizes = rb.points, rb.sample_inds, rb.sample_sizes
        m.grid_size = float(stride) * pm.grid_size
        m.downsample_indices = rb.center_source_indices
        m.i, m.j, m.k = rb.i, rb.j, rb.k
        m.seg_offs = kernel_offset_segments(m.k, taps)
        m.num_neighbors = rb.num_neighbors
        m.contract = TripletContract(k_sorted=True)
        pm.i_upsample, pm.j_upsample, pm.k_upsample = rb.i_upsample, rb.j_upsample, rb.k_upsample
        pm.seg_offs_upsample = kernel_offset_segments(rb.k_upsample, taps)
        pm.full_cover_point_to_initial_center = rb.point_to_initial_center
        pm.full_cover_initial_center_indices = rb.initial_center_source_indices
        pm.full_cover_additional_center_indices = rb.additional_center_source_indices
        pm.full_cover_coverage_per_input = rb.coverage_per_input
        pm.full_cover_telemetry = {
            "radius": rb.radius, "radius_scaler": rb.radius_scaler,
            "initial_center_count": int(rb.initial_center_source_indices.numel()),
            "additional_center_count": int(rb.additional_center_source_indices.numel()),
            "selector_round_count": rb.selector_round_count, "edge_count": int(rb.k.numel())}
    x = conv_op(x, m.i, m.j, m.k, m.num_points(), contract=m.contract, seg_offs=m.seg_offs)
    return x, m
