"""Reference-style import surface.

``install()`` makes the reference's own names resolve to this package, so that code written
against the reference runs unchanged:

    import pointelligence_b200.compat as compat; compat.install()
    from sparse_engines.ops import sparse_matrix_vector_multiplication_reduction
    from sparse_engines.tig import TigIndex, tig_mvmr
    from layers import PointConv3d, MetaData, conv_with_stride
    from internals.neighbors import radius_search

and registers the three convolution operators under the reference's dispatcher namespace
(``sparse_engines::sparse_matrix_vector_multiplication_reduction``,
``sparse_engines::sparse_vector_vector_outer_product_reduction`` and ``sparse_engines::tig_mvmr``
with the schemas of sparse_engines/mvmr_triton.py:145-152, vvor_triton.py:113-120 and
tig.py:1508-1515), each with its shape-only fake kernel and its autograd rule.

Nothing happens on import: the aliases would shadow a checkout of the reference that is on the
path as well, so they are opt-in, and ``install()`` refuses when packages of these names that are
not this library's are already loaded.
"""
from __future__ import annotations

import importlib
import pkgutil
import sys
from typing import Optional

import torch
from torch import Tensor

_PACKAGES = ("sparse_engines", "layers", "internals")
_installed = False


def _alias_package(name):
    ours = importlib.import_module(f"pointelligence_b200.{name}")
    for info in pkgutil.walk_packages(ours.__path__, prefix=f"pointelligence_b200.{name}."):
        importlib.import_module(info.name)           # load every submodule once, under its real name
    prefix = f"pointelligence_b200.{name}"
    for full, module in list(sys.modules.items()):
        if full == prefix or full.startswith(prefix + "."):
            sys.modules[name + full[len(prefix):]] = module


def _register_reference_ops():
    from ..sparse_engines import mvmr as _mvmr, tig as _tig, vvor as _vvor

    try:
        torch.ops.sparse_engines.tig_mvmr      # already there (a second install, or the reference itself)
        return
    except (AttributeError, RuntimeError):
        pass

    @torch.library.custom_op("sparse_engines::tig_mvmr", mutates_args=())
    def tig_mvmr(weight: Tensor, feat: Tensor, flat_i: Tensor, flat_j: Tensor, flat_seg: Tensor, n_out: int,
                 n_in: int, num_kernel_offsets: int, exact_cover_out: bool, exact_cover_in: bool,
                 uniform_seg_len: int, input_precision: str) -> Tensor:
        index = _tig.TigIndex.from_flat(flat_i, flat_j, flat_seg, n_out, n_in, num_kernel_offsets, exact_cover_out,
                                        exact_cover_in, uniform_seg_len)
        return _tig.tig_forward(weight, feat, index)

    @tig_mvmr.register_fake
    def _(weight, feat, flat_i, flat_j, flat_seg, n_out, n_in, num_kernel_offsets, exact_cover_out, exact_cover_in,
          uniform_seg_len, input_precision):
        groups = weight.shape[1] if weight.dim() == 4 else 1
        return feat.new_empty((n_out, groups * weight.shape[-1]))

    tig_mvmr.register_autograd(_tig._tig_backward, setup_context=_tig._tig_setup)

    @torch.library.custom_op("sparse_engines::sparse_matrix_vector_multiplication_reduction", mutates_args=())
    def mvmr(a: Tensor, a_idx: Tensor, b: Tensor, b_idx: Tensor, o_idx: Tensor, n_o: int,
             seg_offs: Optional[Tensor] = None) -> Tensor:
        return _mvmr.sparse_matrix_vector_multiplication_reduction(a, a_idx, b, b_idx, o_idx, n_o, seg_offs)

    @mvmr.register_fake
    def _(a, a_idx, b, b_idx, o_idx, n_o, seg_offs=None):
        return a.new_empty((n_o, a.shape[1], a.shape[3]), dtype=torch.promote_types(a.dtype, b.dtype))

    def mvmr_setup(ctx, inputs, output):
        a, a_idx, b, b_idx, o_idx, n_o, seg_offs = inputs
        ctx.save_for_backward(a, a_idx, b, b_idx, o_idx)
        ctx.seg_offs = seg_offs

    def mvmr_backward(ctx, grad):
        # the duality of sparse_engines/mvmr_triton.py:272-329: the weight gradient is a VVOR, the
        # input gradient an MVMR with the weight used transposed
        a, a_idx, b, b_idx, o_idx = ctx.saved_tensors
        ga = gb = None
        if ctx.needs_input_grad[0]:
            ga = _vvor.sparse_vector_vector_outer_product_reduction(b, b_idx, grad, o_idx, a_idx, a.shape[0],
                                                                    ctx.seg_offs).to(a.dtype)
        if ctx.needs_input_grad[2]:
            gb = _mvmr.sparse_matrix_vector_multiplication_reduction(a.transpose(2, 3).contiguous(), a_idx, grad, o_idx,
                                                                     b_idx, b.shape[0], ctx.seg_offs).to(b.dtype)
        return ga, None, gb, None, None, None, None

    mvmr.register_autograd(mvmr_backward, setup_context=mvmr_setup)

    @torch.library.custom_op("sparse_engines::sparse_vector_vector_outer_product_reduction", mutates_args=())
    def vvor(a: Tensor, a_idx: Tensor, b: Tensor, b_idx: Tensor, o_idx: Tensor, n_o: int,
             seg_offs: Optional[Tensor] = None) -> Tensor:
        return _vvor.sparse_vector_vector_outer_product_reduction(a, a_idx, b, b_idx, o_idx, n_o, seg_offs)

    @vvor.register_fake
    def _(a, a_idx, b, b_idx, o_idx, n_o, seg_offs=None):
        return a.new_empty((n_o, a.shape[1], a.shape[2], b.shape[2]), dtype=torch.promote_types(a.dtype, b.dtype))

    def vvor_setup(ctx, inputs, output):
        a, a_idx, b, b_idx, o_idx, n_o, seg_offs = inputs
        ctx.save_for_backward(a, a_idx, b, b_idx, o_idx)
        ctx.seg_offs = seg_offs

    def vvor_backward(ctx, grad):
        # sparse_engines/vvor_triton.py:239-294: both input gradients are MVMRs over the output as weight bank
        a, a_idx, b, b_idx, o_idx = ctx.saved_tensors
        ga = gb = None
        if ctx.needs_input_grad[0]:
            ga = _mvmr.sparse_matrix_vector_multiplication_reduction(grad.transpose(2, 3).contiguous(), o_idx, b, b_idx,
                                                                     a_idx, a.shape[0], ctx.seg_offs).to(a.dtype)
        if ctx.needs_input_grad[2]:
            gb = _mvmr.sparse_matrix_vector_multiplication_reduction(grad.contiguous(), o_idx, a, a_idx, b_idx,
                                                                     b.shape[0], ctx.seg_offs).to(b.dtype)
        return ga, None, gb, None, None, None, None

    vvor.register_autograd(vvor_backward, setup_context=vvor_setup)


def install():
    """Alias ``sparse_engines``, ``layers`` and ``internals`` (with all their submodules) to this
    package and register the ``sparse_engines::`` operators.  Idempotent."""
    global _installed
    if _installed:
        return
    for name in _PACKAGES:
        loaded = sys.modules.get(name)
        if loaded is not None and not getattr(loaded, "__name__", "").startswith("pointelligence_b200."):
            raise RuntimeError(f"a package named '{name}' that is not this library's is already imported "
                               "(the reference itself?): the aliases would shadow it")
    for name in _PACKAGES:
        _alias_package(name)
    _register_reference_ops()
    _installed = True
