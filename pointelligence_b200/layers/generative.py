"""Generative point convolution: the output point set is invented, not inherited
(interface of ``layers/generative.py:49-460`` of the reference).

``GeneratedSites`` carries the invented points together with the rulebook that wires them to the
input; a ``CoordinateGenerator`` produces one from a ``MetaData``.  Two generators:

* ``KernelStampGenerator``: every input point stamps the K taps of a stencil on the grid refined
  by ``expansion``; the output set is the union of the stamped voxels (one point per voxel, at its
  centre).  Every stamp is a triplet, so every output point has a contributor by construction.
* ``SubdivisionGenerator``: every input voxel generates exactly its ``e**3`` children; nothing to
  deduplicate, the rulebook is closed-form and every output row has exactly one triplet.

The stamps are laid out tap-major from the start (tap ``k`` of all N points, then tap ``k + 1``),
so the rulebook leaves the builder grouped by tap with exactly N triplets per tap and needs neither
a sort nor a permutation of ``j`` / ``k``; only the voxel deduplication (a sort of N*K keys inside
``torch.unique``) touches the data.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Protocol, runtime_checkable

import torch
from torch import Tensor
from torch.nn.modules.utils import _triple

from ..internals.grid_indexing import reduce_indices_to_1d
from .contract import TripletContract
from .metadata import MetaData

__all__ = ["GeneratedSites", "CoordinateGenerator", "KernelStampGenerator", "SubdivisionGenerator",
           "build_generative_triplets"]

_INT32_MAX = 2 ** 31 - 1


@dataclass
class GeneratedSites:
    """Generated output points ``(M, 3)`` with their sample ids and sizes, the output resolution,
    and the rulebook: ``i`` in ``[0, M)``, ``j`` in ``[0, N)``, ``k`` in ``[0, K)``.  ``aux``: optional
    by-products of a learned generator.  ``uniform_seg_len``: every tap owns exactly this many
    triplets (tap-major stamps), else None.  ``exact_cover_out``: every output row has exactly one
    triplet (nothing was merged)."""
    points: Tensor
    sample_inds: Tensor
    sample_sizes: Tensor
    grid_size: float
    i: Tensor
    j: Tensor
    k: Tensor
    aux: Optional[dict] = None
    uniform_seg_len: Optional[int] = None
    exact_cover_out: bool = False

    @property
    def n_out(self) -> int:
        return self.points.shape[0]

    def validate(self) -> None:
        """Every output row needs at least one triplet, or the convolution is undefined there."""
        if self.n_out == 0:
            return
        hits = torch.bincount(self.i.long(), minlength=self.n_out)
        orphans = int((hits == 0).sum())
        if orphans:
            raise RuntimeError(f"GeneratedSites: {orphans} of {self.n_out} output point(s) have zero contributing "
                               "input neighbours — the generative conv is undefined for them. A CoordinateGenerator "
                               "must cover every output index in the rulebook `i`.")

    def to_contract(self) -> TripletContract:
        return TripletContract(k_sorted=True, exact_cover_out=self.exact_cover_out, exact_cover_in=False,
                               uniform_seg_len=self.uniform_seg_len)

    def to_metadata(self, parent: Optional[MetaData]) -> MetaData:
        return MetaData(points=self.points, sample_inds=self.sample_inds, sample_sizes=self.sample_sizes,
                        grid_size=self.grid_size, i=self.i, j=self.j, k=self.k, contract=self.to_contract(),
                        parent=parent, auto_build_triplets=False)


@runtime_checkable
class CoordinateGenerator(Protocol):
    """``kernel_taps`` must equal the tap count of the convolution weight."""
    kernel_taps: int

    def __call__(self, m: MetaData) -> GeneratedSites: ...


def _cube_stencil(kernel_size, device) -> Tensor:
    """(K, 3) integer offsets of the dense kernel cube, x most significant (the tap order of
    ``voxelize_3d``): tap (kx, ky, kz) has offset (kx - k0 // 2, ky - k1 // 2, kz - k2 // 2)."""
    axes = [torch.arange(s, device=device) - (s // 2) for s in kernel_size]
    return torch.cartesian_prod(*axes).to(torch.int64).reshape(-1, 3)


def _empty_sites(points, sample_sizes, grid_size, **flags) -> GeneratedSites:
    dev = points.device
    none = torch.empty(0, dtype=torch.int32, device=dev)
    return GeneratedSites(points=points.new_empty((0, 3)), sample_inds=torch.empty(0, dtype=torch.int64, device=dev),
                          sample_sizes=torch.zeros(sample_sizes.numel(), dtype=torch.int64, device=dev),
                          grid_size=grid_size, i=none, j=none.clone(), k=none.clone(), **flags)


def _index_dtype(*sizes):
    return torch.int32 if max(sizes) <= _INT32_MAX else torch.int64


@torch.compiler.disable
def build_generative_triplets(points, sample_inds, sample_sizes, grid_size, kernel_size=(3, 3, 3), expansion=2.0,
                              stencil: Optional[Tensor] = None, sort_by: str = "k") -> GeneratedSites:
    """Stamp-and-deduplicate rulebook (``layers/generative.py:186-341`` of the reference).

    Every input point is quantised once to the output grid (``grid_size / expansion``) and stamps
    the stencil by integer addition; the output points are the distinct stamped voxels of a sample,
    in ascending (sample, z, y, x) order, placed at the voxel centres; ``i`` is the voxel of every
    stamp.  ``sort_by="k"``: tap-major, N triplets per tap; ``sort_by="i"``: ascending output row.
    """
    if sort_by not in ("k", "i"):
        raise ValueError(f'sort_by must be "k" or "i", got "{sort_by}"')
    with torch.no_grad():
        dev, N = points.device, points.shape[0]
        stencil = _cube_stencil(_triple(kernel_size), dev) if stencil is None else stencil.to(device=dev)
        K = stencil.shape[0]
        fine = grid_size / expansion
        if N == 0:
            return _empty_sites(points, sample_sizes, fine)
        voxel = torch.div(points, fine, rounding_mode="floor").to(torch.int32)              # (N, 3)
        stamped = stencil.to(torch.int32).unsqueeze(1) + voxel.unsqueeze(0)                 # (K, N, 3) tap-major
        sample_col = sample_inds.to(torch.int32).view(1, N, 1).expand(K, N, 1)
        cells = torch.cat([stamped, sample_col], dim=2).reshape(K * N, 4).contiguous()
        keys, lo, stride, _ = reduce_indices_to_1d(cells)
        distinct, i = torch.unique(keys, sorted=True, return_inverse=True)
        n_out = distinct.numel()
        # the key is sum_d (cell_d - lo_d) * stride_d with mixed-radix strides: decode its digits
        lo, stride = lo.reshape(-1), stride.reshape(-1).to(torch.int64)
        extent = (cells.amax(0) - lo + 1).to(torch.int64)
        decoded = ((distinct.unsqueeze(1) // stride) % extent + lo).to(torch.int32)         # (n_out, 4)
        out_points = (decoded[:, :3].to(points.dtype) + 0.5) * fine
        out_sample = decoded[:, 3].long()
        j = torch.arange(N, device=dev).repeat(K)
        k = torch.arange(K, device=dev).repeat_interleave(N)
        if sort_by == "i":
            i, order = torch.sort(i)       # not stable, as in the reference: ties in i come in any order
            j, k = j[order], k[order]
        dt = _index_dtype(n_out, N)
    return GeneratedSites(points=out_points, sample_inds=out_sample,
                          sample_sizes=torch.bincount(out_sample, minlength=sample_sizes.numel()), grid_size=fine,
                          i=i.to(dt), j=j.to(dt), k=k.to(dt), uniform_seg_len=(N if sort_by == "k" else None),
                          exact_cover_out=(n_out == N * K))


class KernelStampGenerator:
    """Deterministic generator: stencil stamps on the refined grid, deduplicated per voxel.
    ``stencil``: optional (K, 3) integer offsets instead of the dense kernel cube."""

    def __init__(self, kernel_size, expansion: float = 2.0, stencil: Optional[Tensor] = None) -> None:
        if expansion < 1:
            raise ValueError(f"expansion must be >= 1, got {expansion}")
        self.kernel_size = _triple(kernel_size)
        self.expansion = float(expansion)
        self._stencil = stencil
        self.kernel_taps = math.prod(self.kernel_size) if stencil is None else int(stencil.shape[0])

    def __call__(self, m: MetaData) -> GeneratedSites:
        return build_generative_triplets(m.points, m.sample_inds, m.sample_sizes, m.grid_size, self.kernel_size,
                                         self.expansion, self._stencil, sort_by="k")


class SubdivisionGenerator:
    """Every input voxel generates its ``e**3`` children (child = ``e * voxel + delta``): a tiling
    of the fine grid, so output row ``k * N + j`` belongs to exactly one (input ``j``, tap ``k``) and the
    whole rulebook is arithmetic.  The input is quantised at the INPUT grid, where voxel-centred
    points sit mid-cell."""

    def __init__(self, expansion: int = 2) -> None:
        e = int(expansion)
        if e < 2 or e != expansion:
            raise ValueError(f"SubdivisionGenerator needs an integer expansion >= 2, got {expansion}")
        self.expansion = e
        self.kernel_taps = e ** 3

    def __call__(self, m: MetaData) -> GeneratedSites:
        with torch.no_grad():
            points, dev, N, e, K = m.points, m.points.device, m.points.shape[0], self.expansion, self.kernel_taps
            fine = m.grid_size / e
            if N == 0:
                return _empty_sites(points, m.sample_sizes, fine, uniform_seg_len=0, exact_cover_out=True)
            voxel = torch.div(points, m.grid_size, rounding_mode="floor").to(torch.int64)
            delta = torch.cartesian_prod(*([torch.arange(e, device=dev)] * 3)).reshape(K, 3)
            child = (voxel.unsqueeze(0) * e + delta.unsqueeze(1)).reshape(K * N, 3)          # tap-major
            out_sample = m.sample_inds.repeat(K)
            dt = _index_dtype(N * K)
            return GeneratedSites(points=(child.to(points.dtype) + 0.5) * fine, sample_inds=out_sample,
                                  sample_sizes=torch.bincount(out_sample, minlength=m.sample_sizes.numel()),
                                  grid_size=fine, i=torch.arange(N * K, device=dev, dtype=dt),
                                  j=torch.arange(N, device=dev, dtype=dt).repeat(K),
                                  k=torch.arange(K, device=dev, dtype=dt).repeat_interleave(N),
                                  uniform_seg_len=N, exact_cover_out=True)
