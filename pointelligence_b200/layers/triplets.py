"""Triplet (rulebook) construction (mirror of ``layers/triplets.py``).

``(i, j, k)``: input point ``j`` contributes to output point ``i`` through
kernel tap ``k``.  The convolution path uses ``build_triplets_segmented``
(:584-682): one sorted-grid radius search that emits the pairs already grouped
by tap, with the tap computed on the device exactly like ``voxelize_3d``
(:547-561).  ``build_triplets`` (:686-764) is the generic builder for custom
indexers and other sort orders.
"""
from __future__ import annotations

import math
from functools import partial
from typing import Callable, Optional

import torch
from torch.nn.modules.utils import _triple

from .. import _cabi
from ..internals.indexing import cumsum_exclusive, repeat_interleave_indices
from ..internals.neighbors import radius_search, radius_search_sorted_grid8_segments
from ..internals.triplet_cache import cache_get, cache_put, triplet_key
from ..sparse_engines._seg_offs import kernel_offset_segments
from .contract import TripletContract
from .downsample import downsample
from .metadata import MetaData

_NO_NEIGHBOR_MSG = (
    "Neighborhood search failed for some points, consider increase the neighbor_radius. "
    "It is likely that this happens in an *upsample* phase, where the query_points are not "
    "a subset of the points.")


def full_cover_radius_scaler(stride, radius_margin=1e-2):
    if stride <= 0:
        raise ValueError(f"stride must be positive; got {stride}")
    if radius_margin < 0:
        raise ValueError(f"radius_margin must be non-negative; got {radius_margin}")
    return (math.sqrt(3.0) / 2.0) * float(stride) * (1.0 + float(radius_margin))


def minimum_full_cover_kernel_size(radius_scaler):
    return 2 * int(math.ceil(float(radius_scaler))) + 1


def radius_scaler_for_kernel_size(kernel_size, receptive_field_scaler=1.0, distance_type="ball"):
    """``neighbor_radius = grid_size * radius_scaler``: the ball (or cube) whose
    volume is ``receptive_field_scaler`` times the kernel cube's."""
    kmax = max(_triple(kernel_size))
    if distance_type == "cube":
        return kmax * math.pow(receptive_field_scaler, 1 / 3) / 2.0
    volume = math.pow(kmax, 3) * receptive_field_scaler
    return math.pow(3 * volume / (4 * math.pi), 1 / 3)


def voxelize_3d(kernel_size, points, grid_size=None):
    """Tap of every offset: round-half-even of ``offset / grid_size``, shifted
    by ``K // 2``, clamped to the kernel, x most significant."""
    with torch.no_grad():
        ks = _triple(kernel_size)[0]
        cell = (points / grid_size).round().int()
        cell = torch.clamp(cell + (ks // 2), min=0, max=ks - 1)
        mult = torch.tensor([ks * ks, ks, 1], device=points.device, dtype=torch.int32)
        return torch.sum(cell * mult, dim=1)


def should_use_direct_segmented_triplets(kernel_size):
    s = _triple(kernel_size)
    return s[0] == s[1] == s[2] and int(s[0]) >= 1 and int(s[0]) % 2 == 1


def _resolve_queries(points, sample_inds, sample_sizes, query_points, query_sample_inds, query_sample_sizes):
    if query_points is None or query_sample_inds is None or query_sample_sizes is None:
        assert query_points is None and query_sample_inds is None and query_sample_sizes is None
        return points, sample_inds, sample_sizes
    return query_points, query_sample_inds, query_sample_sizes


@torch.compiler.disable
@_cabi.on_geometry_stream
def build_triplets_segmented(points, sample_inds, sample_sizes, neighbor_radius, kernel_size,
                             query_points=None, query_sample_inds=None, query_sample_sizes=None,
                             return_num_neighbors=False, radius_scaler=None, tap_stripes=32):
    """Returns ``(i, j, k int32, seg_offs int64, num_neighbors or None)`` with the
    triplets grouped by tap.  Raises when a query has no neighbour."""
    sizes = _triple(kernel_size)
    if not (sizes[0] == sizes[1] == sizes[2]):
        raise ValueError(f"segmented triplet construction requires a cubic kernel; got {sizes}")
    ks = int(sizes[0])
    if ks <= 0 or ks % 2 == 0:
        raise ValueError(f"segmented triplet construction requires a positive odd kernel; got {ks}")
    if radius_scaler is None or float(radius_scaler) <= 0:
        raise ValueError("segmented triplet construction requires a positive radius_scaler")
    kernel_grid_size = float(neighbor_radius) / float(radius_scaler)
    with torch.no_grad():
        query_points, query_sample_inds, query_sample_sizes = _resolve_queries(
            points, sample_inds, sample_sizes, query_points, query_sample_inds, query_sample_sizes)
        key = triplet_key(points, query_points, neighbor_radius, radius_scaler, "k", return_num_neighbors,
                          sample_inds, query_sample_inds, partial(voxelize_3d, kernel_size=sizes))
        if key is not None:
            key = key + ("segmented",)
        hit = cache_get(key)
        if hit is not None:
            return hit
        i, j, seg_offs, num_neighbors, k = radius_search_sorted_grid8_segments(
            points=points, queries=query_points, radius=neighbor_radius, kernel_size=ks,
            kernel_grid_size=kernel_grid_size, sample_inds=sample_inds,
            query_sample_inds=query_sample_inds, dtype_num_neighbors=torch.int64,
            distance_type="ball", tap_stripes=tap_stripes, return_k=True)
        lonely = getattr(num_neighbors, "pcx_queries_without_neighbor", None)   # counted by the search itself
        if lonely is None:
            lonely = int((num_neighbors == 0).sum().item()) if num_neighbors.numel() else 0
        if lonely:
            raise AssertionError(_NO_NEIGHBOR_MSG)
        if query_points is points:       # self-search: the rulebook is its own mirror image
            _cabi.mark_symmetric(i, j)
        out = (i, j, k, seg_offs, (num_neighbors if return_num_neighbors else None))
        cache_put(key, out, points)
        return out


def _triplets_from_pairs(points, query_points, neighbor_indices, num_neighbors, kernel_indexer,
                         neighbor_radius, radius_scaler, sort_by, return_num_neighbors):
    with torch.no_grad():
        assert torch.min(num_neighbors) > 0, _NO_NEIGHBOR_MSG
        starts, total = cumsum_exclusive(num_neighbors, return_sum=True)
        i = repeat_interleave_indices(repeats_cumsum=starts, output_size=int(total))
        j = neighbor_indices.long()
        offsets = points[j] - query_points[i]
        k = kernel_indexer(points=offsets, grid_size=neighbor_radius / radius_scaler)
        if sort_by == "j":
            j, order = torch.sort(j)
            i, k = i[order], k[order]
        elif sort_by == "k":
            k, order = torch.sort(k, stable=True)
            i, j = i[order], j[order]
        elif sort_by != "i":
            raise AssertionError(f'Unknown sort_by argument "{sort_by}", it should be i, j, or k!')
        dt = torch.int32 if max(query_points.shape[0], points.shape[0]) <= 2147483647 else torch.int64
        return i.to(dt), j.to(dt), k.to(dt), (num_neighbors if return_num_neighbors else None)


@torch.compiler.disable
@_cabi.on_geometry_stream
def build_triplets(points, sample_inds, sample_sizes, neighbor_radius, kernel_indexer: Callable,
                   query_points=None, query_sample_inds=None, query_sample_sizes=None, sort_by="k",
                   return_num_neighbors=False, radius_scaler: Optional[float] = None):
    """Generic builder: query-major search, tap from ``kernel_indexer``, global sort."""
    with torch.no_grad():
        query_points, query_sample_inds, query_sample_sizes = _resolve_queries(
            points, sample_inds, sample_sizes, query_points, query_sample_inds, query_sample_sizes)
        key = triplet_key(points, query_points, neighbor_radius, radius_scaler, sort_by, return_num_neighbors,
                          sample_inds, query_sample_inds, kernel_indexer)
        hit = cache_get(key)
        if hit is not None:
            return hit
        grid_size = neighbor_radius / radius_scaler if radius_scaler is not None else None
        neighbor_indices, num_neighbors = radius_search(
            points=points, query_points=query_points, radius=neighbor_radius, sample_inds=sample_inds,
            sample_sizes=sample_sizes, query_sample_inds=query_sample_inds,
            query_sample_sizes=query_sample_sizes, grid_size=grid_size)
    out = _triplets_from_pairs(points, query_points, neighbor_indices, num_neighbors, kernel_indexer,
                               neighbor_radius, radius_scaler, sort_by, return_num_neighbors)
    cache_put(key, out, points)
    return out


def _same_cloud(a: MetaData, b: MetaData):
    return (a is not None and a.points.shape == b.points.shape and a.grid_size == b.grid_size
            and torch.equal(a.points, b.points) and torch.equal(a.sample_inds, b.sample_inds))


def _build_for(m_points, m_sample_inds, m_sample_sizes, neighbor_radius, kernel_size, radius_scaler,
               sort_by, distance_type, return_num_neighbors, query=None):
    qp, qi, qs = query if query is not None else (None, None, None)
    if sort_by == "k" and distance_type == "ball" and should_use_direct_segmented_triplets(kernel_size):
        return build_triplets_segmented(
            points=m_points, sample_inds=m_sample_inds, sample_sizes=m_sample_sizes,
            neighbor_radius=neighbor_radius, kernel_size=kernel_size, query_points=qp,
            query_sample_inds=qi, query_sample_sizes=qs, return_num_neighbors=return_num_neighbors,
            radius_scaler=radius_scaler)
    i, j, k, nn = build_triplets(
        points=m_points, sample_inds=m_sample_inds, sample_sizes=m_sample_sizes,
        neighbor_radius=neighbor_radius, kernel_indexer=partial(voxelize_3d, kernel_size=kernel_size),
        query_points=qp, query_sample_inds=qi, query_sample_sizes=qs, sort_by=sort_by,
        return_num_neighbors=return_num_neighbors, radius_scaler=radius_scaler)
    seg = kernel_offset_segments(k, math.prod(_triple(kernel_size))) if sort_by == "k" else None
    return i, j, k, seg, nn


@torch.compiler.disable
@_cabi.on_geometry_stream
def handle_stride_and_build_triplets(m: MetaData, stride, kernel_size=_triple(3),
                                     receptive_field_scaler=1.0, sort_by="k",
                                     return_num_neighbors=False, distance_type="ball") -> MetaData:
    """Down-sample ``m`` by ``stride`` (when != 1) and attach the triplets that
    connect the parent cloud to the (down-sampled) query cloud.  The mirrored
    edges are cached on the parent for a later up-sampling layer."""
    with torch.no_grad():
        radius_scaler = radius_scaler_for_kernel_size(kernel_size, receptive_field_scaler, distance_type)
        if stride != 1:
            if _same_cloud(m.parent, m):
                parent = m.parent
            else:
                parent = MetaData(points=m.points, sample_inds=m.sample_inds, sample_sizes=m.sample_sizes,
                                  grid_size=m.grid_size, parent=m.parent)
                m.parent = parent
            neighbor_radius = parent.grid_size * radius_scaler
            m.points, m.sample_inds, m.grid_size, m.downsample_indices = downsample(
                m.points, m.sample_inds, m.grid_size, stride)
            m.sample_sizes = torch.bincount(m.sample_inds)
            m.i, m.j, m.k, m.seg_offs, m.num_neighbors = _build_for(
                parent.points, parent.sample_inds, parent.sample_sizes, neighbor_radius, kernel_size,
                radius_scaler, sort_by, distance_type, return_num_neighbors,
                query=(m.points, m.sample_inds, m.sample_sizes))
            parent.i_upsample, parent.j_upsample = m.j, m.i
            parent.k_upsample, parent.seg_offs_upsample = m.k, m.seg_offs
        if m.empty_triplets():
            neighbor_radius = m.grid_size * radius_scaler
            m.i, m.j, m.k, m.seg_offs, m.num_neighbors = _build_for(
                m.points, m.sample_inds, m.sample_sizes, neighbor_radius, kernel_size, radius_scaler,
                sort_by, distance_type, return_num_neighbors)
    m.contract = TripletContract(k_sorted=(sort_by == "k"))
    return m


def _own_parent(m: MetaData) -> MetaData:
    """The geometry of ``m`` before a strided layer changes it, linked as ``m.parent`` (reused when
    the existing parent already is that cloud)."""
    if _same_cloud(m.parent, m):
        return m.parent
    parent = MetaData(points=m.points, sample_inds=m.sample_inds, sample_sizes=m.sample_sizes,
                      grid_size=m.grid_size, parent=m.parent)
    m.parent = parent
    return parent


def partition_slots(points, cell_size, slots_per_axis):
    """Sub-voxel slot of every point inside its cell of side ``cell_size``: the cell is the floor
    division the grid sampler uses, the slot ``floor(frac * K)`` per axis (clamped to ``[0, K)`` against
    rounding at the upper face), x most significant (``layers/triplets.py:1130-1134`` of the reference;
    the same torch expressions, so that both run the same device arithmetic)."""
    K = int(slots_per_axis)
    cell = torch.div(points, cell_size, rounding_mode="floor")
    sub = torch.floor((points / cell_size - cell) * K).to(torch.long).clamp_(0, K - 1)
    return (sub[:, 0] * K + sub[:, 1]) * K + sub[:, 2]


@torch.compiler.disable
@_cabi.on_geometry_stream
def handle_stride_disjoint_and_build_triplets(m: MetaData, stride, kernel_size=_triple(3), sort_by="k") -> MetaData:
    """Strided convolution as a grid partition (``layers/triplets.py:1042-1167`` of the reference):
    no search.  Every input point belongs to exactly one cell of side ``stride * grid_size``; the
    output token is the cell centre, the tap is the point's sub-voxel slot in its cell (cubic
    kernel, ``K**3`` slots), so the rulebook has one triplet per input point.  The mirrored edges
    cached on the parent make ``Upsample(straight_recover=True, recompute_k=False)`` the exact inverse.

    With ``sort_by="k"`` the triplets are grouped by slot with a stable sort (inside a slot in point
    order; the reference's ``argsort`` leaves that order open)."""
    if stride <= 1:
        raise ValueError(f"handle_stride_disjoint_and_build_triplets requires stride > 1 (downsample case); "
                         f"got stride={stride}.")
    ks = _triple(kernel_size)
    if not (ks[0] == ks[1] == ks[2]):
        raise ValueError(f"partition disjoint conv requires a cubic kernel; got kernel_size={ks}")
    K = int(ks[0])
    with torch.no_grad():
        parent = _own_parent(m)
        pts, cell_size = parent.points, stride * parent.grid_size
        centres, sample_c, kept, token_of = grid_sample_filter(points=pts, grid_size=cell_size,
                                                               sample_inds=parent.sample_inds, reduction="center",
                                                               return_mapping=True)
        m.points, m.sample_inds, m.grid_size = centres.contiguous(), sample_c, cell_size
        m.sample_sizes = torch.bincount(sample_c)
        m.downsample_indices = kept
        slot = partition_slots(pts, cell_size, K)
        point = torch.arange(pts.shape[0], device=pts.device)
        if sort_by == "k":
            slot, order = torch.sort(slot, stable=True)
            point = point[order]
        m.i, m.j, m.k = token_of.to(torch.long)[point], point, slot
        m.seg_offs = kernel_offset_segments(m.k, K ** 3)
        m.num_neighbors = None
        parent.i_upsample, parent.j_upsample = m.j, m.i
        parent.k_upsample, parent.seg_offs_upsample = m.k, m.seg_offs
    # one triplet per input point by construction: the fan-out-1 contract holds whenever the
    # partition actually merges points (as many tokens as points would be the identity case,
    # which the reference leaves to the submanifold contract)
    n_in, n_out = pts.shape[0], m.points.shape[0]
    covers = m.k.numel() == n_in and n_in != n_out and n_in > 0
    m.contract = TripletContract(k_sorted=True, exact_cover_out=False, exact_cover_in=bool(covers),
                                 uniform_seg_len=None)
    return m


# --------------------------------------------------------------------------
# Full-cover strided rulebook (mirror of ``layers/triplets.py:36-465``)
# --------------------------------------------------------------------------
from dataclasses import dataclass  # noqa: E402

from torch import Tensor  # noqa: E402

from ..internals.grid_sample import grid_sample_filter  # noqa: E402


@dataclass(frozen=True)
class FullCoverStridedRulebook:
    """Rulebook of an overlapping strided convolution whose output centres are
    observed input points and whose balls of radius ``radius`` cover every
    input point (field set of the reference's dataclass)."""
    points: Tensor
    sample_inds: Tensor
    sample_sizes: Tensor
    center_source_indices: Tensor
    initial_center_source_indices: Tensor
    additional_center_source_indices: Tensor
    point_to_initial_center: Tensor
    i: Tensor
    j: Tensor
    k: Tensor
    num_neighbors: Optional[Tensor]
    i_upsample: Tensor
    j_upsample: Tensor
    k_upsample: Tensor
    radius: float
    radius_scaler: float
    initial_center_counts: Tensor
    additional_center_counts: Tensor
    selector_round_count: int
    coverage_per_input: Tensor


def _strict_taps(offsets, grid_size, K, context):
    """Tap of every offset without clamping: an offset outside the kernel is an error."""
    half = K // 2
    d = torch.round(offsets / float(grid_size)).to(torch.int64)
    if d.numel():
        worst = int(d.abs().max().item())
        if worst > half:
            raise ValueError(
                f"{context} kernel_size={K} is insufficient for observed offset {worst} grid steps; "
                f"need at least K{2 * worst + 1}. Full-cover strided convolution never clamps or "
                "aliases out-of-range offsets.")
    return ((d[:, 0] + half) * K + (d[:, 1] + half)) * K + (d[:, 2] + half), d


def _edges(points, sample_inds, centers, center_sample, radius, backend):
    """(centre ordinal, point index, per-centre counts) of all pairs within ``radius``."""
    nb, counts = radius_search(points=points, query_points=centers, radius=radius, sample_inds=sample_inds,
                               query_sample_inds=center_sample, backend=backend)
    owner = torch.repeat_interleave(torch.arange(counts.numel(), device=points.device), counts,
                                    output_size=int(nb.numel()))
    return owner, nb.long(), counts


def _residual_net(points, sample_inds, c0_points, point_to_c0, uncovered, radius, backend):
    """Deterministic maximal R-net over the points no initial centre covers (the device selector
    ``pcx_rnet_rounds``; the reference's host loop is layers/triplets.py:156-232).  Returns the
    chosen source indices ordered by (sample, index) and the number of rounds."""
    from .. import _cabi

    src = torch.nonzero(uncovered).squeeze(1)
    if src.numel() == 0:
        return torch.empty(0, dtype=torch.long, device=points.device), 0
    up, us = points[src], sample_inds[src]
    _, nb, counts = _edges(up, us, up, us, radius, backend)
    offsets = torch.zeros(src.numel() + 1, dtype=torch.int64, device=points.device)
    torch.cumsum(counts, 0, out=offsets[1:])
    chosen, rounds = _cabi.rnet_select(up, c0_points, point_to_c0[src], nb, offsets, src)
    added = src[chosen]      # ascending source index; stable by sample below
    return added[torch.argsort(sample_inds[added], stable=True)], rounds


@torch.compiler.disable
@_cabi.on_geometry_stream
def build_full_cover_strided_rulebook(points, sample_inds, sample_sizes, *, stride, input_grid_size,
                                      kernel_size, radius_margin=1e-2, radius_backend="auto",
                                      return_num_neighbors=True) -> FullCoverStridedRulebook:
    """Centres = the observed point nearest every occupied stride cell's centre,
    plus a residual R-net over the points those centres leave uncovered; edges =
    all (centre, point) pairs within ``R = sqrt(3)/2 * stride * grid * (1 + margin)``;
    taps by strict (non-clamping) voxelisation; the mirrored rulebook for the
    matching up-sampling layer comes with it."""
    with torch.no_grad():
        if points.dim() != 2 or points.shape[1] != 3:
            raise ValueError(f"points must have shape (N, 3); got {tuple(points.shape)}")
        dev = points.device
        N = points.shape[0]
        if sample_inds is None:
            sample_inds = torch.zeros(N, device=dev, dtype=torch.long)
        sample_inds = sample_inds.to(torch.long)
        if sample_sizes is None:
            sample_sizes = torch.bincount(sample_inds)
        if points.numel() == 0:
            e = torch.empty(0, device=dev, dtype=torch.long)
            z = torch.zeros(0, device=dev, dtype=torch.long)
            return FullCoverStridedRulebook(points, sample_inds, sample_sizes, e, e, e, e, e, e, e,
                                            z if return_num_neighbors else None, e, e, e, 0.0, 0.0,
                                            torch.zeros_like(sample_sizes), torch.zeros_like(sample_sizes), 0, z)
        radius_scaler = full_cover_radius_scaler(stride, radius_margin)
        radius = float(input_grid_size) * radius_scaler
        need = minimum_full_cover_kernel_size(radius_scaler)
        ks = _triple(kernel_size)
        K = int(ks[0])
        if not (ks[0] == ks[1] == ks[2]):
            raise ValueError(f"full-cover strided conv requires a cubic kernel; got {ks}")
        if K < need:
            raise ValueError(f"full-cover stride={stride} at grid_size={input_grid_size} "
                             f"needs kernel_size >= {need}; got {kernel_size}")

        # initial centres: one per occupied stride cell, ordered by (sample, source index)
        _, _, cell_pick, cell_of_point = grid_sample_filter(
            points, float(stride) * float(input_grid_size), sample_inds, reduction="center_nearest",
            return_mapping=True)
        by_source = torch.argsort(sample_inds[cell_pick] * (N + 1) + cell_pick, stable=True)
        c0 = cell_pick[by_source]
        rank_of_cell = torch.empty_like(by_source)
        rank_of_cell[by_source] = torch.arange(by_source.numel(), device=dev)
        point_to_c0 = rank_of_cell[cell_of_point]

        c0_owner, c0_nb, c0_counts = _edges(points, sample_inds, points[c0], sample_inds[c0], radius, radius_backend)
        covered = torch.zeros(N, dtype=torch.bool, device=dev)
        covered[c0_nb] = True
        c1, rounds = _residual_net(points, sample_inds, points[c0], point_to_c0, ~covered, radius, radius_backend)

        multi = sample_sizes.numel() > 1
        if c1.numel() and multi:
            both = torch.cat([c0, c1])
            group = torch.cat([torch.zeros_like(c0), torch.ones_like(c1)])
            order = torch.argsort(sample_inds[both] * (2 * (N + 1)) + group * (N + 1) + both, stable=True)
            centers = both[order]
        else:
            centers = torch.cat([c0, c1]) if c1.numel() else c0
        slot = torch.empty(N, dtype=torch.long, device=dev)
        slot[centers] = torch.arange(centers.numel(), device=dev)
        point_to_center = slot[c0[point_to_c0]]

        center_points = points[centers].contiguous()
        center_sample = sample_inds[centers].contiguous()
        i_parts, j_parts = [slot[c0[c0_owner]]], [c0_nb]
        num_neighbors = torch.zeros(centers.numel(), dtype=c0_counts.dtype, device=dev)
        num_neighbors[slot[c0]] = c0_counts
        if c1.numel():
            c1_owner, c1_nb, c1_counts = _edges(points, sample_inds, points[c1], sample_inds[c1], radius, radius_backend)
            i_parts.append(slot[c1[c1_owner]])
            j_parts.append(c1_nb)
            num_neighbors[slot[c1]] = c1_counts
        i, j = torch.cat(i_parts), torch.cat(j_parts)
        k, d = _strict_taps(points[j] - center_points[i], input_grid_size, K, "full-cover patchify")
        k, order = torch.sort(k, stable=True)
        i, j, d = i[order], j[order], d[order]

        coverage = torch.bincount(j, minlength=N)
        if bool((coverage == 0).any().item()):
            raise RuntimeError("full-cover rulebook construction failed: some input points have zero incident edges")
        k_up, _ = _strict_taps(-d.to(points.dtype) * float(input_grid_size), input_grid_size, K,
                               "full-cover unpatchify")
        k_up, up_order = torch.sort(k_up, stable=True)
        idt = torch.int32 if max(N, centers.numel()) <= 2147483647 else torch.int64
        nS = sample_sizes.numel()
        return FullCoverStridedRulebook(
            points=center_points, sample_inds=center_sample,
            sample_sizes=torch.bincount(center_sample, minlength=nS),
            center_source_indices=centers.to(idt), initial_center_source_indices=c0.to(idt),
            additional_center_source_indices=c1.to(idt), point_to_initial_center=point_to_center.to(idt),
            i=i.to(idt), j=j.to(idt), k=k.to(idt),
            num_neighbors=num_neighbors if return_num_neighbors else None,
            i_upsample=j[up_order].to(idt), j_upsample=i[up_order].to(idt), k_upsample=k_up.to(idt),
            radius=radius, radius_scaler=radius_scaler,
            initial_center_counts=torch.bincount(sample_inds[c0], minlength=nS),
            additional_center_counts=torch.bincount(sample_inds[c1], minlength=nS),
            selector_round_count=rounds, coverage_per_input=coverage.to(idt))
