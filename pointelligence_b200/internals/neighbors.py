"""Exact fixed-radius neighbour search (mirror of ``internals/neighbors.py``:
``radius_search`` :281-339, ``radius_search_sorted_grid8`` :886-916,
``radius_search_sorted_grid8_segments`` :919-955).

One implementation serves every backend name the reference accepts: points are
binned into cells of side ``2 R``, sorted by a 64-bit cell key, and every query
scans the eight cells its radius box touches with the reference's fp32
predicate ``sqrt((dx^2 + dy^2) + dz^2) <= float32(R)``.  Neighbour order inside
a query / inside a tap is deterministic but, as in the reference, not part of
the contract.
"""
from __future__ import annotations

from contextlib import contextmanager

import torch

from .. import _cabi

_PREDICATES = {"ieee": 0, "fma": 1, "fma_approx_sqrt": 2}


@contextmanager
def radius_predicate(mode):
    """Scope the fp32 arithmetic of the distance predicate.

    ``"fma"`` (default) is what the reference's Triton kernels compute on a
    B200 (the compiler contracts the sum of squares into fused multiply-adds);
    ``"ieee"`` rounds every operation, which is what the same kernels compute
    under Triton's CPU interpreter.  The two differ only for pairs within an
    ulp or two of the radius."""
    if mode not in _PREDICATES:
        raise ValueError(f"radius predicate must be one of {sorted(_PREDICATES)}; got {mode!r}")
    lib = _cabi.lib()
    prev = lib.pcx_get_radius_predicate()
    _cabi.check(lib.pcx_set_radius_predicate(_PREDICATES[mode]))
    try:
        yield
    finally:
        _cabi.check(lib.pcx_set_radius_predicate(prev))


_BACKENDS = {"auto", "sorted8_materialized", "sorted27_materialized", "tiled", "sorted_grid8", "fixed_grid"}


def _distance_code(distance_type):
    if distance_type not in ("ball", "chebyshev"):
        raise ValueError(f"distance_type must be 'ball' or 'chebyshev'; got {distance_type!r}")
    return 0 if distance_type == "ball" else 1


def _check_inputs(points, queries, sample_inds, query_sample_inds):
    assert points.dim() == 2 and points.shape[1] == 3
    assert queries.dim() == 2 and queries.shape[1] == 3
    assert points.dtype == queries.dtype, (points.dtype, queries.dtype)
    assert points.device == queries.device
    if sample_inds is not None:
        assert query_sample_inds is not None
    else:
        assert query_sample_inds is None
    _cabi.require_cuda(points, queries, sample_inds, query_sample_inds)


def _f32(x):
    return x.detach().float().contiguous()


@torch.no_grad()
@_cabi.on_geometry_stream
def radius_search_sorted_grid8(points, queries, radius, sample_inds=None, query_sample_inds=None,
                               return_distances=False, dtype_num_neighbors=torch.int64,
                               distance_type="ball"):
    """Returns ``(neighbors, num_neighbors[, distances])``, query-major.

    ``neighbors`` is int64 (int32 when empty, as in the reference); distances
    are in the points' dtype.
    """
    if float(radius) <= 0:
        raise ValueError(f"radius must be positive; got {radius}")
    code = _distance_code(distance_type)
    _check_inputs(points, queries, sample_inds, query_sample_inds)
    dev = points.device
    P, Q = points.shape[0], queries.shape[0]
    if P == 0 or Q == 0:
        empty = torch.empty(0, dtype=torch.int32, device=dev)
        counts = torch.zeros(Q, dtype=dtype_num_neighbors, device=dev)
        if return_distances:
            return empty, counts, torch.empty(0, dtype=points.dtype, device=dev)
        return empty, counts
    nb, counts, dist = _cabi.radius_search(_f32(points), _f32(queries), float(radius), sample_inds,
                                           query_sample_inds, code, return_distances=return_distances)
    counts = counts.to(dtype_num_neighbors)
    if nb.numel() == 0:
        nb = torch.empty(0, dtype=torch.int32, device=dev)
    if return_distances:
        return nb, counts, dist.to(points.dtype)
    return nb, counts


@torch.no_grad()
@_cabi.on_geometry_stream
def radius_search_sorted_grid8_segments(points, queries, radius, kernel_size, kernel_grid_size,
                                        sample_inds=None, query_sample_inds=None,
                                        dtype_num_neighbors=torch.int64, distance_type="ball",
                                        tap_stripes=32, return_k=False):
    """Returns ``(i, j, seg_offs, num_neighbors)``: accepted (query, point)
    pairs grouped by kernel tap (int32), the ``kernel_size**3 + 1`` int64 tap
    offsets and the per-query counts.  ``tap_stripes`` is validated for source
    compatibility; emission here is a deterministic scan + stable sort, so it
    has no effect.  With ``return_k`` the tap of every pair is appended.
    """
    if float(radius) <= 0:
        raise ValueError(f"radius must be positive; got {radius}")
    code = _distance_code(distance_type)
    if kernel_size is None or kernel_grid_size is None:
        raise ValueError("kernel_size and kernel_grid_size must be supplied together")
    kernel_size = int(kernel_size)
    if kernel_size <= 0 or kernel_size % 2 == 0:
        raise ValueError(f"kernel_size must be a positive odd integer; got {kernel_size}")
    if float(kernel_grid_size) <= 0:
        raise ValueError(f"kernel_grid_size must be positive; got {kernel_grid_size}")
    tap_stripes = int(tap_stripes)
    if tap_stripes <= 0 or tap_stripes > 256 or tap_stripes & (tap_stripes - 1):
        raise ValueError(f"tap_stripes must be a power of two in [1, 256]; got {tap_stripes}")
    _check_inputs(points, queries, sample_inds, query_sample_inds)
    dev = points.device
    P, Q = points.shape[0], queries.shape[0]
    if P == 0 or Q == 0:
        empty = torch.empty(0, dtype=torch.int32, device=dev)
        seg = torch.zeros(kernel_size ** 3 + 1, dtype=torch.int64, device=dev)
        out = (empty, empty.clone(), seg, torch.zeros(Q, dtype=dtype_num_neighbors, device=dev))
        return out + (empty.clone(),) if return_k else out
    i, j, k, seg, counts = _cabi.radius_search(_f32(points), _f32(queries), float(radius), sample_inds,
                                               query_sample_inds, code, kernel_size=kernel_size,
                                               kernel_grid_size=float(kernel_grid_size), want_k=return_k)
    cast = counts.to(dtype_num_neighbors)
    if hasattr(counts, "pcx_queries_without_neighbor"):
        cast.pcx_queries_without_neighbor = counts.pcx_queries_without_neighbor
    out = (i, j, seg, cast)
    return out + (k,) if return_k else out


def radius_search_fixed_grid(points, queries, radius, sample_inds=None, query_sample_inds=None,
                             return_distances=False, dtype_num_neighbors=torch.int64, distance_type="ball"):
    """The reference's 27-cell variant returns the same pair set as the
    eight-cell search (its own tests assert that); one search serves both."""
    return radius_search_sorted_grid8(points, queries, radius, sample_inds, query_sample_inds,
                                      return_distances, dtype_num_neighbors, distance_type)


def radius_search(points, query_points, radius, sample_inds=None, query_sample_inds=None,
                  return_distances=False, point_num_max=1000000, sample_sizes=None,
                  query_sample_sizes=None, distance_type="ball", tiled_batch_threshold=20000,
                  grid_size=None, tiled_radius_multiplier_threshold=4.5, backend="auto",
                  fixed_grid_radius_multiplier_threshold=2.75):
    """Top-level entry point; legacy tuning arguments are accepted and ignored."""
    if backend not in _BACKENDS:
        raise ValueError("backend must be auto, sorted8_materialized, sorted27_materialized, or tiled; "
                         f"got {backend!r}")
    if grid_size is not None and float(grid_size) <= 0:
        raise ValueError(f"grid_size must be positive; got {grid_size}")
    return radius_search_sorted_grid8(points, query_points, radius, sample_inds, query_sample_inds,
                                      return_distances, torch.int64, distance_type)
