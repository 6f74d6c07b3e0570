"""numpy restatement of the reference geometry stage (TEST INFRASTRUCTURE).

Every function states the reference lines it follows.  All arithmetic that
decides set membership is done in IEEE float32 with one rounding per
operation, exactly as written in the reference source:

* candidate cells          internals/neighbors.py:603-681
* radius predicate         sparse_engines/strided_grid_radius_triton_kernel.py:25-31,127
* kernel-tap index         sparse_engines/strided_grid_radius_triton_kernel.py:71-92
                           (== layers/triplets.py:547-561, ``voxelize_3d``)
* tap-segment offsets      internals/neighbors.py:755-759
* grid cell of a point     internals/grid_indexing.py:20-27
* mixed-radix cell key     internals/grid_indexing.py:30-67
* centre-nearest selector  internals/grid_sample.py:14-39,
                           internals/grid_sample_triton_kernel.py:55-106
* radius scalers           layers/triplets.py:61-70,767-807

Outputs use a canonical order (documented per function) because the reference
leaves the order inside a tap / inside a query unspecified.
"""
from __future__ import annotations

import math

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# scalar formulas
# --------------------------------------------------------------------------
def radius_scaler_for_kernel_size(kernel_size, receptive_field_scaler=1.0,
                                  distance_type="ball"):
    """layers/triplets.py:767-807."""
    if isinstance(kernel_size, int):
        kernel_size = (kernel_size,) * 3
    kmax = max(kernel_size)
    if distance_type == "cube":
        return kmax * math.pow(receptive_field_scaler, 1 / 3) / 2.0
    volume = math.pow(kmax, 3) * receptive_field_scaler
    return math.pow(3 * volume / (4 * math.pi), 1 / 3)


def full_cover_radius_scaler(stride, radius_margin=1e-2):
    """layers/triplets.py:61-66."""
    return (math.sqrt(3.0) / 2.0) * float(stride) * (1.0 + float(radius_margin))


def minimum_full_cover_kernel_size(radius_scaler):
    """layers/triplets.py:69-70."""
    return 2 * int(math.ceil(float(radius_scaler))) + 1


# --------------------------------------------------------------------------
# fixed-radius search
# --------------------------------------------------------------------------
def _as_f32(x):
    return np.ascontiguousarray(np.asarray(x, dtype=F32))


def radius_distance(q, p, distance_type="ball", fma=False):
    """Distance of the predicate, float32.

    sparse_engines/strided_grid_radius_triton_kernel.py:25-31: ``d = q - p``
    per axis, ``sqrt((dx*dx + dy*dy) + dz*dz)`` for the ball, ``max |d|`` for
    the Chebyshev variant.  ``fma=False`` rounds every operation (the
    expression as written; Triton's CPU interpreter).  ``fma=True`` restates
    what the GPU compiler makes of it, ``fma(dz,dz, fma(dx,dx, dy*dy))``: the
    products are exact in float64 and each fused step is rounded once to fp32.
    """
    d = (q - p).astype(F32)
    if distance_type == "ball" and fma:
        d64 = d.astype(np.float64)
        s = (d[..., 1] * d[..., 1]).astype(F32)
        s = (d64[..., 0] * d64[..., 0] + s.astype(np.float64)).astype(F32)
        s = (d64[..., 2] * d64[..., 2] + s.astype(np.float64)).astype(F32)
        return np.sqrt(s).astype(F32)
    if distance_type == "ball":
        s = (d[..., 0] * d[..., 0]).astype(F32)
        s = (s + (d[..., 1] * d[..., 1]).astype(F32)).astype(F32)
        s = (s + (d[..., 2] * d[..., 2]).astype(F32)).astype(F32)
        return np.sqrt(s).astype(F32)
    return np.max(np.abs(d), axis=-1).astype(F32)


def tap_index(p, q, kernel_grid_size, kernel_size):
    """Kernel tap of the offset ``p - q`` (point minus query).

    sparse_engines/strided_grid_radius_triton_kernel.py:71-92: correctly
    rounded fp32 division by ``float32(kernel_grid_size)``, round half to
    even, shift by ``K // 2``, clamp to ``[0, K-1]``, x most significant.
    """
    g = F32(kernel_grid_size)
    K = int(kernel_size)
    half = K // 2
    d = np.rint(((p - q).astype(F32) / g).astype(F32)).astype(np.int64)
    kk = np.clip(d + half, 0, K - 1)
    return (kk[..., 0] * K + kk[..., 1]) * K + kk[..., 2]


def _candidate_pairs(points, queries, radius, sample_inds, query_sample_inds):
    """All (query, point) pairs the eight-cell lookup inspects.

    internals/neighbors.py:603-681 with ``cell_cover_mode="exact8"``: cell side
    ``2 R``; a point lives in ``floor(p * inv)``, a query looks at the eight
    cells ``floor((q - R) * inv) + {0,1}^3`` of its own sample.
    Returns flat int64 arrays (cand_q, cand_p) ordered by query, then cell
    offset (x slowest), then sorted-point position.
    """
    P, Q = points.shape[0], queries.shape[0]
    R32 = F32(float(radius))
    inv = F32(1.0 / (2.0 * float(radius)))
    cell_in = np.floor((points * inv).astype(F32)).astype(np.int64)
    cell_out = np.floor((((queries - R32).astype(F32)) * inv).astype(F32)).astype(np.int64)
    base = np.minimum(cell_in.min(0), cell_out.min(0)) - 1
    top = np.maximum(cell_in.max(0), cell_out.max(0)) + 1 + 1
    extent = np.maximum(top - base, 1)
    sx, sy = extent[1] * extent[2], extent[2]
    ci, co = cell_in - base, cell_out - base
    hash_in = ci[:, 0] * sx + ci[:, 1] * sy + ci[:, 2]
    hash_out = co[:, 0] * sx + co[:, 1] * sy + co[:, 2]
    if sample_inds is not None:
        vol = int(extent.prod())
        hash_in = hash_in + np.asarray(sample_inds, dtype=np.int64) * vol
        hash_out = hash_out + np.asarray(query_sample_inds, dtype=np.int64) * vol
    perm = np.argsort(hash_in, kind="stable")
    sorted_hash = hash_in[perm]
    offs = np.array([(a, b, c) for a in (0, 1) for b in (0, 1) for c in (0, 1)],
                    dtype=np.int64)
    off_hash = offs[:, 0] * sx + offs[:, 1] * sy + offs[:, 2]
    flat = (hash_out[:, None] + off_hash[None, :]).reshape(-1)
    start = np.searchsorted(sorted_hash, flat, side="left")
    end = np.searchsorted(sorted_hash, flat + 1, side="left")
    counts = end - start
    total = int(counts.sum())
    if total == 0:
        z = np.zeros(0, dtype=np.int64)
        return z, z
    cell_of = np.repeat(np.arange(Q * 8, dtype=np.int64), counts)
    first = np.cumsum(counts) - counts
    inner = np.arange(total, dtype=np.int64) - first[cell_of]
    cand_p = perm[start[cell_of] + inner]
    cand_q = cell_of // 8
    return cand_q, cand_p


def radius_search_sorted_grid8(points, queries, radius, sample_inds=None,
                               query_sample_inds=None, return_distances=False,
                               distance_type="ball", fma=False):
    """Exact fixed-radius neighbours, query-major.

    internals/neighbors.py:886-916 (→ 469-838).  Membership: fp32
    ``dist <= float32(radius)``, self pairs included, same sample only.
    Canonical order: query ascending, then point index ascending.
    Returns ``(neighbors int64 (E,), num_neighbors int64 (Q,)[, distances])``.
    """
    if float(radius) <= 0:
        raise ValueError(f"radius must be positive; got {radius}")
    points, queries = _as_f32(points), _as_f32(queries)
    Q = queries.shape[0]
    if points.shape[0] == 0 or Q == 0:
        out = (np.zeros(0, np.int64), np.zeros(Q, np.int64))
        return out + ((np.zeros(0, F32),) if return_distances else ())
    cq, cp = _candidate_pairs(points, queries, radius, sample_inds, query_sample_inds)
    dist = radius_distance(queries[cq], points[cp], distance_type, fma)
    keep = dist <= F32(float(radius))
    cq, cp, dist = cq[keep], cp[keep], dist[keep]
    order = np.lexsort((cp, cq))
    cq, cp, dist = cq[order], cp[order], dist[order]
    counts = np.bincount(cq, minlength=Q).astype(np.int64)
    if return_distances:
        return cp, counts, dist
    return cp, counts


def radius_search_sorted_grid8_segments(points, queries, radius, kernel_size,
                                        kernel_grid_size, sample_inds=None,
                                        query_sample_inds=None,
                                        distance_type="ball", fma=False):
    """Neighbour pairs grouped by kernel tap.

    internals/neighbors.py:919-955 (→ 469-838, prepared-segment branch).
    Canonical order: tap ascending, then query ``i`` ascending, then point
    ``j`` ascending (a legal instance of the reference's "order inside a tap
    is unspecified").  Returns ``(i int32, j int32, seg_offs int64 (K^3+1,),
    num_neighbors int64 (Q,))``.
    """
    if float(radius) <= 0:
        raise ValueError(f"radius must be positive; got {radius}")
    K = int(kernel_size)
    if K <= 0 or K % 2 == 0:
        raise ValueError(f"kernel_size must be a positive odd integer; got {K}")
    if float(kernel_grid_size) <= 0:
        raise ValueError(f"kernel_grid_size must be positive; got {kernel_grid_size}")
    points, queries = _as_f32(points), _as_f32(queries)
    Q = queries.shape[0]
    nk = K ** 3
    if points.shape[0] == 0 or Q == 0:
        e = np.zeros(0, np.int32)
        return e, e.copy(), np.zeros(nk + 1, np.int64), np.zeros(Q, np.int64)
    cq, cp = _candidate_pairs(points, queries, radius, sample_inds, query_sample_inds)
    dist = radius_distance(queries[cq], points[cp], distance_type, fma)
    keep = dist <= F32(float(radius))
    cq, cp = cq[keep], cp[keep]
    k = tap_index(points[cp], queries[cq], kernel_grid_size, K)
    order = np.lexsort((cp, cq, k))
    cq, cp, k = cq[order], cp[order], k[order]
    seg = np.zeros(nk + 1, np.int64)
    seg[1:] = np.cumsum(np.bincount(k, minlength=nk))
    counts = np.bincount(cq, minlength=Q).astype(np.int64)
    return cq.astype(np.int32), cp.astype(np.int32), seg, counts


def voxelize_3d(kernel_size, offsets, grid_size):
    """layers/triplets.py:547-561 on fp32 offsets with an fp32 grid size."""
    z = np.zeros_like(_as_f32(offsets))
    return tap_index(_as_f32(offsets), z, grid_size, kernel_size).astype(np.int32)


def canonical_triplet_keys(i, j, k, num_queries, num_points):
    """tests/unittest/test_radius_search_sorted_grid.py:129-137."""
    key = (np.asarray(k, np.int64) * (num_queries * num_points)
           + np.asarray(i, np.int64) * num_points + np.asarray(j, np.int64))
    return np.sort(key)


# --------------------------------------------------------------------------
# centre-nearest grid down-sampling
# --------------------------------------------------------------------------
def grid_cell_indices(points, grid_size):
    """Cell of every point, int32.

    internals/grid_indexing.py:20-27: ``points.div(grid_size,
    rounding_mode="floor")`` – Python-style floor division evaluated in the
    points' dtype (fmod, subtract, divide, round-to-nearest-integer fix-up),
    i.e. the floor of the exact quotient by ``float32(grid_size)``, not
    ``floor(p * (1 / grid))``.  numpy's ``floor_divide`` on float32 uses the
    same algorithm.
    """
    pts = _as_f32(points)
    return np.floor_divide(pts, F32(grid_size)).astype(np.int32)


def grid_keys(grid_inds):
    """Mixed-radix key, first column fastest, last column (sample) slowest.

    internals/grid_indexing.py:30-67.
    """
    g = np.asarray(grid_inds, dtype=np.int64)
    gmin = g.min(0, keepdims=True)
    step = g.max(0, keepdims=True) + 1 - gmin
    stride = np.cumprod(step, axis=-1)
    stride = np.roll(stride, 1, axis=-1)
    stride[0, 0] = 1
    return ((g - gmin) * stride).sum(-1)


def grid_sample_center_nearest(points, grid_size, sample_inds=None,
                               return_mapping=False):
    """One representative per occupied cell: the point nearest the centre.

    internals/grid_sample.py:42-121 with ``reduction="center_nearest"``;
    selector arithmetic from internals/grid_sample_triton_kernel.py:68-104
    (``c = (g + 0.5) * cell``, ``d = c - p``, ``(dx^2 + dy^2) + dz^2``, every
    operation rounded to fp32, ties to the lowest source index).  Cells are
    emitted by ascending key (sample-major, then z, y, x).
    Returns ``(points_f, sample_inds_f or None, indices int64, mapping or None)``.
    """
    pts = _as_f32(points)
    N = pts.shape[0]
    g = grid_cell_indices(pts, grid_size)
    cols = g if sample_inds is None else np.concatenate(
        [g, np.asarray(sample_inds).reshape(-1, 1).astype(np.int32)], axis=1)
    if N == 0:
        idx = np.zeros(0, np.int64)
        return pts[idx], (None if sample_inds is None else np.asarray(sample_inds)[idx]), idx, (
            np.zeros(0, np.int64) if return_mapping else None)
    keys = grid_keys(cols)
    uniq, inverse = np.unique(keys, return_inverse=True)
    cs = F32(grid_size)
    c = ((g.astype(F32) + F32(0.5)).astype(F32) * cs).astype(F32)
    d = (c - pts).astype(F32)
    d2 = (d[:, 0] * d[:, 0]).astype(F32)
    d2 = (d2 + (d[:, 1] * d[:, 1]).astype(F32)).astype(F32)
    d2 = (d2 + (d[:, 2] * d[:, 2]).astype(F32)).astype(F32)
    order = np.lexsort((np.arange(N), d2, inverse))
    first = np.ones(N, bool)
    first[1:] = inverse[order][1:] != inverse[order][:-1]
    indices = order[first].astype(np.int64)
    si = None if sample_inds is None else np.asarray(sample_inds)[indices]
    return pts[indices], si, indices, (inverse.astype(np.int64) if return_mapping else None)


# --------------------------------------------------------------------------
# grid partition (patchify) rulebook
# --------------------------------------------------------------------------
def partition_triplets(points, grid_size, stride, kernel_size, sample_inds=None):
    """Rulebook of the disjoint strided convolution: one triplet per input point.

    layers/triplets.py:1042-1167 (``handle_stride_disjoint_and_build_triplets``): the token of a
    point is its cell of side ``stride * grid_size`` (cells in the order of
    ``grid_sample_center_nearest``, token coordinate = cell centre ``(g + 0.5) * cell``), the tap is
    ``floor(frac * K)`` per axis with ``frac = p / cell - floor_div(p, cell)`` in fp32, clamped to
    ``[0, K)``, x most significant; triplets grouped by tap (stable, point order inside a tap).
    Returns ``(i int64, j int64, k int64, centres fp32 (S, 3), slack)`` where ``slack`` is, per
    point, the distance of ``frac * K`` (evaluated in float64) from the nearest integer: a device
    that divides by multiplying with the reciprocal may move points with a slack of a few ulp into
    the neighbouring slot.
    """
    pts = _as_f32(points)
    K = int(kernel_size)
    cell = F32(float(stride) * float(grid_size))
    _, _, indices, token_of = grid_sample_center_nearest(pts, cell, sample_inds, return_mapping=True)
    g = grid_cell_indices(pts, cell)
    centres = ((g[indices].astype(F32) + F32(0.5)).astype(F32) * cell).astype(F32)
    frac = ((pts / cell).astype(F32) - g.astype(F32)).astype(F32)
    sub = np.clip(np.floor((frac * F32(K)).astype(F32)).astype(np.int64), 0, K - 1)
    slot = (sub[:, 0] * K + sub[:, 1]) * K + sub[:, 2]
    exact = pts.astype(np.float64) / float(cell)
    scaled = (exact - np.floor(exact)) * K
    slack = np.abs(scaled - np.round(scaled)).min(axis=1)
    order = np.argsort(slot, kind="stable")
    return token_of[order].astype(np.int64), order.astype(np.int64), slot[order], centres, slack[order]
