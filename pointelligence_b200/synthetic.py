"""Seeded synthetic point clouds that stand in for the datasets the reference
measures on (ScanNet-like indoor rooms, nuScenes/Waymo-like LiDAR sweeps).

Only shapes, scales and value distributions are modelled: metre units, 2 cm
indoor sampling, 64-beam spinning scans.  All generators are numpy
``Generator(PCG64(seed))`` based and return float32 arrays.
"""
from __future__ import annotations

import numpy as np


def _box_faces(lo, hi, include_bottom):
    """Axis-aligned faces of a box as (origin, edge_u, edge_v) triples."""
    lo, hi = np.asarray(lo, float), np.asarray(hi, float)
    d = hi - lo
    faces = []
    for axis in range(3):
        u, v = [a for a in range(3) if a != axis]
        for side in (0, 1):
            if axis == 2 and side == 0 and not include_bottom:
                continue
            o = lo.copy()
            if side:
                o[axis] = hi[axis]
            eu = np.zeros(3)
            ev = np.zeros(3)
            eu[u], ev[v] = d[u], d[v]
            faces.append((o, eu, ev))
    return faces


def indoor_scene(n_points, seed, voxel=0.02, jitter=0.005, max_rounds=64):
    """Room 6 x 6 x 3 m plus 20 random boxes (edges U[0.3, 1.5] m) resting on
    the floor; points sampled uniformly (area weighted) on all room faces and
    the five exposed faces of every box, Gaussian jitter ``jitter`` per
    coordinate, de-duplicated on a ``voxel`` grid (first point per voxel wins).
    Returns up to ``n_points`` survivors of a seeded permutation, float32 (N, 3).
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    room_lo, room_hi = np.zeros(3), np.array([6.0, 6.0, 3.0])
    faces = _box_faces(room_lo, room_hi, include_bottom=True)
    for _ in range(20):
        size = rng.uniform(0.3, 1.5, 3)
        lo = np.array([rng.uniform(0, 6.0 - size[0]), rng.uniform(0, 6.0 - size[1]), 0.0])
        faces += _box_faces(lo, lo + size, include_bottom=False)
    origin = np.stack([f[0] for f in faces])
    eu = np.stack([f[1] for f in faces])
    ev = np.stack([f[2] for f in faces])
    area = np.linalg.norm(np.cross(eu, ev), axis=1)
    prob = area / area.sum()

    def draw(count):
        f = rng.choice(len(faces), size=count, p=prob)
        a, b = rng.random((count, 1)), rng.random((count, 1))
        p = origin[f] + a * eu[f] + b * ev[f]
        p = p + rng.normal(0.0, jitter, size=p.shape)
        return p.astype(np.float32)

    pts = draw(3 * n_points)
    keep = None
    for _ in range(max_rounds):
        cells = np.floor(pts / np.float32(voxel)).astype(np.int64)
        cells -= cells.min(0)
        ext = cells.max(0) + 1
        key = (cells[:, 0] * ext[1] + cells[:, 1]) * ext[2] + cells[:, 2]
        _, first = np.unique(key, return_index=True)
        keep = np.sort(first)
        if keep.size >= n_points:
            break
        pts = np.concatenate([pts, draw(n_points)])
    survivors = pts[keep]
    order = rng.permutation(survivors.shape[0])
    return np.ascontiguousarray(survivors[order][:n_points])


def lidar_sweep(seed, beams=64, azimuths=2048, max_range=80.0, keep=0.9):
    """One 64-beam spinning scan: sensor at (0, 0, 1.73), elevations
    -25 deg..+3 deg, ground plane z = 0 and 40 random boxes (footprint
    U[1,5] x U[1,3] m, height U[1,3] m, centres in the 3-50 m annulus).
    Returns the hit points, float32 (N, 3), roughly 100-120 k of them.
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    sensor = np.array([0.0, 0.0, 1.73])
    elev = np.deg2rad(np.linspace(-25.0, 3.0, beams))
    azim = 2 * np.pi * np.arange(azimuths) / azimuths
    ce, se = np.cos(elev)[:, None], np.sin(elev)[:, None]
    dirs = np.stack([ce * np.cos(azim)[None], ce * np.sin(azim)[None],
                     np.broadcast_to(se, (beams, azimuths))], axis=-1).reshape(-1, 3)
    t_best = np.full(dirs.shape[0], np.inf)
    down = dirs[:, 2] < 0
    t_best[down] = -sensor[2] / dirs[down, 2]
    for _ in range(40):
        fx, fy, h = rng.uniform(1, 5), rng.uniform(1, 3), rng.uniform(1, 3)
        r = np.sqrt(rng.uniform(3.0 ** 2, 50.0 ** 2))
        th = rng.uniform(0, 2 * np.pi)
        c = np.array([r * np.cos(th), r * np.sin(th)])
        lo = np.array([c[0] - fx / 2, c[1] - fy / 2, 0.0])
        hi = np.array([c[0] + fx / 2, c[1] + fy / 2, h])
        with np.errstate(divide="ignore", invalid="ignore"):
            t1 = (lo - sensor) / dirs
            t2 = (hi - sensor) / dirs
        tn = np.nanmax(np.minimum(t1, t2), axis=1)
        tf = np.nanmin(np.maximum(t1, t2), axis=1)
        hit = (tn <= tf) & (tf > 0)
        t = np.where(tn > 0, tn, tf)
        t_best = np.where(hit & (t < t_best), t, t_best)
    ok = np.isfinite(t_best) & (t_best <= max_range) & (rng.random(dirs.shape[0]) < keep)
    pts = sensor + dirs[ok] * t_best[ok, None]
    return np.ascontiguousarray(pts.astype(np.float32))


def ragged_batch(clouds):
    """Concatenate clouds: ``(points (sum N,3) f32, sample_inds int64, sample_sizes int64)``."""
    sizes = np.array([c.shape[0] for c in clouds], dtype=np.int64)
    points = np.concatenate(clouds).astype(np.float32)
    inds = np.repeat(np.arange(len(clouds), dtype=np.int64), sizes)
    return points, inds, sizes
