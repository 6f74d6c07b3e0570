"""CPU checks of the rulebook plan's restatement (``oracle/mvmr_plan.py``) and of the host-side
engine choice: no GPU, no library call."""
import numpy as np

from oracle import geometry as og
from oracle import mvmr_plan as omp


def _surface_rulebook(n=40_000, seed=0, grid=0.02):
    """Self-search rulebook of a synthetic indoor scene (floor, walls, furniture: points on surfaces),
    27 taps on the convolution's own tap grid, tap-major and ascending row inside a tap."""
    from scipy.spatial import cKDTree

    from pointelligence_b200.synthetic import indoor_scene

    pts = og.grid_sample_center_nearest(indoor_scene(n, seed), grid)[0]
    radius = grid * og.radius_scaler_for_kernel_size(3, 2.5)
    pairs = cKDTree(pts).query_pairs(radius, output_type="ndarray")
    own = np.arange(len(pts))
    i = np.concatenate([pairs[:, 0], pairs[:, 1], own])
    j = np.concatenate([pairs[:, 1], pairs[:, 0], own])
    k = og.tap_index(pts[j], pts[i], grid, 3)
    order = np.lexsort((j, i, k))
    return i[order], j[order], k[order], len(pts)


def _tiles(perm, scatter, tap, K):
    """Non-empty (block of 128 rows, tap) tiles under the row order ``perm``."""
    rank = np.empty(len(perm), np.int64)
    rank[perm] = np.arange(len(perm))
    return len(np.unique((rank[scatter] >> 7) * K + tap))


def test_plane_order_of_the_plan_rows_needs_fewer_tiles_than_the_signature_alone():
    i, j, k, n = _surface_rulebook()
    plan = omp.build(i, j, k, n, 27)
    perm = plan["perm"][:n]
    assert sorted(perm.tolist()) == list(range(n))                       # a permutation of the rows
    sig = np.zeros(n, np.int64)
    np.bitwise_or.at(sig, i, 1 << k)
    by_signature = np.argsort(sig, kind="stable")
    ours, before, own = _tiles(perm, i, k, 27), _tiles(by_signature, i, k, 27), _tiles(np.arange(n), i, k, 27)
    assert ours == int((np.diff(plan["tile_offs"]) > 0).sum())          # what the plan itself says
    assert ours < 0.85 * before and before < 0.5 * own, (ours, before, own)   # measured: 1480, 1996, 7462


def test_plan_is_a_regrouping_of_the_rulebook():
    i, j, k, n = _surface_rulebook(n=6000, seed=1)
    plan = omp.build(i, j, k, n, 27)
    assert plan["tile_offs"][-1] == len(i) and np.all(np.diff(plan["tile_offs"]) >= 0)
    # every triplet appears once: the multiset of (output row, source row, tap) survives the regrouping
    perm = plan["perm"]
    key = plan["key"]
    rows_out = perm[(key >> 7) // 27 * 128 + (key & 127)]
    got = np.stack([rows_out, plan["rows"], (key >> 7) % 27], 1)
    want = np.stack([i, j, k], 1)
    assert np.array_equal(got[np.lexsort(got.T[::-1])], want[np.lexsort(want.T[::-1])])
    # a single tap or more than 32 taps: rows by signature only
    one = omp.build(i, j, np.zeros_like(k), n, 1)
    assert np.array_equal(one["perm"][:n], np.arange(n))                # every row has the same signature: stable order


def test_engine_choice_rules():
    from pointelligence_b200 import _cabi

    pays = _cabi._planned_pays
    assert pays(T=12_500_000, n_out=375_000, outw=256, K=27)            # dense neighbourhoods
    assert pays(T=900_000, n_out=150_000, outw=128, K=27)               # large accumulator, 6 triplets per row
    assert not pays(T=900_000, n_out=150_000, outw=64, K=27)            # the accumulator fits half of the L2
    assert not pays(T=18_200_000, n_out=1_100_000, outw=32, K=125)      # thin in tap space
    assert not pays(T=1_100_000, n_out=1_100_000, outw=256, K=1)        # a single tap
