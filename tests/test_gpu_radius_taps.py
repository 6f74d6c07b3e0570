"""The one-hand-over tap-segmented search (``pcx_radius_taps_*``) against the two-call search
(``pcx_radius_count`` + ``pcx_radius_fill``), which the golden vectors and the oracle pin elsewhere.

The two paths bin the points differently (hashed buckets against injective cell keys), walk the
candidates differently (one lane per cell against one warp per query) and place the pairs
differently (direct tap-major placement against a radix sort by tap), so bit-equal ``i, j, k``,
segment offsets and neighbour counts on the same inputs is a strong check of each.  Cases: both
distances, kernel sizes 3 and 5, batched samples with separate queries, negative coordinates,
a run far longer than the 64-candidate mask (identical points), the boundary shell of pairs within
3 ulp of the radius under all three predicate roundings, and the capacity protocol of the C ABI.
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(pts, qry, ps, qs, radius, k, grid, dt=0):
    from pointelligence_b200 import _cabi

    old = os.environ.get("PCX_RADIUS_TAPS")
    try:
        os.environ["PCX_RADIUS_TAPS"] = "0"
        ref = _cabi.radius_search(pts, qry, radius, ps, qs, dt, k, grid, want_k=True)
        os.environ["PCX_RADIUS_TAPS"] = "1"
        got = _cabi.radius_search(pts, qry, radius, ps, qs, dt, k, grid, want_k=True)
    finally:
        if old is None:
            os.environ.pop("PCX_RADIUS_TAPS", None)
        else:
            os.environ["PCX_RADIUS_TAPS"] = old
    return ref, got


def _assert_same(ref, got):
    for name, a, b in zip(("i", "j", "k", "seg_offs", "num_neighbors"), ref, got):
        assert a.dtype == b.dtype and a.shape == b.shape, name
        assert torch.equal(a, b), name


@pytest.mark.parametrize("n,radius,k,dt", [(60000, 0.05, 3, 0), (60000, 0.05, 3, 1), (20000, 0.08, 5, 0),
                                           (20000, 0.08, 5, 1), (37, 0.3, 3, 0), (1, 0.1, 3, 0)])
def test_scene_equals_two_call_search(n, radius, k, dt):
    from pointelligence_b200 import _cabi
    from pointelligence_b200.synthetic import indoor_scene

    dev = torch.device("cuda:0")
    torch.manual_seed(n)
    pts = torch.from_numpy(indoor_scene(n, 1)).to(dev) if n > 100 else torch.rand(n, 3, device=dev)
    grid = radius / 2.5 if k == 3 else radius / 4.5
    _cabi._TAPS_RATIO.clear()
    ref, got = _both(pts, pts, None, None, radius, k, grid, dt)       # counted first call
    _assert_same(ref, got)
    assert got[0].numel() == int(got[4].sum())
    ref, got = _both(pts, pts, None, None, radius, k, grid, dt)       # estimated capacity
    _assert_same(ref, got)


def test_batched_samples_separate_queries_and_capacity_retry():
    from pointelligence_b200 import _cabi
    from pointelligence_b200.synthetic import indoor_scene

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    pts = torch.cat([torch.from_numpy(indoor_scene(30000, s)) for s in range(3)]).to(dev)
    smp = torch.arange(3, device=dev).repeat_interleave(30000)
    qi = torch.randperm(pts.shape[0], device=dev)[:40000].sort().values
    qry, qs = pts[qi] + 0.003 * torch.randn(40000, 3, device=dev), smp[qi]
    _cabi._TAPS_RATIO.clear()
    _assert_same(*_both(pts, qry, smp, qs, 0.05, 3, 0.02))
    # every sample holds the same coordinates: a query's bucket mixes the three samples
    same = torch.from_numpy(indoor_scene(20000, 7)).to(dev).repeat(3, 1)
    smp3 = torch.arange(3, device=dev).repeat_interleave(20000)
    ref, got = _both(same, same, smp3, smp3, 0.05, 3, 0.02)
    _assert_same(ref, got)
    assert bool((smp3[got[0].long()] == smp3[got[1].long()]).all())
    # an estimate that is far too small: the wrapper retries the fill pass with the exact size
    _cabi._TAPS_RATIO[(3, 0, 0.05)] = 0.01
    _assert_same(*_both(pts, qry, smp, qs, 0.05, 3, 0.02))
    assert _cabi._TAPS_RATIO[(3, 0, 0.05)] > 1.0


def test_long_runs_and_negative_coordinates():
    from pointelligence_b200 import _cabi
    from pointelligence_b200.synthetic import indoor_scene

    dev = torch.device("cuda:0")
    _cabi._TAPS_RATIO.clear()
    same = torch.zeros(1500, 3, device=dev) + 0.5              # one bucket, 1500 candidates per lane
    ref, got = _both(same, same, None, None, 0.05, 3, 0.02)
    _assert_same(ref, got)
    assert got[0].numel() == 1500 * 1500
    _cabi._TAPS_RATIO.clear()
    neg = torch.from_numpy(indoor_scene(50000, 3)).to(dev) - 5.0
    _assert_same(*_both(neg, neg, None, None, 0.05, 3, 0.02))


def test_boundary_shell_all_predicate_roundings():
    from pointelligence_b200 import _cabi

    dev = torch.device("cuda:0")
    rng = np.random.default_rng(0)
    nq, per, radius = 2048, 64, 0.05
    q = (rng.random((nq, 3)) * 50).astype(np.float32)
    d = rng.standard_normal((nq, per, 3))
    d /= np.linalg.norm(d, axis=-1, keepdims=True)
    scale = radius * (1 + rng.integers(-3, 4, (nq, per, 1)) * 2.0 ** -24)
    p = (q[:, None, :].astype(np.float64) + d * scale).astype(np.float32).reshape(-1, 3)
    qt, pt = torch.from_numpy(q).to(dev), torch.from_numpy(p).to(dev)
    totals = []
    try:
        for variant in (0, 1, 2):
            _cabi.check(_cabi.lib().pcx_set_radius_predicate(variant))
            _cabi._TAPS_RATIO.clear()
            ref, got = _both(pt, qt, None, None, radius, 3, 0.02)
            _assert_same(ref, got)
            totals.append(got[0].numel())
    finally:
        _cabi.check(_cabi.lib().pcx_set_radius_predicate(1))
    assert 0 < totals[1] < nq * per and totals[0] != totals[1]   # the shell separates the roundings


def test_c_abi_capacity_protocol_and_argument_errors():
    from pointelligence_b200 import _cabi
    from pointelligence_b200._cabi import c_int64, ptr, stream_ptr, workspace
    from pointelligence_b200.synthetic import indoor_scene

    dev = torch.device("cuda:0")
    L = _cabi.lib()
    pts = torch.from_numpy(indoor_scene(5000, 2)).to(dev)
    n = pts.shape[0]
    assert L.pcx_radius_taps_supported(3) == 1 and L.pcx_radius_taps_supported(5) == 1
    assert L.pcx_radius_taps_supported(7) == 0 and L.pcx_radius_taps_supported(4) == 0
    assert L.pcx_radius_taps_workspace_bytes(n, n, 7) == 0
    ws = workspace(L.pcx_radius_taps_workspace_bytes(n, n, 3), dev)
    nn = torch.empty(n, dtype=torch.int64, device=dev)
    seg = torch.empty(28, dtype=torch.int64, device=dev)
    args = (ptr(pts), ptr(pts), None, None, n, n, 0.05, 0, 3, 0.02, ptr(nn), ptr(seg))
    assert L.pcx_radius_taps_count(*args, ptr(ws), 128, stream_ptr()) == _cabi.PCX_E_CAPACITY   # workspace too small
    assert L.pcx_radius_taps_count(ptr(pts), ptr(pts), None, None, n, n, -1.0, 0, 3, 0.02, ptr(nn), ptr(seg),
                                   ptr(ws), ws.numel(), stream_ptr()) == -1                    # PCX_E_ARG
    assert L.pcx_radius_taps_count(ptr(pts), ptr(pts), None, None, n, n, 0.05, 0, 7, 0.02, ptr(nn), ptr(seg),
                                   ptr(ws), ws.numel(), stream_ptr()) == -6                    # PCX_E_UNSUPPORTED
    _cabi.check(L.pcx_radius_taps_count(*args, ptr(ws), ws.numel(), stream_ptr()))
    total = (c_int64 * 3)()
    _cabi.check(L.pcx_radius_taps_total(n, n, 3, total, ptr(ws), ws.numel(), stream_ptr()))
    t = int(total[0])
    assert t == int(nn.sum()) and int(seg[-1]) == t and int(total[1]) == 0
    small = torch.full((t - 1,), -7, dtype=torch.int32, device=dev)
    got = (c_int64 * 3)()
    rc = L.pcx_radius_taps_fill(ptr(pts), None, None, n, n, 0.05, 0, 3, 0.02, t - 1, ptr(small), ptr(small), None,
                                got, ptr(ws), ws.numel(), stream_ptr())
    assert rc == _cabi.PCX_E_CAPACITY and int(got[0]) == t
    assert bool((small == -7).all())                         # nothing was written
    oi = torch.empty(t, dtype=torch.int32, device=dev)
    oj = torch.empty_like(oi)
    _cabi.check(L.pcx_radius_taps_fill(ptr(pts), None, None, n, n, 0.05, 0, 3, 0.02, t, ptr(oi), ptr(oj), None,
                                       got, ptr(ws), ws.numel(), stream_ptr()))
    os.environ["PCX_RADIUS_TAPS"] = "0"
    try:
        ref = _cabi.radius_search(pts, pts, 0.05, None, None, 0, 3, 0.02, want_k=False)
    finally:
        os.environ.pop("PCX_RADIUS_TAPS", None)
    assert torch.equal(oi, ref[0]) and torch.equal(oj, ref[1])
    # queries with no neighbour are counted for the caller
    far = torch.cat([pts[:100], pts[:7] + 100.0])
    ws = workspace(L.pcx_radius_taps_workspace_bytes(n, 107, 3), dev)
    nn = torch.empty(107, dtype=torch.int64, device=dev)
    _cabi.check(L.pcx_radius_taps_count(ptr(pts), ptr(far), None, None, n, 107, 0.05, 0, 3, 0.02, ptr(nn), ptr(seg),
                                        ptr(ws), ws.numel(), stream_ptr()))
    _cabi.check(L.pcx_radius_taps_total(n, 107, 3, total, ptr(ws), ws.numel(), stream_ptr()))
    assert int(total[1]) == 7 and int((nn == 0).sum()) == 7


def test_builder_raises_for_a_query_without_neighbour():
    from pointelligence_b200.layers.triplets import build_triplets_segmented
    from pointelligence_b200.synthetic import indoor_scene

    dev = torch.device("cuda:0")
    pts = torch.from_numpy(indoor_scene(3000, 4)).to(dev)
    smp = torch.zeros(3000, dtype=torch.int64, device=dev)
    qry = torch.cat([pts[:50], pts[:1] + 100.0])
    qsm = torch.zeros(51, dtype=torch.int64, device=dev)
    with pytest.raises(AssertionError):
        build_triplets_segmented(pts, smp, torch.tensor([3000], device=dev), 0.05, 3, query_points=qry,
                                 query_sample_inds=qsm, query_sample_sizes=torch.tensor([51], device=dev),
                                 radius_scaler=2.5)


def test_tap_ties_on_a_half_grid_lattice():
    """Points on a lattice of half the tap grid: every offset divided by the tap grid is an integer
    or a half-integer, the round-half-even cases the division-free tap computation must hand to
    the exact division."""
    from pointelligence_b200 import _cabi

    dev = torch.device("cuda:0")
    g = 0.02
    axis = torch.arange(24, device=dev, dtype=torch.float32) * (g / 2)
    pts = torch.cartesian_prod(axis, axis, axis).contiguous()
    pts = pts + torch.tensor([0.3, -0.2, 1.7], device=dev)          # lattice offsets that are not representable exactly
    for k, radius in ((3, 0.05), (5, 0.045)):
        _cabi._TAPS_RATIO.clear()
        ref, got = _both(pts, pts, None, None, radius, k, g)
        _assert_same(ref, got)
        assert got[0].numel() > 20 * pts.shape[0]
