"""GPU tests of the output-stationary MVMR engine (``pcx_mvmr_plan_build`` + ``pcx_mvmr_planned``).

The plan is compared bit for bit with its numpy restatement (``oracle/mvmr_plan.py``); the
convolution (forward and, with the roles swapped, the input gradient) with the fp64 oracle within
the reference's bounds (relative Frobenius error 2e-2 for bf16, 2e-3 for fp16:
tests/unittest/test_tig_forward.py:127-135), over channel counts that exercise one and several
64-channel slices, partial slices, both ways of loading the weight tiles, one and two CTAs per
SM, many taps, a single tap, empty taps, rows and whole blocks without triplets, buckets with
several triplets, and an empty rulebook.  Launching twice from one plan must give identical bits
(the plan's work counter re-arms itself).
"""
import os

import numpy as np
import pytest
import torch

from oracle import mvmr_plan as omp
from oracle import sparse_ops as oso

pytestmark = pytest.mark.gpu
TOL = {torch.float16: 2e-3, torch.bfloat16: 2e-2}
DEV = "cuda:0"


def _rulebook(seed, n_in, n_out, K, T, dup=0.2, skip_tap=None):
    rng = np.random.default_rng(seed)
    i = rng.integers(0, n_out, T)
    j = rng.integers(0, n_in, T)
    k = rng.integers(0, K, T)
    nd = int(T * dup)          # repeat (row, tap) pairs: buckets with several triplets
    if nd:
        src = rng.integers(0, T, nd)
        i[:nd], k[:nd] = i[src], k[src]
    if skip_tap is not None and K > 1:
        k[k == skip_tap] = (skip_tap + 1) % K
    order = np.lexsort((i, k))
    i, j, k = i[order], j[order], k[order]
    seg = np.searchsorted(k, np.arange(K + 1))
    return i.astype(np.int32), j.astype(np.int32), k.astype(np.int32), seg.astype(np.int64)


def _t(x):
    return torch.as_tensor(x).to(DEV)


def _check_plan(plan, i, j, k, n_out, K):
    want = omp.build(i, j, k, n_out, K)
    v = plan.views()
    assert np.array_equal(v["perm"].cpu().numpy(), want["perm"])
    assert np.array_equal(v["tile_offs"].cpu().numpy(), want["tile_offs"])
    ent = v["entries"].cpu().numpy().astype(np.int64) & 0xFFFFFFFF
    assert np.array_equal(ent[:, 0] & 127, want["slot"])
    assert np.array_equal(ent[:, 0] >> 8, want["pos"])
    assert np.array_equal(ent[:, 1], want["rows"])
    heads = np.flatnonzero(want["pos"] == 0)
    lens = np.diff(np.concatenate((heads, [len(want["pos"])])))
    table = v["tile_rows"].cpu().numpy().reshape(-1)
    single, multi = heads[lens == 1], heads[lens > 1]
    assert np.array_equal(table[want["key"][single]], want["rows"][single])
    assert np.all(table[want["key"][multi]] <= -2) and (table != -1).sum() == len(heads)
    assert plan.multi_buckets == len(multi)
    buckets = v["buckets"].cpu().numpy()
    by_start = buckets[np.argsort(buckets[:, 0])] if len(multi) else buckets
    assert np.array_equal(by_start[:, 0], multi) and np.array_equal(by_start[:, 1], lens[lens > 1])
    G = plan.group_blocks
    nb = want["nblocks"]
    ng = (nb + G - 1) // G
    tiles = np.diff(want["tile_offs"]) > 0
    cost = np.concatenate((tiles, np.zeros(ng * G * K - nb * K, bool))).reshape(ng, G * K).sum(1)
    order = v["group_order"].cpu().numpy()
    assert sorted(order.tolist()) == list(range(ng)) and np.all(np.diff(cost[order]) <= 0)


CASES = [
    # name, n_in, n_out, K, T, C, M, dtype, transpose
    ("c64", 5000, 4000, 27, 40000, 64, 64, torch.bfloat16, 0),
    ("c64_dgrad_f16", 5000, 4000, 27, 40000, 64, 64, torch.float16, 1),
    ("c128", 3000, 3000, 27, 30000, 128, 128, torch.bfloat16, 0),
    ("c128_dgrad", 3000, 3000, 27, 30000, 128, 128, torch.bfloat16, 1),
    ("c256", 3000, 2500, 27, 30000, 256, 256, torch.bfloat16, 0),
    ("c256_dgrad", 3000, 2500, 27, 30000, 256, 256, torch.bfloat16, 1),
    ("c64_to_128", 3000, 2500, 27, 30000, 64, 128, torch.bfloat16, 0),
    ("c64_to_128_dgrad", 3000, 2500, 27, 30000, 64, 128, torch.bfloat16, 1),
    ("c192_to_64", 2000, 2500, 27, 20000, 192, 64, torch.bfloat16, 0),
    ("c192_to_64_dgrad", 2000, 2500, 27, 20000, 192, 64, torch.bfloat16, 1),
    ("c384_to_96", 1500, 1500, 27, 12000, 384, 96, torch.bfloat16, 0),
    ("c32", 3000, 3000, 27, 30000, 32, 32, torch.bfloat16, 0),
    ("c48_to_96_dgrad", 3000, 3000, 27, 30000, 48, 96, torch.bfloat16, 1),
    ("c16_f16", 3000, 3000, 27, 30000, 16, 16, torch.float16, 0),
    ("taps125", 2000, 1500, 125, 30000, 64, 64, torch.bfloat16, 0),
    ("one_tap", 2000, 2000, 1, 2000, 64, 64, torch.bfloat16, 0),
    ("mostly_empty_rows", 1000, 5000, 27, 3000, 64, 64, torch.bfloat16, 0),
    ("tiny", 300, 200, 27, 1500, 64, 64, torch.bfloat16, 1),
    ("dense", 700, 600, 27, 30000, 64, 64, torch.bfloat16, 0),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_planned_engine_against_oracle(case, monkeypatch):
    from pointelligence_b200 import _cabi

    name, n_in, n_out, K, T, C, M, dtype, transpose = case
    i, j, k, seg = _rulebook(len(name), n_in, n_out, K, T, skip_tap=2)
    inw, outw = (M, C) if transpose else (C, M)
    rng = np.random.default_rng(1)
    w = _t(rng.standard_normal((K, 1, C, M)) / np.sqrt(inw)).to(dtype)
    x = _t(rng.standard_normal((n_in, inw))).to(dtype)
    G = _cabi.plan_group_blocks(outw)
    plan = _cabi.mvmr_plan(_t(i), _t(j), _t(seg), K, n_out, G)
    _check_plan(plan, i, j, k, n_out, K)
    wn = w.float().cpu().numpy().astype(np.float64)
    ref = oso.mvmr_f64_taps(np.swapaxes(wn, 2, 3) if transpose else wn, seg, x.float().cpu().numpy(), j, i, n_out)
    for weights_by_tma, ctas in (("1", "2"), ("0", "1")):
        monkeypatch.setenv("PCX_OS_WTMA", weights_by_tma)
        monkeypatch.setenv("PCX_OS_CTAS", ctas)
        out = _cabi.mvmr_planned(w, x, plan, transpose)
        again = _cabi.mvmr_planned(w, x, plan, transpose)
        assert out.shape == (n_out, outw) and out.dtype == dtype
        assert oso.rel_frobenius(out.float().cpu().numpy(), ref) < TOL[dtype], (name, weights_by_tma, ctas)
        assert torch.equal(out, again)
    untouched = np.setdiff1d(np.arange(n_out), i)
    if len(untouched):
        assert torch.all(out[_t(untouched)] == 0)
    assert _cabi.device_status() == 0


def _kernels_of(fn):
    """Labels of the dominant kernels the library launched during ``fn()``."""
    from pointelligence_b200 import _cabi

    _cabi.profile_enable(True)
    try:
        out = fn()
        torch.cuda.synchronize()
        names = [name for name, _ in _cabi.profile_records()]
    finally:
        _cabi.profile_enable(False)
    return out, names


def test_automatic_engine_takes_the_planned_kernel_for_dense_or_large_layers():
    from pointelligence_b200 import _cabi

    def close(a, b):   # the scatter engine adds in fp32 in an order that varies from run to run
        return float((a.float() - b.float()).norm() / b.float().norm()) < 1e-2

    i, j, k, seg = _rulebook(3, 900, 800, 27, 30000)          # 37 triplets per output row
    w = torch.randn(27, 1, 64, 64, device=DEV).bfloat16() / 8
    x = torch.randn(900, 64, device=DEV).bfloat16()
    ti, tj, tseg = _t(i), _t(j), _t(seg)
    auto, names = _kernels_of(lambda: _cabi.mvmr(w, x, tj, ti, tseg, None, 800, False))
    assert [n for n in names if n != "bucket_sum_kernel"] == ["mvmr_os_kernel(fwd)"]   # dense neighbourhood
    forced = _cabi.mvmr(w, x, tj, ti, tseg, None, 800, False, engine=_cabi.ENGINE_PLANNED)
    scatter, names = _kernels_of(lambda: _cabi.mvmr(w, x, tj, ti, tseg, None, 800, False, engine=_cabi.ENGINE_TENSOR))
    assert names == ["mvmr_tc_kernel(fwd)"] and torch.equal(auto, forced) and close(auto, scatter)
    i, j, k, seg = _rulebook(4, 4000, 4000, 27, 12000, dup=0.0)   # 3 triplets per row
    ti, tj, tseg = _t(i), _t(j), _t(seg)
    x = torch.randn(4000, 64, device=DEV).bfloat16()
    _, names = _kernels_of(lambda: _cabi.mvmr(w, x, tj, ti, tseg, None, 4000, False))
    assert names == ["mvmr_tc_kernel(fwd)"]                    # sparse and 64 channels wide: scatter engine
    # a large accumulator (n_out x width x 4 bytes beyond half of the L2) at four triplets per row and more
    assert _cabi._planned_pays(T=900_000, n_out=150_000, outw=128, K=27)
    assert not _cabi._planned_pays(T=900_000, n_out=150_000, outw=64, K=27)
    assert not _cabi._planned_pays(T=133_000, n_out=50_000, outw=256, K=27)      # too sparse
    assert _cabi._planned_pays(T=7_000_000, n_out=1_100_000, outw=32, K=27)
    assert not _cabi._planned_pays(T=1_100_000, n_out=1_100_000, outw=256, K=1)   # a single tap
    assert not _cabi._planned_pays(T=18_200_000, n_out=1_100_000, outw=32, K=125)  # 0.13 triplets per row and tap: tiles of padding
    with pytest.raises(NotImplementedError):                   # fp32 has no tensor-core engine
        _cabi.mvmr(w.float(), x.float(), tj, ti, tseg, None, 4000, False, engine=_cabi.ENGINE_PLANNED)


def test_planned_engine_empty_rulebook_and_argument_errors():
    from pointelligence_b200 import _cabi

    e = torch.empty(0, dtype=torch.int32, device=DEV)
    seg = torch.zeros(28, dtype=torch.int64, device=DEV)
    plan = _cabi.mvmr_plan(e, e, seg, 27, 300, 2)
    w = torch.randn(27, 1, 32, 32, device=DEV).bfloat16()
    x = torch.randn(10, 32, device=DEV).bfloat16()
    out = _cabi.mvmr_planned(w, x, plan, False)
    assert out.shape == (300, 32) and torch.all(out == 0)
    with pytest.raises(NotImplementedError):
        _cabi.mvmr_plan(e, e, seg, 27, 300, 9)                 # more blocks per group than the kernel has accumulators for
    L = _cabi.lib()
    assert L.pcx_mvmr_plan_bytes(10, 100, 27, 0) == 0 and L.pcx_mvmr_plan_bytes(10, 0, 27, 2) == 0
    assert L.pcx_mvmr_plan_group_blocks(64) == 2 and L.pcx_mvmr_plan_group_blocks(512) == 0
    bad = torch.randn(27, 1, 24, 32, device=DEV).bfloat16()    # 24 channels: not a multiple of 16
    with pytest.raises(NotImplementedError):
        _cabi.mvmr_planned(bad, torch.randn(10, 24, device=DEV).bfloat16(), plan, False)


def test_bounded_wait_that_runs_out_is_reported():
    """A kernel whose wait nobody answers gives up after its limit, returns by itself and leaves
    its bit in the device status word; reading the word clears it."""
    from pointelligence_b200 import _cabi

    assert _cabi.device_status() == 0
    _cabi.debug_wait_runs_out(1_000_000)                        # one millisecond
    torch.cuda.synchronize()
    assert _cabi.device_status() == 8
    assert _cabi.device_status() == 0
    # the host-side wrappers notice it at their next hand-over: the geometry stage raises
    from pointelligence_b200.internals.neighbors import radius_search_sorted_grid8

    _cabi.debug_wait_runs_out(1_000_000)
    pts = torch.rand(64, 3, device=DEV)
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        radius_search_sorted_grid8(pts, pts, 0.2)
    assert _cabi.device_status() == 0
    radius_search_sorted_grid8(pts, pts, 0.2)
    with pytest.raises(ValueError):
        _cabi.debug_wait_runs_out(10 ** 12)


def test_symmetric_rulebook_input_gradient_reuses_the_forward_plan(monkeypatch):
    """A self-search rulebook is its own mirror image, so the input gradient runs as a forward
    schedule over the same rulebook with reversed taps: same result as the separate transposed
    pass (and as the fp64 oracle), and no second plan is built."""
    from pointelligence_b200 import _cabi
    from pointelligence_b200.layers import PointConv3d
    from pointelligence_b200.layers.triplets import build_triplets_segmented
    from pointelligence_b200.synthetic import indoor_scene

    dev = torch.device("cuda:0")
    monkeypatch.setattr(_cabi, "_PLANNED_DENSE_RATIO", 0.0)      # every tap-sorted bf16 layer takes the planned engine
    monkeypatch.setattr(_cabi, "_PLANNED_MIN_TAP_FILL", 0.0)
    pts = torch.from_numpy(indoor_scene(20000, 9)).to(dev)
    n = pts.shape[0]
    smp = torch.zeros(n, dtype=torch.int64, device=dev)
    i, j, k, seg, _ = build_triplets_segmented(pts, smp, torch.tensor([n], device=dev), 0.05, 3, radius_scaler=2.5)
    assert _cabi.is_symmetric(i, j)
    key = lambda a, b, c: torch.sort(c.long() * n * n + a.long() * n + b.long()).values
    assert torch.equal(key(i, j, k), key(j, i, 26 - k))             # the mirror property itself
    torch.manual_seed(0)
    conv = PointConv3d(32, 64, kernel_size=3, bias=False).to(dev).to(torch.bfloat16)
    x0 = torch.randn(n, 32, device=dev).to(torch.bfloat16)
    go = torch.randn(n, 64, device=dev).to(torch.bfloat16)
    grads = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("PCX_SYMMETRIC_DGRAD", mode)
        _cabi._PLAN_CACHE.clear()
        x = x0.clone().requires_grad_(True)
        conv(x, i, j, k, n, seg_offs=seg).backward(go)
        grads[mode] = (x.grad.float(), len(_cabi._PLAN_CACHE))
    assert grads["1"][1] == 1 and grads["0"][1] == 2                 # one plan against two
    w = conv.weight.detach().double()[:, 0]
    want = torch.zeros(n, 32, dtype=torch.float64, device=dev)
    want.index_add_(0, j.long(), torch.einsum("tm,tcm->tc", go.double()[i.long()], w[k.long()]))
    for mode in ("1", "0"):
        err = (grads[mode][0].double() - want).norm() / want.norm()
        assert float(err) < 1e-2, (mode, float(err))
