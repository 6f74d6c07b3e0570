"""Benchmark-size parity: all three passes of the convolution against the fp64 oracle.

The small-shape suites compare whole results; here the rulebooks have 0.9 M (the benchmark's
150k-point scene, 64 channels) and more than 1 M triplets (a 200k-point scene, 256 channels), so
that the persistent schedules of the tensor kernels (block ranges per CTA, ticket order, several
accumulator groups per CTA) are exercised at the sizes the measurements are taken at.  The oracle
is the tap-grouped fp64 restatement (``oracle/sparse_ops.py``); for the wide case it is evaluated
on a sample of output rows / taps, which keeps the CPU time to seconds.  Tolerance: relative
Frobenius error below 2e-2 for bf16 inputs (tests/unittest/test_tig_forward.py:127-135 of the
reference).
"""
import numpy as np
import pytest
import torch

from oracle import sparse_ops as oso

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _scene_rulebook(n_points, seed):
    from pointelligence_b200.layers.triplets import build_triplets_segmented
    from pointelligence_b200.synthetic import indoor_scene

    dev = torch.device("cuda:0")
    pts = torch.from_numpy(indoor_scene(n_points, seed)).to(dev)
    n = pts.shape[0]
    s = torch.zeros(n, dtype=torch.int64, device=dev)
    i, j, k, seg, _ = build_triplets_segmented(pts, s, torch.tensor([n], device=dev), 0.05, 3,
                                               return_num_neighbors=True, radius_scaler=2.5)
    return n, i, j, k, seg


def _operands(n, C, seed):
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, C, device=dev, generator=g).bfloat16()
    go = torch.randn(n, C, device=dev, generator=g).bfloat16()
    w = ((torch.rand(27, 1, C, C, device=dev, generator=g) * 2 - 1) / np.sqrt(C * 27)).bfloat16()
    return x, go, w


def _np64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def test_three_passes_150k_scene_64_channels_against_oracle():
    from pointelligence_b200 import _cabi
    from pointelligence_b200.sparse_engines.tig import TigIndex, tig_forward, tig_grad_input, tig_grad_weight

    n, i, j, k, seg = _scene_rulebook(150000, 0)
    assert i.numel() == 896518
    x, go, w = _operands(n, 64, 1)
    idx = TigIndex.from_flat(i, j, seg, n, n, 27)
    i_n, j_n, seg_n = i.cpu().numpy(), j.cpu().numpy(), seg.cpu().numpy()
    wn = _np64(w)

    y = tig_forward(w, x, idx)
    assert oso.rel_frobenius(_np64(y), oso.mvmr_f64_taps(wn, seg_n, _np64(x), j_n, i_n, n)) < TOL_BF16
    gx = tig_grad_input(w, go, idx)
    ref = oso.mvmr_f64_taps(np.swapaxes(wn, 2, 3), seg_n, _np64(go), i_n, j_n, n)
    assert oso.rel_frobenius(_np64(gx), ref) < TOL_BF16
    gw = tig_grad_weight(x, go, idx, w.shape)
    ref = oso.vvor_f64_taps(_np64(x), j_n, _np64(go), i_n, seg_n)
    assert oso.rel_frobenius(_np64(gw)[:, 0], ref) < TOL_BF16
    # every engine of the library agrees with the oracle at this size
    for engine in (_cabi.ENGINE_TENSOR,):
        y2 = _cabi.mvmr(w, x, j, i, seg, None, n, False, engine=engine)
        assert oso.rel_frobenius(_np64(y2), oso.mvmr_f64_taps(wn, seg_n, _np64(x), j_n, i_n, n)) < TOL_BF16
    assert _cabi.device_status() == 0


def test_three_passes_200k_scene_256_channels_against_sampled_oracle():
    from pointelligence_b200 import _cabi
    from pointelligence_b200.sparse_engines.tig import TigIndex, tig_forward, tig_grad_input, tig_grad_weight

    n, i, j, k, seg = _scene_rulebook(200000, 1)
    assert i.numel() >= 1_000_000
    x, go, w = _operands(n, 256, 2)
    idx = TigIndex.from_flat(i, j, seg, n, n, 27)
    i_n, j_n, seg_n = i.cpu().numpy(), j.cpu().numpy(), seg.cpu().numpy()
    wn = _np64(w)
    rows = np.unique(np.random.default_rng(0).integers(0, n, 4096))   # includes rows of every block range
    rows = np.union1d(rows, np.arange(n - 300, n))                     # and the ragged last block

    y = tig_forward(w, x, idx)
    ref = oso.mvmr_f64_taps(wn, seg_n, _np64(x), j_n, i_n, n, rows=rows)
    assert oso.rel_frobenius(_np64(y)[rows], ref) < TOL_BF16
    gx = tig_grad_input(w, go, idx)
    ref = oso.mvmr_f64_taps(np.swapaxes(wn, 2, 3), seg_n, _np64(go), i_n, j_n, n, rows=rows)
    assert oso.rel_frobenius(_np64(gx)[rows], ref) < TOL_BF16
    gw = tig_grad_weight(x, go, idx, w.shape)
    taps = [0, 13, 26]
    ref = oso.vvor_f64_taps(_np64(x), j_n, _np64(go), i_n, seg_n, taps=taps)
    assert oso.rel_frobenius(_np64(gw)[taps, 0], ref) < TOL_BF16
    # a checksum over ALL rows: the column sums of the forward equal those of the oracle's
    # per-tap products, which need no scatter
    colsum = np.zeros(256)
    xs = _np64(x)
    for t in range(27):
        lo, hi = int(seg_n[t]), int(seg_n[t + 1])
        colsum += xs[j_n[lo:hi]].sum(0) @ wn[t, 0]
    got = _np64(y).sum(0)
    assert np.linalg.norm(got - colsum) / np.linalg.norm(colsum) < TOL_BF16
    assert _cabi.device_status() == 0
