"""GPU tests of the dense-tap schedule (one GEMM over all taps followed by the
per-output indexed sum): it agrees with the float64 oracle within the bf16 /
fp16 bounds (2e-2 / 2e-3 relative Frobenius) and with the scatter engine, for the
forward and the input gradient, and the automatic route takes it only for dense
neighbourhoods."""
import numpy as np
import pytest
import torch

from oracle import sparse_ops as oso

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 2e-3, torch.bfloat16: 2e-2}


def _t(x, dtype=None):
    t = torch.as_tensor(np.asarray(x)).to("cuda:0")
    return t.to(dtype) if dtype is not None else t


def _triplets(rng, K, n_in, n_out, T):
    k = np.sort(rng.integers(0, K, T))
    k = k[k != 2] if K > 2 else k
    i = rng.integers(0, n_out, len(k))
    i[i == 5] = 6                      # an output row without any triplet
    order = np.lexsort((i, k))
    return i[order].astype(np.int32), rng.integers(0, n_in, len(k)).astype(np.int32), k.astype(np.int32)


def test_output_lists_regroup_the_triplets_by_output_row():
    from pointelligence_b200 import _cabi

    rng = np.random.default_rng(0)
    K, n_in, n_out = 27, 300, 250
    i, j, k = _triplets(rng, K, n_in, n_out, 9000)
    seg = _cabi.seg_offs_from_sorted(_t(k), K)
    src, lengths = _cabi.output_lists(_t(i), _t(j), seg, K, n_out, n_in)
    order = np.argsort(i, kind="stable")
    assert np.array_equal(src.cpu().numpy(), (j.astype(np.int64) * K + k)[order])
    assert np.array_equal(lengths.cpu().numpy(), np.bincount(i, minlength=n_out))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("K,C,M", [(27, 64, 64), (27, 192, 128), (27, 256, 256), (125, 16, 32), (1, 96, 32), (27, 24, 40)])
def test_dense_tap_schedule_matches_oracle_and_scatter_engine(dtype, K, C, M):
    from pointelligence_b200 import _cabi

    rng = np.random.default_rng(K + C + M)
    n_in, n_out, T = 700, 900, 30000
    i, j, k = _triplets(rng, K, n_in, n_out, T)
    w = _t(rng.standard_normal((K, 1, C, M)) / np.sqrt(C), dtype)
    x = _t(rng.standard_normal((n_in, C)), dtype)
    go = _t(rng.standard_normal((n_out, M)), dtype)
    ti, tj = _t(i), _t(j)
    seg = _cabi.seg_offs_from_sorted(_t(k), K)
    assert _cabi.dense_taps_applies(w, x, tj, ti, seg, n_out)            # 30000 triplets over 700 rows
    out = _cabi.mvmr_dense_taps(w, x, tj, ti, seg, n_out, False)
    gx = _cabi.mvmr_dense_taps(w, go, ti, tj, seg, n_in, True)
    wn, xn, gn = (t.float().cpu().numpy().astype(np.float64) for t in (w, x, go))
    ref = oso.mvmr_f64(wn, k, xn[:, None, :], j, i, n_out)[:, 0]
    assert oso.rel_frobenius(out.float().cpu().numpy(), ref) < TOL[dtype]
    assert torch.all(out[5] == 0)
    ref_t = oso.mvmr_f64(np.swapaxes(wn, 2, 3), k, gn[:, None, :], i, j, n_in)[:, 0]
    assert oso.rel_frobenius(gx.float().cpu().numpy(), ref_t) < TOL[dtype]
    if C % 16 == 0 and M % 16 == 0:
        scat = _cabi.mvmr(w, x, tj, ti, seg, None, n_out, False, _cabi.ENGINE_TENSOR)
        assert oso.rel_frobenius(out.float().cpu().numpy(), scat.float().cpu().numpy()) < TOL[dtype]


def test_automatic_route_keeps_sparse_neighbourhoods_on_the_scatter_engine():
    from pointelligence_b200 import _cabi

    rng = np.random.default_rng(9)
    K, C, M, n = 27, 64, 64, 4000
    i, j, k = _triplets(rng, K, n, n, 24000)        # 6 triplets per row, like the headline scene
    w = _t(rng.standard_normal((K, 1, C, M)) / 8, torch.bfloat16)
    x = _t(rng.standard_normal((n, C)), torch.bfloat16)
    seg = _cabi.seg_offs_from_sorted(_t(k), K)
    assert not _cabi.dense_taps_applies(w, x, _t(j), _t(i), seg, n)
    assert not _cabi.dense_taps_applies(w.float(), x.float(), _t(j), _t(i), seg, n)


def test_pointconv3d_on_a_dense_cloud_takes_the_dense_tap_schedule_and_matches_the_oracle():
    """End to end through the layer API: a cloud with about 30 neighbours per point (more than
    the 27 taps) runs forward and input gradient on the dense-tap schedule, the weight gradient
    on the tensor kernel, and all three agree with the float64 oracle on the reference's
    triplets (bf16 bound 2e-2)."""
    from oracle import geometry as og
    from pointelligence_b200 import _cabi
    from pointelligence_b200.layers import MetaData, PointConv3d, conv_with_stride

    rng = np.random.default_rng(21)
    pts = (rng.random((6000, 3)) * 0.5).astype(np.float32)          # 6000 points in a 0.5 m cube
    n, C, M = len(pts), 64, 32
    dev = "cuda:0"
    conv = PointConv3d(C, M, 3, bias=False, device=dev, dtype=torch.bfloat16)
    x = torch.randn(n, C, device=dev).bfloat16().requires_grad_(True)
    m = MetaData(points=_t(pts), sample_inds=torch.zeros(n, dtype=torch.int64, device=dev),
                 sample_sizes=torch.tensor([n], device=dev), grid_size=0.02)
    _cabi.profile_enable(True)
    y, m = conv_with_stride(conv, x, m, 1, receptive_field_scaler=2.5)
    go = torch.randn_like(y)
    y.backward(go)
    torch.cuda.synchronize()
    names = [name for name, _ in _cabi.profile_records()]
    _cabi.profile_enable(False)
    T = int(m.i.numel())
    assert T >= 12 * n, (T, n)
    assert names.count("idx_reduce_kernel") == 2 and "vvor_tc_kernel" in names, names
    assert not any(name.startswith("mvmr_tc_kernel") for name in names), names
    rs = og.radius_scaler_for_kernel_size(3, 2.5)
    oi, oj, oseg, _ = og.radius_search_sorted_grid8_segments(pts, pts, 0.02 * rs, 3, 0.02, fma=True)
    ok = np.repeat(np.arange(27), np.diff(oseg)).astype(np.int32)
    assert np.array_equal(og.canonical_triplet_keys(m.i.cpu().numpy(), m.j.cpu().numpy(), m.k.cpu().numpy(), n, n),
                          og.canonical_triplet_keys(oi, oj, ok, n, n))
    wn = conv.weight.detach().float().cpu().numpy().astype(np.float64)
    xn = x.detach().float().cpu().numpy().astype(np.float64)
    gn = go.float().cpu().numpy().astype(np.float64)
    ref = oso.mvmr_f64(wn, ok, xn[:, None, :], oj, oi, n)[:, 0]
    assert oso.rel_frobenius(y.detach().float().cpu().numpy(), ref) < 2e-2
    ref_gx = oso.mvmr_f64(np.swapaxes(wn, 2, 3), ok, gn[:, None, :], oi, oj, n)[:, 0]
    assert oso.rel_frobenius(x.grad.float().cpu().numpy(), ref_gx) < 2e-2
    ref_gw = oso.vvor_f64(xn[:, None, :], oj, gn[:, None, :], oi, ok, 27)
    assert oso.rel_frobenius(conv.weight.grad.float().cpu().numpy(), ref_gw) < 2e-2
