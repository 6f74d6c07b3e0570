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
