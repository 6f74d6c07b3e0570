"""The grid-partition (patchify) strided convolution: properties the reference tests
(``tests/unittest/test_conv_with_stride_disjoint_parity.py``: full coverage, bounded slots, tokens
at cell centres, the cached edges as the exact inverse), the rulebook against the numpy oracle, and
the convolution through the library against a dense fp64 evaluation of the same rulebook."""
import numpy as np
import pytest
import torch

from oracle import geometry as ogeo

pytestmark = pytest.mark.gpu


def _meta(n=20000, scale=4.0, g0=0.02, nbatch=1, seed=0):
    from pointelligence_b200.layers.metadata import MetaData

    gen = torch.Generator(device="cuda").manual_seed(seed)
    pts = torch.rand(n, 3, device="cuda", generator=gen) * scale - scale / 3     # negative coordinates too
    si = torch.randint(0, nbatch, (n,), device="cuda", generator=gen).sort().values
    return MetaData(points=pts, sample_inds=si, sample_sizes=torch.bincount(si, minlength=nbatch), grid_size=g0)


@pytest.mark.parametrize("nbatch,K", [(1, 8), (3, 8), (2, 4)])
def test_partition_properties(nbatch, K):
    from pointelligence_b200.layers.triplets import handle_stride_disjoint_and_build_triplets

    m = _meta(nbatch=nbatch)
    n, g0 = m.points.shape[0], m.grid_size
    parent_points = m.points
    m = handle_stride_disjoint_and_build_triplets(m, stride=K, kernel_size=K)
    assert m.j.numel() == n and torch.unique(m.j).numel() == n                    # one edge per point, none orphaned
    assert torch.unique(m.parent.i_upsample).numel() == n
    assert int(m.k.min()) >= 0 and int(m.k.max()) < K ** 3
    assert bool((m.k[1:] >= m.k[:-1]).all()) and int(m.seg_offs[-1]) == n         # grouped by slot
    cell = g0 * K
    frac = m.points / cell - torch.floor(m.points / cell)
    assert torch.allclose(frac, torch.full_like(frac, 0.5), atol=1e-4)            # tokens at cell centres
    inside = (parent_points[m.j] - m.points[m.i]).abs().max()
    assert float(inside) <= cell / 2 * (1 + 1e-4)                                  # every point lies in its token's cell
    assert bool((m.sample_inds[m.i] == m.parent.sample_inds[m.j]).all())
    assert m.contract.k_sorted and m.contract.exact_cover_in and not m.contract.exact_cover_out
    with pytest.raises(ValueError):
        handle_stride_disjoint_and_build_triplets(_meta(), stride=1, kernel_size=4)
    with pytest.raises(ValueError):
        handle_stride_disjoint_and_build_triplets(_meta(), stride=4, kernel_size=(4, 4, 2))


def test_partition_rulebook_matches_oracle():
    from pointelligence_b200.layers.triplets import handle_stride_disjoint_and_build_triplets

    K = 8
    m = _meta(n=6000, nbatch=2, seed=3)
    pts, smp, g0 = m.points.cpu().numpy(), m.sample_inds.cpu().numpy(), m.grid_size
    m = handle_stride_disjoint_and_build_triplets(m, stride=K, kernel_size=K)
    oi, oj, ok, centres, slack = ogeo.partition_triplets(pts, g0, K, K, smp)
    assert np.allclose(m.points.cpu().numpy(), centres, atol=1e-6)
    got = {int(j): (int(i), int(k)) for i, j, k in zip(m.i.cpu(), m.j.cpu(), m.k.cpu())}
    moved = 0
    for i, j, k, room in zip(oi, oj, ok, slack):
        gi, gk = got[int(j)]
        assert gi == int(i)
        if gk != int(k):                      # only a point a few ulp from a slot face may sit next door
            assert room < 1e-4, (int(j), gk, int(k), room)
            moved += 1
    assert moved <= 3
    sure = slack >= 1e-4                       # where the arithmetic cannot matter the order is identical too
    keep = torch.from_numpy(sure).to(m.j.device)
    if moved == 0:
        assert np.array_equal(m.j.cpu().numpy(), oj) and np.array_equal(m.k.cpu().numpy(), ok)
    assert int(keep.sum()) > 0.99 * len(oj)


@pytest.mark.parametrize("dtype,cin", [(torch.float32, 6), (torch.bfloat16, 16)])
def test_patchify_convolution_and_unpatchify(dtype, cin):
    from pointelligence_b200.layers import PointConv3d, Upsample, conv_with_stride_disjoint

    K, cout = 4, 32
    torch.manual_seed(0)
    m = _meta(n=5000, nbatch=2, seed=5)
    n = m.points.shape[0]
    conv = PointConv3d(cin, cout, kernel_size=K, bias=False).cuda().to(dtype)
    x = torch.randn(n, cin, device="cuda").to(dtype).requires_grad_(True)
    y, m2 = conv_with_stride_disjoint(conv, x, m, stride=K)
    assert y.shape == (m2.points.shape[0], cout) and y.dtype == dtype
    w = conv.weight.detach().double()[:, 0]                                     # (K^3, cin, cout)
    want = torch.zeros(y.shape, dtype=torch.float64, device="cuda")
    want.index_add_(0, m2.i, torch.einsum("tc,tcm->tm", x.detach().double()[m2.j], w[m2.k]))
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert (y.detach().double() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    go = torch.randn_like(y)
    from pointelligence_b200 import _cabi

    _cabi.profile_enable(True)
    y.backward(go)
    labels = [name for name, _ in _cabi.profile_records()]
    _cabi.profile_enable(False)
    if dtype == torch.bfloat16:   # one triplet per input point: the input gradient is stored row by row
        assert m2.contract.exact_cover_in and "mvmr_tc_kernel(dgrad, store)" in labels, labels
    want_dx = torch.zeros(n, cin, dtype=torch.float64, device="cuda")
    want_dx.index_add_(0, m2.j, torch.einsum("tm,tcm->tc", go.double()[m2.i], w[m2.k]))
    assert (x.grad.double() - want_dx).abs().max() <= tol * max(1.0, float(want_dx.abs().max()))
    # the cached edges invert the partition: the unpatchify gives every input point a row back
    up = Upsample(cout, cin, kernel_size=K, bias=False, straight_recover=True, recompute_k=False).cuda().to(dtype)
    z, m3 = up(y.detach(), m2)
    assert z.shape == (n, cin) and m3.points.shape[0] == n
    wu = up.conv.weight.detach().double()[:, 0]
    want_z = torch.zeros(n, cin, dtype=torch.float64, device="cuda")
    want_z.index_add_(0, m2.j, torch.einsum("tm,tmc->tc", y.detach().double()[m2.i], wu[m2.k]))
    assert (z.double() - want_z).abs().max() <= tol * max(1.0, float(want_z.abs().max()))
