"""``GenerativePointConv3d`` on the GPU: the generated sites equal the CPU build of the same
inputs, and the convolution through the library (uniform tap segments, no ``seg_offs`` given) equals
a dense fp64 evaluation of the rulebook, forward and input gradient."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _meta(n=3000, seed=0, device="cuda"):
    from pointelligence_b200.layers.metadata import MetaData

    g = torch.Generator().manual_seed(seed)
    grid = 0.1
    pts = (torch.div(torch.rand(n, 3, generator=g) * 3 - 1, grid, rounding_mode="floor") + 0.5) * grid
    pts = torch.unique(pts, dim=0)
    smp = (torch.arange(pts.shape[0]) >= pts.shape[0] // 2).long()
    return MetaData(points=pts.to(device), sample_inds=smp.to(device), sample_sizes=torch.bincount(smp).to(device),
                    grid_size=grid, auto_build_triplets=False)


@pytest.mark.parametrize("dtype,generator", [(torch.float32, "stamp"), (torch.bfloat16, "stamp"),
                                             (torch.bfloat16, "subdivision")])
def test_generative_convolution_matches_dense_evaluation(dtype, generator):
    from pointelligence_b200.layers import GenerativePointConv3d, SubdivisionGenerator

    m, m_cpu = _meta(), _meta(device="cpu")
    n, cin, cout = m.points.shape[0], 32, 48
    torch.manual_seed(0)
    gen = SubdivisionGenerator(2) if generator == "subdivision" else None
    conv = GenerativePointConv3d(cin, cout, kernel_size=3, expansion=2.0, generator=gen, bias=False).cuda().to(dtype)
    sites, sites_cpu = conv.generator(m), conv.generator(m_cpu)
    for name in ("points", "sample_inds", "sample_sizes", "i", "j", "k"):
        assert torch.equal(getattr(sites, name).cpu(), getattr(sites_cpu, name)), name
    x = torch.randn(n, cin, device="cuda").to(dtype).requires_grad_(True)
    from pointelligence_b200 import _cabi

    _cabi.profile_enable(True)
    y, m_out = conv(x, m, sites=sites)
    labels = [name for name, _ in _cabi.profile_records()]
    _cabi.profile_enable(False)
    if dtype == torch.bfloat16:   # fan-in 1 (nothing merged): rows are stored by the tensor kernel, not reduced
        assert ("mvmr_tc_kernel(fwd, store)" in labels) == sites.exact_cover_out, labels
    assert y.shape == (sites.n_out, cout) and m_out.parent is m and m_out.points.shape[0] == sites.n_out
    w = conv.weight.detach().double()[:, 0]
    i, j, k = sites.i.long(), sites.j.long(), sites.k.long()
    want = torch.zeros(y.shape, dtype=torch.float64, device="cuda")
    want.index_add_(0, i, torch.einsum("tc,tcm->tm", x.detach().double()[j], w[k]))
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert (y.detach().double() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    go = torch.randn_like(y)
    y.backward(go)
    want_dx = torch.zeros(n, cin, dtype=torch.float64, device="cuda")
    want_dx.index_add_(0, j, torch.einsum("tm,tcm->tc", go.double()[i], w[k]))
    assert (x.grad.double() - want_dx).abs().max() <= tol * max(1.0, float(want_dx.abs().max()))
    y2, _ = conv(x.detach(), m)                       # the generator runs inside forward as well
    assert torch.allclose(y2.float(), y.detach().float(), atol=tol, rtol=tol)


def test_fan_in_one_flag_through_the_c_abi():
    """``PCX_ENGINE_FLAG_FAN_IN_ONE``: a permutation rulebook (one triplet per output row) stored by
    the tensor kernel equals the reduced result bit for bit; the flag with T != n_out is refused;
    the CUDA-core engine ignores it."""
    from pointelligence_b200 import _cabi

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    K, C, M, n = 8, 32, 48, 5000
    w = torch.randn(K, 1, C, M, device=dev).to(torch.bfloat16)
    x = torch.randn(n, C, device=dev).to(torch.bfloat16)
    tap = torch.sort(torch.randint(0, K, (n,), device=dev)).values
    seg = torch.searchsorted(tap, torch.arange(K + 1, device=dev)).to(torch.int64)
    scatter = torch.randperm(n, device=dev).to(torch.int32)          # every output row exactly once
    gather = torch.randint(0, n, (n,), device=dev).to(torch.int32)
    reduced = _cabi.mvmr(w, x, gather, scatter, seg, None, n, False, _cabi.ENGINE_TENSOR)
    stored = _cabi.mvmr(w, x, gather, scatter, seg, None, n, False, _cabi.ENGINE_TENSOR | _cabi.ENGINE_FLAG_FAN_IN_ONE)
    assert torch.equal(stored, reduced)
    core = _cabi.mvmr(w, x, gather, scatter, seg, None, n, False, _cabi.ENGINE_CUDA_CORE | _cabi.ENGINE_FLAG_FAN_IN_ONE)
    assert torch.allclose(core.float(), reduced.float(), atol=2e-2, rtol=2e-2)
    with pytest.raises(ValueError):
        _cabi.mvmr(w, x, gather, scatter, seg, None, n + 1, False, _cabi.ENGINE_TENSOR | _cabi.ENGINE_FLAG_FAN_IN_ONE)
