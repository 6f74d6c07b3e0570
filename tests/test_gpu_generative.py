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
    y, m_out = conv(x, m, sites=sites)
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
