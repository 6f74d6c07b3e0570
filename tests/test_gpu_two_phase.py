"""``ConvOp`` through the two-phase scheduler against the serial ``conv_with_stride`` (what
``tests/unittest/test_two_phase_conv.py`` of the reference checks), plus what this build adds:
the plan of the output-stationary engine is prepared with the indices (no hand-over left in
``apply``), and a prepared chain of convolutions replays from one CUDA graph."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _toy(n=4096, c=16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pts = torch.rand(n, 3, generator=g, device="cuda") * 5.0
    x = torch.randn(n, c, generator=g, device="cuda")
    batch = torch.zeros(n, dtype=torch.long, device="cuda")
    batch[n // 2:] = 1
    return pts, x, batch


def _meta(pts, batch, grid=0.05):
    from pointelligence_b200.layers.metadata import MetaData

    return MetaData(points=pts.clone(), sample_inds=batch.clone(), sample_sizes=torch.bincount(batch), grid_size=grid)


def test_convop_scheduler_matches_serial():
    from pointelligence_b200.internals.two_phase import ForceFused, GeometryScheduler
    from pointelligence_b200.layers.conv import PointConv3d, conv_with_stride
    from pointelligence_b200.layers.two_phase_conv import ConvOp

    pts, x, batch = _toy()
    torch.manual_seed(0)
    conv = PointConv3d(16, 16, kernel_size=3).cuda()
    y_ref, m_ref = conv_with_stride(conv, x.clone(), _meta(pts, batch), stride=2.0)
    bundle = ConvOp(conv, stride=2.0).build_indices(_meta(pts, batch))
    for name in ("i", "j", "k", "seg_offs", "points", "sample_inds"):   # this build's order is deterministic
        assert torch.equal(getattr(bundle.meta, name), getattr(m_ref, name)), name
    assert bundle.meta.contract == m_ref.contract and bundle.next_geom.empty_triplets()
    y = GeometryScheduler().run([ConvOp(conv, stride=2.0)], x.clone(), geom=_meta(pts, batch))
    assert torch.allclose(y, y_ref, atol=1e-5)
    y_forced = GeometryScheduler().run([ForceFused(ConvOp(conv, stride=2.0))], x.clone(), geom=_meta(pts, batch))
    assert torch.allclose(y_forced, y_ref, atol=1e-5)
    # gradients flow through the hoisted order as through the serial one
    xg = x.clone().requires_grad_()
    GeometryScheduler().run([ConvOp(conv, stride=2.0), ConvOp(conv, stride=1.0)], xg, geom=_meta(pts, batch)).sum().backward()
    xr = x.clone().requires_grad_()
    y1, m1 = conv_with_stride(conv, xr, _meta(pts, batch), stride=2.0)
    m1.dirty_triplets()                                     # what a model does after a strided convolution
    conv_with_stride(conv, y1, m1, stride=1.0)[0].sum().backward()
    assert torch.allclose(xg.grad, xr.grad, atol=1e-4)


def test_plan_is_prepared_with_the_indices(monkeypatch):
    from pointelligence_b200 import _cabi
    from pointelligence_b200.layers.conv import PointConv3d
    from pointelligence_b200.layers.two_phase_conv import ConvOp

    monkeypatch.setattr(_cabi, "_PLANNED_DENSE_RATIO", 0.0)     # send every tap-sorted bf16 layer to the planned engine
    monkeypatch.setattr(_cabi, "_PLANNED_MIN_TAP_FILL", 0.0)
    monkeypatch.setattr(_cabi, "_PLANNED_ENABLED", True)
    pts, x, batch = _toy(c=32)
    conv = PointConv3d(32, 32, kernel_size=3).cuda().to(torch.bfloat16)
    op = ConvOp(conv, stride=1.0)
    _cabi._PLAN_CACHE.clear()
    bundle = op.build_indices(_meta(pts, batch, grid=0.2))
    assert len(_cabi._PLAN_CACHE) == 1                           # built in phase 1 ...
    _cabi.profile_enable(True)
    y = op.apply(x.to(torch.bfloat16), bundle)
    labels = [name for name, _ in _cabi.profile_records()]
    _cabi.profile_enable(False)
    assert len(_cabi._PLAN_CACHE) == 1                           # ... and found, not rebuilt, by the feature pass
    assert any("mvmr_os_kernel" in name for name in labels), labels
    assert torch.isfinite(y.float()).all()


def test_prepared_chain_replays_from_a_cuda_graph():
    from pointelligence_b200.internals.two_phase import GeometryScheduler
    from pointelligence_b200.layers.conv import PointConv3d
    from pointelligence_b200.layers.two_phase_conv import ConvOp

    pts, x, batch = _toy(c=32)
    torch.manual_seed(1)
    convs = [PointConv3d(32, 32, kernel_size=3).cuda().to(torch.bfloat16) for _ in range(3)]
    ops = [ConvOp(convs[0], stride=1.0), ConvOp(convs[1], stride=2.0), ConvOp(convs[2], stride=1.0)]
    with torch.no_grad():
        eager = GeometryScheduler().prepare(ops, _meta(pts, batch, grid=0.2))
        graphed = GeometryScheduler().prepare(ops, _meta(pts, batch, grid=0.2), compile_segments=True)
        for seed in range(3):                                   # first call captures, the others replay
            xs = torch.randn(x.shape[0], 32, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed))
            xs = xs.to(torch.bfloat16)
            want, got = eager(xs), graphed(xs)
            assert got.shape == want.shape
            assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
