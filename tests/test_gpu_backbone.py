"""GPU test of the benchmark backbone: one training step on a small ragged batch
runs through the CUDA path end to end, produces finite logits of the right shape
and a finite, non-zero gradient for every parameter; the wide-input convolution
(more than 256 input channels, split into two tensor-core passes) agrees with
the float64 oracle within the bf16 tolerance of 2e-2."""
import numpy as np
import pytest
import torch

from oracle import sparse_ops as oso

pytestmark = pytest.mark.gpu


def test_resunet_training_step_on_small_batch():
    import torch.nn.functional as F

    from pointelligence_b200.backbone import ResUNet
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    pts, inds, sizes = ragged_batch([indoor_scene(6000, 1), indoor_scene(4000, 2)])
    dev = "cuda:0"
    pts, inds, sizes = (torch.from_numpy(a).to(dev) for a in (pts, inds, sizes))
    n = pts.shape[0]
    g = torch.Generator(device=dev).manual_seed(0)
    feat = torch.randn(n, 3, device=dev, generator=g)
    labels = torch.randint(0, 20, (n,), device=dev, generator=g)
    torch.manual_seed(0)
    model = ResUNet(in_channels=3, num_classes=20).to(dev)
    losses = []
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    for _ in range(3):
        opt.zero_grad()
        logits = model(feat, pts, inds, sizes, 0.02)
        assert logits.shape == (n, 20) and torch.isfinite(logits.float()).all()
        loss = F.cross_entropy(logits.float(), labels)
        loss.backward()
        for name, p in model.named_parameters():
            assert p.grad is not None and torch.isfinite(p.grad).all(), name
        opt.step()
        losses.append(float(loss.detach()))
    assert any(float(p.grad.abs().max()) > 0 for p in model.parameters())
    assert losses[-1] < losses[0], losses


def test_wide_input_convolution_is_split_and_matches_oracle():
    from pointelligence_b200.layers import PointConv3d
    from pointelligence_b200.sparse_engines._seg_offs import kernel_offset_segments

    rng = np.random.default_rng(4)
    K, C, M, n_in, n_out, T = 27, 384, 128, 500, 400, 6000
    k = np.sort(rng.integers(0, K, T)).astype(np.int32)
    i = rng.integers(0, n_out, T).astype(np.int32)
    j = rng.integers(0, n_in, T).astype(np.int32)
    dev = "cuda:0"
    conv = PointConv3d(C, M, kernel_size=3, bias=False).to(dev).to(torch.bfloat16)
    x = torch.randn(n_in, C, device=dev).bfloat16()
    ti, tj, tk = (torch.from_numpy(a).to(dev) for a in (i, j, k))
    out = conv(x, ti, tj, tk, n_out, seg_offs=kernel_offset_segments(tk, K))
    wn = conv.weight.detach().float().cpu().numpy().astype(np.float64)
    ref = oso.mvmr_f64(wn, k, x.float().cpu().numpy().astype(np.float64)[:, None, :], j, i, n_out)[:, 0]
    assert oso.rel_frobenius(out.detach().float().cpu().numpy(), ref) < 2e-2


def test_geometry_on_its_own_stream_gives_the_same_step(monkeypatch):
    """The backbone builds its geometry on a side stream beside the feature kernels
    (``_cabi.geometry_overlap``); with the scope switched off the same step must come out: same
    rulebooks, logits and gradients equal up to the order of the fp32 atomics."""
    import torch.nn.functional as F

    from pointelligence_b200 import _cabi
    from pointelligence_b200.backbone import ResUNet
    from pointelligence_b200.layers.metadata import MetaData
    from pointelligence_b200.layers.triplets import handle_stride_and_build_triplets
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    pts, inds, sizes = ragged_batch([indoor_scene(20000, 3), indoor_scene(9000, 4), indoor_scene(14000, 5)])
    dev = torch.device("cuda:0")
    pts, inds, sizes = (torch.from_numpy(a).to(dev) for a in (pts, inds, sizes))
    n = pts.shape[0]
    feat = torch.randn(n, 3, device=dev, generator=torch.Generator(device=dev).manual_seed(0))
    labels = torch.randint(0, 20, (n,), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    torch.manual_seed(0)
    model = ResUNet(in_channels=3, num_classes=20).to(dev)
    runs = []
    for mode in ("0", "0", "1", "1"):
        monkeypatch.setenv("PCX_GEOMETRY_OVERLAP", mode)
        model.zero_grad(set_to_none=True)
        # a long kernel queue in front of the step: the side stream must not run ahead of its inputs
        busy = torch.randn(4096, 4096, device=dev)
        for _ in range(20):
            busy = busy @ busy * 1e-3
        logits = model(feat + busy[0, 0] * 0, pts, inds, sizes, 0.02)
        F.cross_entropy(logits.float(), labels).backward()
        grads = torch.cat([p.grad.flatten().float() for p in model.parameters()])
        runs.append((logits.detach().float(), grads))
    # two runs of the same bf16 step differ by the order of their fp32 atomics; a run with the
    # geometry on its own stream must differ from a plain run by no more than that
    rel = lambda a, b: float((a - b).norm() / b.norm())
    for part in (0, 1):
        noise = rel(runs[1][part], runs[0][part])
        for overlapped in (runs[2], runs[3]):
            assert torch.isfinite(overlapped[part]).all()
            assert rel(overlapped[part], runs[0][part]) <= 3 * noise + 1e-3, (part, noise)
    # the rulebook of a strided layer, built inside and outside a scope, is bit-identical
    books = []
    for scoped in (True, False):
        m = MetaData(points=pts, sample_inds=inds, sample_sizes=sizes, grid_size=0.02)
        if scoped:
            with _cabi.geometry_overlap(dev):
                m = handle_stride_and_build_triplets(m, 2.0, (3, 3, 3), 1.0)
        else:
            m = handle_stride_and_build_triplets(m, 2.0, (3, 3, 3), 1.0)
        torch.cuda.synchronize()
        books.append(m)
    for name in ("i", "j", "k", "seg_offs", "points", "sample_inds", "downsample_indices"):
        assert torch.equal(getattr(books[0], name), getattr(books[1], name)), name
