"""GPU parity tests of the segment reductions, the ragged norm layers and the
pooling layers: the CUDA kernels, called through the C ABI, against the golden
vectors produced by the reference and against the float64 oracle.

Tolerances: fp32 1e-5 (sums are re-associated), fp16 2e-3, bf16 1e-2 relative
to the largest magnitude of the expected result; max / min are exact.
"""
import numpy as np
import pytest
import torch

from oracle import segment_ops as seg

pytestmark = pytest.mark.gpu

OPS = ("sum", "mean", "max", "min")
TOL = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1e-2}


def _t(x, dtype=None):
    t = torch.as_tensor(np.asarray(x)).to("cuda:0")
    return t.to(dtype) if dtype is not None else t


def _close(got, want, tol, msg=""):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape, msg)
    finite = np.isfinite(want)
    assert np.array_equal(np.isnan(got), np.isnan(want)), msg
    assert np.array_equal(got[~finite & ~np.isnan(want)], want[~finite & ~np.isnan(want)]), msg
    scale = max(1.0, np.abs(want[finite]).max() if finite.any() else 1.0)
    assert np.abs(got[finite] - want[finite]).max() <= tol * scale, (np.abs(got[finite] - want[finite]).max(), msg)


def _cases(z, prefix):
    return sorted({k.split(".")[1] for k in z.files if k.startswith(prefix + ".")})


def test_large_segment_reduce_matches_reference_golden(golden):
    from pointelligence_b200.sparse_engines.ops import large_segment_reduce

    z = golden("segment")
    for name in _cases(z, "large"):
        lengths = _t(z[f"large.{name}.lengths"])
        for op in OPS:
            x = _t(z[f"large.{name}.x"]).requires_grad_(True)
            y = large_segment_reduce(x, op, lengths=lengths)
            _close(y, z[f"large.{name}.{op}"], 1e-5, f"{name} {op}")
            y.backward(_t(z[f"large.{name}.go"]))
            _close(x.grad, z[f"large.{name}.{op}.grad"], 1e-5, f"{name} {op} grad")


def test_indexed_segment_reduce_matches_reference_golden(golden):
    from pointelligence_b200.sparse_engines.ops import indexed_segment_reduce

    z = golden("segment")
    for name in _cases(z, "indexed"):
        lengths, idx = _t(z[f"indexed.{name}.lengths"]), _t(z[f"indexed.{name}.indices"])
        for op in OPS:
            x = _t(z[f"indexed.{name}.x"]).requires_grad_(True)
            y = indexed_segment_reduce(x, op, idx, lengths=lengths)
            _close(y, z[f"indexed.{name}.{op}"], 1e-5, f"{name} {op}")
            # an empty list has no gradient to give; NaN (mean of nothing) must not leak into it
            go = _t(z[f"indexed.{name}.go"])
            y.backward(go)
            _close(x.grad, z[f"indexed.{name}.{op}.grad"], 1e-5, f"{name} {op} grad")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("C", [3, 64, 200])
def test_large_segment_reduce_against_oracle(dtype, C):
    from pointelligence_b200.sparse_engines.ops import large_segment_reduce

    rng = np.random.default_rng(C)
    lengths = np.array([1, 0, 30000, 127, 129, 0, 17000, 128])
    x = _t(rng.standard_normal((lengths.sum(), C)), dtype)
    go = _t(rng.standard_normal((len(lengths), C)), dtype)
    xn, gn = x.float().cpu().numpy(), go.float().cpu().numpy()
    for op in OPS:
        xr = x.clone().requires_grad_(True)
        y = large_segment_reduce(xr, op, lengths=_t(lengths))
        assert y.dtype == dtype
        want = seg.large_segment_reduce(xn, lengths, op)
        if dtype == torch.float16:   # the reference clamps fp16 results (large_segment_reduce_triton.py:184-187)
            want = np.clip(want, -65504.0, 65504.0)
        # sums over 30000 rows: error relative to the sum of magnitudes
        tol = TOL[dtype] * (np.sqrt(lengths.max()) if op == "sum" else 1.0)
        _close(y, want, tol, op)
        y.backward(go)
        got_out = y.detach().float().cpu().numpy()
        _close(xr.grad, seg.large_segment_reduce_grad(gn, xn, got_out, lengths, op), TOL[dtype], op + " grad")


@pytest.mark.parametrize("op", ["max", "min"])
def test_large_segment_reduce_gradient_of_a_column_slice(op):
    """max / min gradients of a non-contiguous input (a column slice of a wider matrix): the
    backward must compare against the values the forward read, not against the wider rows."""
    from pointelligence_b200.sparse_engines.ops import large_segment_reduce

    rng = np.random.default_rng(2)
    lengths = np.array([40, 0, 300, 7])
    wide = _t(np.round(rng.standard_normal((lengths.sum(), 96)) * 4) / 4, torch.float32).requires_grad_(True)
    go = _t(rng.standard_normal((len(lengths), 64)), torch.float32)
    y = large_segment_reduce(wide[:, :64], op, lengths=_t(lengths))
    y.backward(go)
    ref = wide.detach().clone().requires_grad_(True)
    want = torch.segment_reduce(ref[:, :64].contiguous(), op, lengths=_t(lengths), unsafe=True)
    ok = torch.isfinite(want)                     # the empty segment reduces to +-inf in torch
    assert torch.equal(y[ok], want[ok])
    torch.where(ok, want, torch.zeros_like(want)).backward(go)
    # torch splits the gradient among ties, the reference (and this library) gives it to every
    # tied row: compare where the extreme value is unique
    xs = wide.detach()[:, :64]
    seg_id = torch.repeat_interleave(torch.arange(len(lengths), device=xs.device), _t(lengths))
    hit = xs == y.detach()[seg_id]
    unique = (torch.zeros_like(y).index_add_(0, seg_id, hit.float()) == 1)[seg_id]
    assert torch.allclose(wide.grad[:, :64][unique], ref.grad[:, :64][unique])
    assert torch.all(wide.grad[:, 64:] == 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_max_pool3d_and_global_pool_on_scene(dtype):
    from pointelligence_b200.layers import GlobalPool, MetaData, max_pool3d
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    pts, sample, sizes = ragged_batch([indoor_scene(4000, 3), indoor_scene(2500, 4)])
    pts_t, sample_t, sizes_t = _t(pts), _t(sample), _t(sizes)
    rng = np.random.default_rng(0)
    x = _t(rng.standard_normal((len(pts), 32)), dtype).requires_grad_(True)
    m = MetaData(points=pts_t, sample_inds=sample_t, sample_sizes=sizes_t, grid_size=0.02)
    y, m2 = max_pool3d(x, m, kernel_size=3, stride=2)
    assert y.shape == (m2.points.shape[0], 32) and y.dtype == dtype
    j, nn_ = m2.j.cpu().numpy(), m2.num_neighbors.cpu().numpy()
    assert nn_.sum() == len(j) and nn_.min() >= 1
    xn = x.detach().float().cpu().numpy()
    want = seg.indexed_segment_reduce(xn, j, nn_, "max")
    _close(y, want, 0.0, "max_pool3d")
    go = _t(rng.standard_normal(y.shape), dtype)
    y.backward(go)
    _close(x.grad, seg.indexed_segment_reduce_grad(go.float().cpu().numpy(), xn, want, j, nn_, "max", len(xn)),
           TOL[dtype], "max_pool3d grad")
    for method in ("mean", "max", "min"):
        pooled = GlobalPool(method)(x.detach(), sizes_t)
        _close(pooled, seg.large_segment_reduce(xn, sizes, method), TOL[dtype], method)


def test_ragged_norms_match_reference_golden_and_torch_gradients(golden):
    from pointelligence_b200.layers import RaggedGroupNorm, RaggedInstanceNorm, RaggedLayerNorm

    z = golden("segment")
    lengths = _t(z["norm.lengths"])

    def torch_reduce(v, reduce, lengths):
        return torch.segment_reduce(v, reduce=reduce, lengths=lengths, axis=0)

    for kind, make in (("layer", lambda **kw: RaggedLayerNorm(24, **kw)),
                       ("instance", lambda **kw: RaggedInstanceNorm(24, affine=True, **kw)),
                       ("group", lambda **kw: RaggedGroupNorm(4, 24, **kw))):
        grads = []
        for reduce_fn in (None, torch_reduce):
            layer = make(reduce_fn=reduce_fn).to("cuda:0")
            layer.weight.data = _t(z["norm.weight"])
            layer.bias.data = _t(z["norm.bias"])
            x = _t(z["norm.x"]).requires_grad_(True)
            y = layer(x, lengths)
            _close(y, z[f"norm.{kind}"], 1e-4, kind)
            y.square().sum().backward()
            grads.append((x.grad.clone(), layer.weight.grad.clone(), layer.bias.grad.clone()))
        for a, b in zip(*grads):
            _close(a, b.cpu().numpy(), 1e-4, kind + " gradients")
    layer = RaggedLayerNorm(24).to("cuda:0")
    with pytest.raises(ValueError):
        layer(_t(z["norm.x"]))
    y16 = layer(_t(z["norm.x"], torch.bfloat16), lengths)
    assert y16.dtype == torch.bfloat16


def test_segment_reduce_rejects_bad_arguments_and_handles_empty():
    from pointelligence_b200 import _cabi
    from pointelligence_b200.sparse_engines.ops import indexed_segment_reduce, large_segment_reduce

    x = torch.zeros((0, 8), device="cuda:0")
    lengths = torch.zeros(3, dtype=torch.int64, device="cuda:0")
    assert torch.all(large_segment_reduce(x, "sum", lengths=lengths) == 0)
    assert torch.all(torch.isinf(large_segment_reduce(x, "max", lengths=lengths)))
    empty_idx = torch.zeros(0, dtype=torch.int32, device="cuda:0")
    assert torch.all(indexed_segment_reduce(torch.ones((4, 8), device="cuda:0"), "sum", empty_idx, lengths=lengths) == 0)
    with pytest.raises(ValueError):
        large_segment_reduce(x, "median", lengths=lengths)
    with pytest.raises(RuntimeError):
        large_segment_reduce(torch.zeros((4, 8)), "sum", lengths=torch.tensor([4]))
    with pytest.raises(ValueError):
        _cabi.segment_reduce(torch.ones((4, 8), device="cuda:0"), torch.tensor([4], device="cuda:0"), 7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_layer_norm_residual_relu_matches_composition(dtype):
    """The fused kernel (statistics + affine + residual + ReLU, forward and backward)
    against the layer composed from torch operators, on samples that span many blocks
    and on boundaries inside a block."""
    from pointelligence_b200.layers import RaggedLayerNorm
    from pointelligence_b200.layers.norm import fused_layer_norm

    def torch_reduce(v, reduce, lengths):
        return torch.segment_reduce(v, reduce=reduce, lengths=lengths, axis=0)

    rng = np.random.default_rng(5)
    lengths = _t(np.array([3000, 1, 5000, 300]))
    C = 48
    x0 = _t(rng.standard_normal((8301, C)) * 2 + 0.5, dtype)
    r0 = _t(rng.standard_normal((8301, C)), dtype)
    composed = RaggedLayerNorm(C, reduce_fn=torch_reduce).to("cuda:0")
    composed.weight.data = _t(rng.standard_normal(C).astype(np.float32))
    composed.bias.data = _t(rng.standard_normal(C).astype(np.float32))
    go = _t(rng.standard_normal((8301, C)), dtype)
    results = []
    for fused in (True, False):
        x, r = x0.clone().requires_grad_(True), r0.clone().requires_grad_(True)
        composed.zero_grad()
        if fused:
            y = fused_layer_norm(x, lengths, composed.weight, composed.bias, composed.eps, residual=r, relu=True)
        else:
            y = torch.relu(composed(x.float(), lengths) + r.float()).to(dtype)
        y.backward(go)
        results.append([t.detach().float().cpu().numpy() for t in
                        (y, x.grad, r.grad, composed.weight.grad, composed.bias.grad)])
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for name, a, b in zip(("y", "dx", "dresidual", "dweight", "dbias"), *results):
        scale = max(1.0, np.abs(b).max())
        assert np.abs(a - b).max() <= tol * scale, (name, np.abs(a - b).max(), scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,C,G", [("group", 64, 8), ("group", 48, 16), ("group", 50, 5), ("instance", 48, 48),
                                      ("instance", 7, 7)])
def test_fused_group_and_instance_norm_match_composition(dtype, kind, C, G):
    """``pcx_ragged_group_norm`` (forward and backward) against the same layer composed from torch
    operators: samples spanning many row blocks, a one-row sample, boundaries inside a block, vector
    and scalar channel layouts, groups narrower and wider than one 16-byte access, with and without
    the affine parameters."""
    from pointelligence_b200 import _cabi
    from pointelligence_b200.layers import RaggedGroupNorm, RaggedInstanceNorm

    def torch_reduce(v, reduce, lengths):
        return torch.segment_reduce(v, reduce=reduce, lengths=lengths, axis=0)

    rng = np.random.default_rng(C * 131 + G)
    lengths = _t(np.array([3000, 1, 5000, 300, 0, 17]))
    n = int(lengths.sum())
    x0 = _t(rng.standard_normal((n, C)) * 2 + 0.5, dtype)
    go = _t(rng.standard_normal((n, C)), dtype)
    for affine in (True, False):
        make = (lambda **kw: RaggedGroupNorm(G, C, affine=affine, **kw)) if kind == "group" else \
               (lambda **kw: RaggedInstanceNorm(C, affine=affine, **kw))
        fused, composed = make().to("cuda:0"), make(reduce_fn=torch_reduce).to("cuda:0")
        if affine:
            w, b = rng.standard_normal(C).astype(np.float32), rng.standard_normal(C).astype(np.float32)
            for layer in (fused, composed):
                layer.weight.data, layer.bias.data = _t(w), _t(b)
        results = []
        for layer in (fused, composed):
            x = x0.clone().requires_grad_(True)
            _cabi.profile_enable(True)
            y = layer(x, lengths)
            names = [name for name, _ in _cabi.profile_records()]
            _cabi.profile_enable(False)
            assert ("gn_apply_kernel" in names) == (layer is fused), names
            assert y.dtype == dtype
            y.backward(go)
            got = [y, x.grad] + ([layer.weight.grad, layer.bias.grad] if affine else [])
            results.append([t.detach().float().cpu().numpy() for t in got])
        tol = 3e-5 if dtype == torch.float32 else 2e-2
        for name, a, b in zip(("y", "dx", "dweight", "dbias"), *results):
            scale = max(1.0, np.abs(b).max())
            assert np.abs(a - b).max() <= tol * scale, (kind, affine, name, np.abs(a - b).max(), scale)


def test_group_norm_rejects_bad_arguments():
    from pointelligence_b200 import _cabi

    x = torch.zeros((10, 24), device="cuda:0")
    lengths = torch.tensor([10], device="cuda:0")
    with pytest.raises(ValueError):
        _cabi.ragged_group_norm(x, lengths, None, None, 5, 1e-5)          # 24 channels, 5 groups
    with pytest.raises(ValueError):
        _cabi.ragged_group_norm(x, lengths, torch.ones(24, device="cuda:0"), None, 4, 1e-5)   # weight without bias
    y, mean, rstd = _cabi.ragged_group_norm(torch.zeros((0, 24), device="cuda:0"),
                                            torch.zeros(2, dtype=torch.int64, device="cuda:0"), None, None, 4, 1e-5)
    assert y.shape == (0, 24) and mean.shape == (8,)


@pytest.mark.parametrize("samples", [100, 5000])
def test_norms_with_many_short_samples(samples):
    """Hundreds and thousands of samples of 0 to 6 rows: many sample boundaries inside every row
    block, both row-offset paths (one small launch up to 4096 samples, the library scan above)."""
    from pointelligence_b200.layers import RaggedGroupNorm, RaggedLayerNorm

    def torch_reduce(v, reduce, lengths):
        return torch.segment_reduce(v, reduce=reduce, lengths=lengths, axis=0)

    rng = np.random.default_rng(samples)
    lens = rng.integers(1, 7, samples)          # torch.segment_reduce gives NaN means for empty samples
    lengths = _t(lens)
    x0 = _t(rng.standard_normal((int(lens.sum()), 32)).astype(np.float32))
    for make in (lambda **kw: RaggedLayerNorm(32, **kw), lambda **kw: RaggedGroupNorm(4, 32, **kw)):
        out = []
        for reduce_fn in (None, torch_reduce):
            layer = make(reduce_fn=reduce_fn).to("cuda:0")
            x = x0.clone().requires_grad_(True)
            y = layer(x, lengths)
            y.square().sum().backward()
            out.append((y.detach().cpu().numpy(), x.grad.cpu().numpy()))
        for a, b in zip(*out):
            assert np.abs(a - b).max() <= 2e-4 * max(1.0, np.abs(b).max())
