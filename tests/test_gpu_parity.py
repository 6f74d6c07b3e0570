"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle, the golden vectors produced by the reference, and size-independent
properties at the benchmark's full size.

Tolerances (relative Frobenius error, tests/unittest/test_tig_forward.py:127-135
of the reference): fp32 1e-5, fp16 2e-3, bf16 2e-2.  Index work is bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import geometry as og
from oracle import sparse_ops as oso

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 2e-2}


def _dev():
    return torch.device("cuda:0")


def _t(x, dtype=None):
    t = torch.as_tensor(np.asarray(x)).to(_dev())
    return t.to(dtype) if dtype is not None else t


def _cases(z):
    return sorted({k.split(".")[0] for k in z.files})


def _qm_keys(neighbors, counts, P):
    q = np.repeat(np.arange(len(counts)), counts)
    return np.sort(q.astype(np.int64) * P + np.asarray(neighbors, np.int64))


# ------------------------------------------------------------------ geometry
def test_radius_search_matches_reference_golden(golden):
    from pointelligence_b200.internals.neighbors import radius_predicate, radius_search_sorted_grid8

    z = golden("radius")
    for name in _cases(z):
        pts, q = z[f"{name}.points"], z[f"{name}.queries"]
        has_s = f"{name}.sample_inds" in z.files
        si = _t(z[f"{name}.sample_inds"]) if has_s else None
        qsi = _t(z[f"{name}.query_sample_inds"]) if has_s else None
        with radius_predicate("ieee"):  # the golden vectors come from Triton's CPU interpreter
            nb, cnt, dist = radius_search_sorted_grid8(_t(pts), _t(q), float(z[f"{name}.radius"]), si, qsi,
                                                       return_distances=True)
        nb, cnt, dist = nb.cpu().numpy(), cnt.cpu().numpy(), dist.cpu().numpy()
        assert nb.dtype == np.int64 and cnt.dtype == np.int64
        assert np.array_equal(cnt, z[f"{name}.num_neighbors"]), name
        assert np.array_equal(_qm_keys(nb, cnt, len(pts)),
                              _qm_keys(z[f"{name}.neighbors"], z[f"{name}.num_neighbors"], len(pts))), name
        rq = np.repeat(np.arange(len(cnt)), cnt)
        mine = dist[np.lexsort((nb, rq))]
        ref = z[f"{name}.distances"][np.lexsort((z[f"{name}.neighbors"], rq))]
        assert np.array_equal(mine, ref), name


def test_tap_segments_match_reference_golden(golden):
    from pointelligence_b200.internals.neighbors import radius_predicate, radius_search_sorted_grid8_segments

    z = golden("radius")
    for name in _cases(z):
        pts, q = z[f"{name}.points"], z[f"{name}.queries"]
        has_s = f"{name}.sample_inds" in z.files
        si = _t(z[f"{name}.sample_inds"]) if has_s else None
        qsi = _t(z[f"{name}.query_sample_inds"]) if has_s else None
        K = int(z[f"{name}.kernel_size"])
        with radius_predicate("ieee"):
            i, j, seg, cnt, k = radius_search_sorted_grid8_segments(
                _t(pts), _t(q), float(z[f"{name}.radius"]), K, float(z[f"{name}.kernel_grid_size"]), si, qsi,
                return_k=True)
        assert i.dtype == torch.int32 and j.dtype == torch.int32 and seg.dtype == torch.int64
        i, j, seg, cnt, k = (x.cpu().numpy() for x in (i, j, seg, cnt, k))
        assert np.array_equal(seg, z[f"{name}.seg_offs"]), name
        assert np.array_equal(cnt, z[f"{name}.seg_num_neighbors"]), name
        assert np.array_equal(k, np.repeat(np.arange(K ** 3), np.diff(seg))), name
        rk = np.repeat(np.arange(K ** 3), np.diff(z[f"{name}.seg_offs"]))
        assert np.array_equal(og.canonical_triplet_keys(i, j, k, len(q), len(pts)),
                              og.canonical_triplet_keys(z[f"{name}.i"], z[f"{name}.j"], rk, len(q), len(pts))), name
        # inside a tap the pairs are ordered by query (what the scatter epilogue merges on)
        for t in range(K ** 3):
            assert np.all(np.diff(i[seg[t]:seg[t + 1]]) >= 0)


@pytest.mark.parametrize("mode", ["fma", "ieee"])
@pytest.mark.parametrize("distance_type", ["ball", "chebyshev"])
def test_radius_search_matches_oracle_random(distance_type, mode):
    from pointelligence_b200.internals.neighbors import (radius_predicate, radius_search_sorted_grid8,
                                                         radius_search_sorted_grid8_segments)

    with radius_predicate(mode):
        _check_radius_search_against_oracle(distance_type, mode == "fma", radius_search_sorted_grid8,
                                            radius_search_sorted_grid8_segments)


def _check_radius_search_against_oracle(distance_type, fma, radius_search_sorted_grid8,
                                        radius_search_sorted_grid8_segments):

    rng = np.random.default_rng(17)
    pts = ((rng.random((6000, 3)) - 0.5) * 4).astype(np.float32)
    qry = np.concatenate([pts[::3], ((rng.random((500, 3)) - 0.5) * 4).astype(np.float32)])
    ps = np.sort(rng.integers(0, 3, len(pts)))
    qs = np.sort(rng.integers(0, 3, len(qry)))
    r = 0.19
    nb, cnt = radius_search_sorted_grid8(_t(pts), _t(qry), r, _t(ps), _t(qs), distance_type=distance_type)
    onb, ocnt = og.radius_search_sorted_grid8(pts, qry, r, ps, qs, distance_type=distance_type, fma=fma)
    assert np.array_equal(cnt.cpu().numpy(), ocnt)
    assert np.array_equal(_qm_keys(nb.cpu().numpy(), ocnt, len(pts)), _qm_keys(onb, ocnt, len(pts)))
    for K, g in ((3, 0.1), (5, 0.07)):
        i, j, seg, c2 = radius_search_sorted_grid8_segments(_t(pts), _t(qry), r, K, g, _t(ps), _t(qs),
                                                            distance_type=distance_type)
        oi, oj, oseg, oc = og.radius_search_sorted_grid8_segments(pts, qry, r, K, g, ps, qs,
                                                                  distance_type=distance_type, fma=fma)
        assert np.array_equal(seg.cpu().numpy(), oseg)
        k = np.repeat(np.arange(K ** 3), np.diff(oseg))
        assert np.array_equal(og.canonical_triplet_keys(i.cpu().numpy(), j.cpu().numpy(), k, len(qry), len(pts)),
                              og.canonical_triplet_keys(oi, oj, k, len(qry), len(pts)))
        assert np.array_equal(c2.cpu().numpy(), oc)


@pytest.mark.parametrize("P,Q", [(0, 0), (0, 3), (3, 0)])
def test_radius_search_empty_inputs(P, Q):
    from pointelligence_b200.internals.neighbors import (radius_search_sorted_grid8,
                                                         radius_search_sorted_grid8_segments)

    pts, q = torch.empty((P, 3), device=_dev()), torch.empty((Q, 3), device=_dev())
    nb, cnt, dist = radius_search_sorted_grid8(pts, q, 1.0, return_distances=True)
    assert nb.numel() == 0 and cnt.shape == (Q,) and dist.numel() == 0
    i, j, seg, cnt = radius_search_sorted_grid8_segments(pts, q, 0.2, 3, 0.2)
    assert i.dtype == torch.int32 and i.numel() == 0 and j.numel() == 0
    assert torch.equal(seg, torch.zeros(28, dtype=torch.int64, device=_dev()))
    assert cnt.shape == (Q,)


def test_radius_search_rejects_bad_arguments():
    from pointelligence_b200.internals.neighbors import radius_search_sorted_grid8_segments as seg

    p = torch.zeros((1, 3), device=_dev())
    for ks, g in ((2, 0.1), (0, 0.1), (3, 0.0)):
        with pytest.raises(ValueError):
            seg(p, p, radius=0.2, kernel_size=ks, kernel_grid_size=g)
    for stripes in (0, 3, 512):
        with pytest.raises(ValueError, match="tap_stripes"):
            seg(p, p, 0.2, 3, 0.2, tap_stripes=stripes)
    with pytest.raises(ValueError):
        seg(p, p, -1.0, 3, 0.2)


def test_downsample_matches_reference_golden(golden):
    from pointelligence_b200.internals.grid_sample import grid_sample_filter

    z = golden("downsample")
    for name in _cases(z):
        has_s = f"{name}.sample_inds" in z.files
        si = _t(z[f"{name}.sample_inds"]) if has_s else None
        p, s, idx, mapping = grid_sample_filter(_t(z[f"{name}.points"]), float(z[f"{name}.cell"]), si,
                                                return_mapping=True)
        assert idx.dtype == torch.int64
        assert np.array_equal(idx.cpu().numpy(), z[f"{name}.out_indices"]), name
        assert np.array_equal(p.cpu().numpy(), z[f"{name}.out_points"]), name
        assert np.array_equal(mapping.cpu().numpy(), z[f"{name}.out_mapping"]), name
        if has_s:
            assert np.array_equal(s.cpu().numpy(), z[f"{name}.out_sample_inds"]), name


def test_downsample_matches_oracle_on_scene():
    from pointelligence_b200.layers.downsample import downsample
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    pts, inds, sizes = ragged_batch([indoor_scene(20000, 3), indoor_scene(12000, 4)])
    p_, s_, g_, idx = downsample(_t(pts), _t(inds), 0.02, 2)
    op, os_, oidx, _ = og.grid_sample_center_nearest(pts, 0.04, inds)
    assert g_ == 0.04
    assert np.array_equal(idx.cpu().numpy(), oidx)
    assert np.array_equal(p_.cpu().numpy(), op)
    assert np.array_equal(s_.cpu().numpy(), os_)


# -------------------------------------------------------------------- sparse
def _random_rulebook(rng, K, n_in, n_out, T, empty_taps=()):
    k = np.sort(rng.integers(0, K, T))
    for e in empty_taps:
        k = k[k != e]
    T = len(k)
    i = rng.integers(0, n_out, T)
    # ordered by query inside a tap, like the builder's output
    order = np.lexsort((i, k))
    return i[order].astype(np.int32), rng.integers(0, n_in, T).astype(np.int32), k.astype(np.int32)


def test_generic_engine_is_close_to_reference_cpu_ops(golden):
    from pointelligence_b200 import _cabi

    z = golden("sparse")
    for name in _cases(z):
        a, b, go = z[f"{name}.a"], z[f"{name}.b"], z[f"{name}.go"]
        ai, bi, oi = z[f"{name}.a_idx"], z[f"{name}.b_idx"], z[f"{name}.o_idx"]
        K, G, C, M = a.shape
        n_o = int(z[f"{name}.n_o"])
        seg = _cabi.seg_offs_from_sorted(_t(ai), K)
        assert np.array_equal(seg.cpu().numpy(), np.searchsorted(ai, np.arange(K + 1)))
        for use_seg in (True, False):
            out = _cabi.mvmr(_t(a), _t(b).view(len(b), -1), _t(bi), _t(oi), seg if use_seg else None,
                             None if use_seg else _t(ai), n_o, False, _cabi.ENGINE_CUDA_CORE)
            assert oso.rel_frobenius(out.view(n_o, G, M).cpu().numpy(), z[f"{name}.mvmr"]) < 1e-5, name
            gw = _cabi.vvor(_t(b), _t(bi), _t(go), _t(oi), seg if use_seg else None,
                            None if use_seg else _t(ai), K, _cabi.ENGINE_CUDA_CORE)
            assert oso.rel_frobenius(gw.cpu().numpy(), z[f"{name}.vvor"]) < 1e-5, name


SHAPES = [(27, 64, 64), (27, 32, 32), (27, 128, 128), (27, 256, 256), (27, 48, 80), (27, 64, 16),
          (125, 32, 64), (1, 64, 32)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("K,C,M", SHAPES)
def test_tensor_engine_forward_dgrad_wgrad(dtype, K, C, M):
    from pointelligence_b200 import _cabi

    rng = np.random.default_rng(K * 1000 + C + M)
    n_in, n_out, T = 900, 700, 9000
    i, j, k = _random_rulebook(rng, K, n_in, n_out, T, empty_taps=(2,) if K > 2 else ())
    T = len(k)
    w = _t(rng.standard_normal((K, 1, C, M)) / np.sqrt(C), dtype)
    x = _t(rng.standard_normal((n_in, C)), dtype)
    go = _t(rng.standard_normal((n_out, M)), dtype)
    seg = _cabi.seg_offs_from_sorted(_t(k), K)
    wn, xn, gn = (t.float().cpu().numpy().astype(np.float64) for t in (w, x, go))

    out = _cabi.mvmr(w, x, _t(j), _t(i), seg, None, n_out, False, _cabi.ENGINE_TENSOR)
    ref = oso.mvmr_f64(wn, k, xn[:, None, :], j, i, n_out)[:, 0]
    assert oso.rel_frobenius(out.float().cpu().numpy(), ref) < TOL[dtype]
    touched = np.zeros(n_out, bool)
    touched[i] = True
    assert torch.all(out[_t(~touched)] == 0)

    gx = _cabi.mvmr(w, go, _t(i), _t(j), seg, None, n_in, True, _cabi.ENGINE_TENSOR)
    ref = oso.mvmr_f64(np.swapaxes(wn, 2, 3), k, gn[:, None, :], i, j, n_in)[:, 0]
    assert oso.rel_frobenius(gx.float().cpu().numpy(), ref) < TOL[dtype]

    gw = _cabi.vvor(x.view(n_in, 1, C), _t(j), go.view(n_out, 1, M), _t(i), seg, None, K, _cabi.ENGINE_TENSOR)
    ref = oso.vvor_f64(xn[:, None, :], j, gn[:, None, :], i, k, K)
    assert oso.rel_frobenius(gw.float().cpu().numpy(), ref) < TOL[dtype]
    assert _cabi.device_status() == 0

    # the CUDA-core engine on the same inputs agrees with the tensor engine
    out_cc = _cabi.mvmr(w, x, _t(j), _t(i), seg, None, n_out, False, _cabi.ENGINE_CUDA_CORE)
    assert oso.rel_frobenius(out_cc.float().cpu().numpy(), out.float().cpu().numpy()) < TOL[dtype]


@pytest.mark.parametrize("Ma,Cb", [(256, 256), (192, 192), (256, 192), (208, 240), (192, 128), (128, 256), (256, 96), (96, 192)])
def test_wide_weight_gradient_many_chunks_per_cta(Ma, Cb):
    """Wide operands run the weight gradient as chunks of 64 triplets through a ring of operand
    buffers, one or two CTAs per SM: every CTA walks dozens of chunks and crosses several taps,
    among them empty taps and taps shorter than a chunk."""
    from pointelligence_b200 import _cabi

    rng = np.random.default_rng(Ma * 7 + Cb)
    K, n_a, n_b, T = 40, 2500, 3000, 420_000
    share = rng.random(K) ** 3          # very uneven taps
    share[[3, 17]] = 0.0                # two empty taps
    k = np.sort(rng.choice(K, size=T, p=share / share.sum())).astype(np.int32)
    k = np.concatenate([k, np.full(5, 3, np.int32)])        # a tap of five triplets
    k.sort()
    T = len(k)
    ia, ib = rng.integers(0, n_a, T).astype(np.int32), rng.integers(0, n_b, T).astype(np.int32)
    a = _t(rng.standard_normal((n_a, Ma)), torch.bfloat16)
    b = _t(rng.standard_normal((n_b, Cb)), torch.bfloat16)
    seg = _cabi.seg_offs_from_sorted(_t(k), K)
    gw = _cabi.vvor(a.view(n_a, 1, Ma), _t(ia), b.view(n_b, 1, Cb), _t(ib), seg, None, K, _cabi.ENGINE_TENSOR)
    assert _cabi.device_status() == 0
    an, bn = (t.float().cpu().numpy().astype(np.float64) for t in (a, b))
    ref = oso.vvor_f64_taps(an, ia, bn, ib, seg.cpu().numpy())        # one fp64 product per tap
    assert oso.rel_frobenius(gw.float().cpu().numpy().reshape(K, Ma, Cb), ref) < TOL[torch.bfloat16]
    assert torch.all(gw[17] == 0)



@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("G,C,M", [(1, 3, 32), (1, 32, 20), (2, 16, 24), (1, 40, 72)])
def test_odd_shapes_take_the_cuda_core_engine(dtype, G, C, M):
    from pointelligence_b200.sparse_engines.tig import TigIndex, tig_forward, tig_grad_input, tig_grad_weight

    rng = np.random.default_rng(G * 100 + C)
    K, n_in, n_out, T = 27, 300, 260, 3000
    i, j, k = _random_rulebook(rng, K, n_in, n_out, T)
    w = _t(rng.standard_normal((K, G, C, M)) / np.sqrt(C), dtype)
    x = _t(rng.standard_normal((n_in, G * C)), dtype)
    go = _t(rng.standard_normal((n_out, G * M)), dtype)
    idx = TigIndex(_t(i), _t(j), _t(k), n_out, K, assume_sorted=True, n_in=n_in)
    wn, xn, gn = (t.float().cpu().numpy().astype(np.float64) for t in (w, x, go))
    out = tig_forward(w, x, idx)
    ref = oso.mvmr_f64(wn, k, xn.reshape(n_in, G, C), j, i, n_out).reshape(n_out, -1)
    assert out.dtype == dtype and oso.rel_frobenius(out.float().cpu().numpy(), ref) < TOL[dtype]
    gx = tig_grad_input(w, go, idx)
    ref = oso.mvmr_f64(np.swapaxes(wn, 2, 3), k, gn.reshape(n_out, G, M), i, j, n_in).reshape(n_in, -1)
    assert oso.rel_frobenius(gx.float().cpu().numpy(), ref) < TOL[dtype]
    gw = tig_grad_weight(x, go, idx, w.shape)
    ref = oso.vvor_f64(xn.reshape(n_in, G, C), j, gn.reshape(n_out, G, M), i, k, K)
    assert gw.shape == w.shape and oso.rel_frobenius(gw.float().cpu().numpy(), ref) < TOL[dtype]


def test_public_ops_autograd_and_unsorted_triplets():
    from pointelligence_b200.sparse_engines.ops import (sparse_matrix_vector_multiplication_reduction as mvmr,
                                                        sparse_vector_vector_outer_product_reduction as vvor)

    rng = np.random.default_rng(5)
    K, G, C, M, n_in, n_out, T = 27, 1, 16, 32, 200, 180, 2500
    i, j, k = _random_rulebook(rng, K, n_in, n_out, T)
    for shuffle in (False, True):
        if shuffle:
            perm = rng.permutation(len(k))
            i, j, k = i[perm], j[perm], k[perm]
        a = _t(rng.standard_normal((K, G, C, M)), torch.float32).requires_grad_(True)
        b = _t(rng.standard_normal((n_in, G, C)), torch.float32).requires_grad_(True)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            o = mvmr(a, _t(k), b, _t(j), _t(i), n_out)
        assert o.shape == (n_out, G, M)
        go = _t(rng.standard_normal(o.shape), torch.float32)
        o.backward(go)
        an, bn, gn = (t.detach().cpu().numpy().astype(np.float64) for t in (a, b, go))
        assert oso.rel_frobenius(o.detach().cpu().numpy(), oso.mvmr_f64(an, k, bn, j, i, n_out)) < 1e-5
        assert oso.rel_frobenius(a.grad.cpu().numpy(), oso.vvor_f64(bn, j, gn, i, k, K)) < 1e-5
        assert oso.rel_frobenius(b.grad.cpu().numpy(),
                                 oso.mvmr_f64(np.swapaxes(an, 2, 3), k, gn, i, j, n_in)) < 1e-5
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            v = vvor(b.detach(), _t(j), go, _t(i), _t(k), K)
        assert v.shape == (K, G, C, M)
        assert oso.rel_frobenius(v.cpu().numpy(), oso.vvor_f64(bn, j, gn, i, k, K)) < 1e-5


def test_sparse_ops_empty_and_errors():
    from pointelligence_b200 import _cabi

    w = torch.zeros((27, 1, 16, 16), device=_dev(), dtype=torch.bfloat16)
    x = torch.zeros((5, 16), device=_dev(), dtype=torch.bfloat16)
    e = torch.empty(0, dtype=torch.int32, device=_dev())
    seg = torch.zeros(28, dtype=torch.int64, device=_dev())
    out = _cabi.mvmr(w, x, e, e, seg, None, 7, False)
    assert out.shape == (7, 16) and torch.all(out == 0)
    gw = _cabi.vvor(x.view(5, 1, 16), e, x.view(5, 1, 16), e, seg, None, 27)
    assert gw.shape == (27, 1, 16, 16) and torch.all(gw == 0)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        _cabi.mvmr(w.cpu(), x.cpu(), e.cpu(), e.cpu(), seg.cpu(), None, 7, False)
    one = torch.zeros(1, dtype=torch.int32, device=_dev())
    seg1 = torch.ones(28, dtype=torch.int64, device=_dev())
    seg1[0] = 0
    with pytest.raises(NotImplementedError):   # fp32 has no tensor-core path
        _cabi.mvmr(w.float(), x.float(), one, one, seg1, None, 7, False, _cabi.ENGINE_TENSOR)
    with pytest.raises(TypeError):
        _cabi.mvmr(w.double(), x.double(), e, e, seg, None, 7, False)


# ---------------------------------------------------------------- end to end
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pointconv3d_forward_backward_on_scene(dtype):
    from pointelligence_b200.layers import MetaData, PointConv3d, conv_with_stride
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    torch.manual_seed(0)
    pts, inds, sizes = ragged_batch([indoor_scene(6000, 1), indoor_scene(4000, 2)])
    C, M = 32, 64
    conv = PointConv3d(C, M, 3, bias=True, device=_dev(), dtype=dtype)
    x = torch.randn(len(pts), C, device=_dev(), dtype=dtype, requires_grad=True)
    for stride in (1, 2):
        m = MetaData(points=_t(pts), sample_inds=_t(inds), sample_sizes=_t(sizes), grid_size=0.02)
        y, m = conv_with_stride(conv, x, m, stride, receptive_field_scaler=2.5)
        assert y.shape == (m.num_points(), M) and y.dtype == dtype
        go = torch.randn_like(y)
        conv.zero_grad()
        x.grad = None
        y.backward(go)
        # oracle: same rulebook from the CPU restatement, fp64 arithmetic
        rs = og.radius_scaler_for_kernel_size(3, 2.5)
        if stride == 1:
            qp, qi = pts, inds
        else:
            qp, qi, oidx, _ = og.grid_sample_center_nearest(pts, 0.04, inds)
            assert np.array_equal(m.downsample_indices.cpu().numpy(), oidx)
        oi, oj, oseg, _ = og.radius_search_sorted_grid8_segments(pts, qp, 0.02 * rs, 3, 0.02, inds, qi, fma=True)
        ok = np.repeat(np.arange(27), np.diff(oseg))
        assert np.array_equal(m.seg_offs.cpu().numpy(), oseg)
        assert np.array_equal(
            og.canonical_triplet_keys(m.i.cpu().numpy(), m.j.cpu().numpy(), m.k.cpu().numpy(), len(qp), len(pts)),
            og.canonical_triplet_keys(oi, oj, ok, len(qp), len(pts)))
        wn = conv.weight.detach().float().cpu().numpy().astype(np.float64)
        xn = x.detach().float().cpu().numpy().astype(np.float64)[:, None, :]
        gn = go.float().cpu().numpy().astype(np.float64)[:, None, :]
        ref = oso.mvmr_f64(wn, ok, xn, oj, oi, len(qp))[:, 0] + conv.bias.detach().float().cpu().numpy()
        assert oso.rel_frobenius(y.detach().float().cpu().numpy(), ref) < TOL[dtype]
        assert oso.rel_frobenius(conv.weight.grad.float().cpu().numpy(),
                                 oso.vvor_f64(xn, oj, gn, oi, ok, 27)) < TOL[dtype]
        assert oso.rel_frobenius(x.grad.float().cpu().numpy(),
                                 oso.mvmr_f64(np.swapaxes(wn, 2, 3), ok, gn, oi, oj, len(pts))[:, 0]) < TOL[dtype]


def test_full_size_properties_150k_scene():
    """Benchmark-size workload checked through properties that do not need the
    CPU oracle: tap offsets vs bincount, per-query counts, pair symmetry of a
    self query, and a checksum of the convolution against torch index math."""
    from pointelligence_b200 import _cabi
    from pointelligence_b200.layers.triplets import build_triplets_segmented
    from pointelligence_b200.synthetic import indoor_scene

    pts = indoor_scene(150000, 0)
    N = len(pts)
    p = _t(pts)
    s = torch.zeros(N, dtype=torch.int64, device=_dev())
    i, j, k, seg, nn = build_triplets_segmented(p, s, torch.tensor([N], device=_dev()), 0.05, 3,
                                                return_num_neighbors=True, radius_scaler=2.5)
    T = i.numel()
    assert T == 896518  # known answer of the CPU oracle for this seeded scene
    assert torch.equal(seg.diff(), torch.bincount(k.long(), minlength=27))
    assert torch.equal(torch.bincount(i.long(), minlength=N), nn) and int(nn.sum()) == T
    fwd = torch.sort(i.long() * N + j.long()).values
    rev = torch.sort(j.long() * N + i.long()).values
    assert torch.equal(fwd, rev) and torch.unique(fwd).numel() == T
    # the mirrored pair sits in the mirrored tap
    kk = torch.stack((k // 9, (k // 3) % 3, k % 3), 1)
    mirrored = ((2 - kk[:, 0]) * 9 + (2 - kk[:, 1]) * 3 + (2 - kk[:, 2])).long()
    key = torch.sort(mirrored * (N * N) + j.long() * N + i.long()).values
    assert torch.equal(key, torch.sort(k.long() * (N * N) + i.long() * N + j.long()).values)

    C = 64
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(N, C, device=_dev(), generator=g).bfloat16()
    w = (torch.rand(27, 1, C, C, device=_dev(), generator=g) * 2 - 1).mul_(1 / np.sqrt(C * 27)).bfloat16()
    out = _cabi.mvmr(w, x, j, i, seg, None, N, False)
    ref = torch.zeros(N, C, device=_dev(), dtype=torch.float32)
    for t in range(27):
        a, b = int(seg[t]), int(seg[t + 1])
        ref.index_add_(0, i[a:b].long(), x[j[a:b].long()].float() @ w[t, 0].float())
    err = (out.float() - ref).norm() / ref.norm()
    assert float(err) < 2e-2
    assert _cabi.device_status() == 0


# ------------------------------------------------------------------ full cover
def _full_cover_fixture():
    pts0 = torch.tensor([[0.001, 0.001, 0.001], [0.399, 0.399, 0.399], [0.401, 0.001, 0.001],
                         [0.799, 0.399, 0.399]], device=_dev())
    pts = torch.cat([pts0, pts0 + torch.tensor([2.0, 0.0, 0.0], device=_dev())])
    si = torch.cat([torch.zeros(4, dtype=torch.long, device=_dev()), torch.ones(4, dtype=torch.long, device=_dev())])
    return pts, si, torch.bincount(si)


def test_full_cover_rulebook_fixture():
    """tests/unittest/test_full_cover_strided.py:52-120 of the reference: K15 is
    required for stride 8 at grid 0.05, edges are exactly the same-sample pairs
    within R, the mirrored rulebook is the transpose with mirrored taps."""
    from pointelligence_b200.layers import build_full_cover_strided_rulebook

    pts, si, sizes = _full_cover_fixture()
    with pytest.raises(ValueError, match="needs kernel_size >= 15"):
        build_full_cover_strided_rulebook(pts, si, sizes, stride=8, input_grid_size=0.05, kernel_size=13)
    rb = build_full_cover_strided_rulebook(pts, si, sizes, stride=8, input_grid_size=0.05, kernel_size=15)
    rb2 = build_full_cover_strided_rulebook(pts, si, sizes, stride=8, input_grid_size=0.05, kernel_size=15)
    for f in ("i", "j", "k", "center_source_indices", "i_upsample", "j_upsample", "k_upsample"):
        assert torch.equal(getattr(rb, f), getattr(rb2, f)), f          # deterministic
    assert rb.radius == pytest.approx(0.34987426, rel=1e-7)
    n = pts.shape[0]
    cpts, cs = rb.points, rb.sample_inds
    within = (torch.cdist(cpts.double(), pts.double()) <= rb.radius) & (cs[:, None] == si[None, :])
    bi, bj = torch.nonzero(within, as_tuple=True)
    assert torch.equal(torch.sort(rb.i.long() * (n + 1) + rb.j.long()).values, torch.sort(bi * (n + 1) + bj).values)
    assert torch.all(rb.coverage_per_input > 0)
    assert torch.equal(rb.points, pts[rb.center_source_indices.long()])
    assert torch.all(rb.k[1:] >= rb.k[:-1]) and torch.all(rb.k_upsample[1:] >= rb.k_upsample[:-1])
    K = 15
    kk = rb.k.long()
    mirrored = ((K - 1 - kk // (K * K)) * K + (K - 1 - (kk // K) % K)) * K + (K - 1 - kk % K)
    nc = cpts.shape[0]
    down = torch.sort(mirrored * (n * nc) + rb.j.long() * nc + rb.i.long()).values
    up = torch.sort(rb.k_upsample.long() * (n * nc) + rb.i_upsample.long() * nc + rb.j_upsample.long()).values
    assert torch.equal(down, up)
    assert torch.equal(torch.bincount(rb.i.long(), minlength=nc), rb.num_neighbors)


@pytest.mark.parametrize("sort_by", ["k", "i", "j"])
def test_generic_build_triplets_against_oracle(sort_by):
    """The generic builder (query-major search, tap from a caller-supplied indexer, global sort;
    layers/triplets.py:686-764 of the reference): its triplet set equals the oracle's canonical
    set for the library's own ``voxelize_3d`` indexer and for a custom one, it is ordered by the
    requested column, and the per-query counts are the oracle's."""
    from functools import partial

    from pointelligence_b200.layers.triplets import build_triplets, voxelize_3d
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    pts, inds, sizes = ragged_batch([indoor_scene(3000, 11), indoor_scene(2000, 12)])
    qp, qi, _, _ = og.grid_sample_center_nearest(pts, 0.04, inds)           # a separate, coarser query set
    qsizes = np.bincount(qi, minlength=2)
    radius, scaler = 0.06, 2.0

    def octant(points, grid_size):   # a custom indexer: the octant of the offset (8 taps)
        return ((points[:, 0] > 0).long() * 2 + (points[:, 1] > 0).long()) * 2 + (points[:, 2] > 0).long()

    onb, ocnt = og.radius_search_sorted_grid8(pts, qp, radius, inds, qi, fma=True)
    oi = np.repeat(np.arange(len(qp)), ocnt)
    off = pts[onb] - qp[oi]
    for indexer, taps, ok in ((partial(voxelize_3d, 3), 27, og.voxelize_3d(3, off, radius / scaler)),
                              (octant, 8, ((off[:, 0] > 0) * 2 + (off[:, 1] > 0)) * 2 + (off[:, 2] > 0))):
        i, j, k, cnt = build_triplets(_t(pts), _t(inds), _t(sizes), radius, indexer, query_points=_t(qp),
                                      query_sample_inds=_t(qi), query_sample_sizes=_t(qsizes), sort_by=sort_by,
                                      return_num_neighbors=True, radius_scaler=scaler)
        assert i.dtype == torch.int32 and j.dtype == torch.int32 and k.dtype == torch.int32
        assert np.array_equal(cnt.cpu().numpy(), ocnt)
        got = og.canonical_triplet_keys(i.cpu().numpy(), j.cpu().numpy(), k.cpu().numpy(), len(qp), len(pts))
        want = og.canonical_triplet_keys(oi, onb, np.asarray(ok), len(qp), len(pts))
        assert np.array_equal(got, want), (sort_by, taps)
        col = {"i": i, "j": j, "k": k}[sort_by]
        assert torch.all(col[1:] >= col[:-1])


def test_full_cover_rulebook_matches_reference_golden(golden):
    """The centres, their order, the per-point bookkeeping and both edge sets equal what the
    reference's own ``build_full_cover_strided_rulebook`` produces on the same inputs (run on CPU
    with its radius search pointed at the restated one; ``tests/golden/make_golden.py``): the
    unit-test fixture, a two-sample scene, and a cloud whose residual selector runs for several
    rounds.  The order of edges inside a tap is unspecified, so edges are compared sorted."""
    from pointelligence_b200.internals.neighbors import radius_predicate
    from pointelligence_b200.layers import build_full_cover_strided_rulebook

    z = golden("full_cover")
    for name in _cases(z):
        pts, si = _t(z[f"{name}.points"]), _t(z[f"{name}.sample_inds"])
        with radius_predicate("ieee"):   # the golden search rounds once per operation
            rb = build_full_cover_strided_rulebook(pts, si, torch.bincount(si), stride=float(z[f"{name}.stride"]),
                                                   input_grid_size=float(z[f"{name}.grid"]),
                                                   kernel_size=int(z[f"{name}.kernel_size"]))
        for f in ("center_source_indices", "initial_center_source_indices", "additional_center_source_indices",
                  "point_to_initial_center", "num_neighbors", "coverage_per_input", "initial_center_counts",
                  "additional_center_counts", "sample_sizes"):
            assert np.array_equal(getattr(rb, f).cpu().numpy().astype(np.int64), z[f"{name}.{f}"]), (name, f)
        assert rb.radius == float(z[f"{name}.radius"]) and rb.selector_round_count == int(z[f"{name}.rounds"]), name
        n, nc = pts.shape[0], rb.points.shape[0]
        edges = torch.sort((rb.k.long() * nc + rb.i.long()) * n + rb.j.long()).values
        assert np.array_equal(edges.cpu().numpy(), z[f"{name}.edges"]), name
        up = torch.sort((rb.k_upsample.long() * n + rb.i_upsample.long()) * nc + rb.j_upsample.long()).values
        assert np.array_equal(up.cpu().numpy(), z[f"{name}.edges_upsample"]), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv_with_stride_full_cover_on_scene(dtype):
    """Stride 2 needs a 5x5x5 kernel (125 taps); centres cover every input and
    residual centres keep their distance; the convolution matches the fp64 oracle."""
    from pointelligence_b200.layers import MetaData, PointConv3d, conv_with_stride_full_cover
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    torch.manual_seed(1)
    pts, inds, sizes = ragged_batch([indoor_scene(5000, 5), indoor_scene(3000, 6)])
    C, M = 32, 32
    conv = PointConv3d(C, M, 5, bias=False, device=_dev(), dtype=dtype)
    with pytest.raises(ValueError, match="needs kernel_size >= 5"):
        conv_with_stride_full_cover(PointConv3d(C, M, 3, device=_dev(), dtype=dtype),
                                    torch.zeros(len(pts), C, device=_dev(), dtype=dtype),
                                    MetaData(points=_t(pts), sample_inds=_t(inds), sample_sizes=_t(sizes),
                                             grid_size=0.02), 2)
    x = torch.randn(len(pts), C, device=_dev(), dtype=dtype, requires_grad=True)
    m = MetaData(points=_t(pts), sample_inds=_t(inds), sample_sizes=_t(sizes), grid_size=0.02)
    y, m = conv_with_stride_full_cover(conv, x, m, 2)
    assert m.grid_size == 0.04 and y.shape == (m.num_points(), M)
    tel = m.parent.full_cover_telemetry
    assert tel["edge_count"] == m.i.numel() and tel["initial_center_count"] > 0
    assert torch.all(m.parent.full_cover_coverage_per_input > 0)
    extra = m.parent.full_cover_additional_center_indices.long()
    if extra.numel() > 1:    # the residual centres form an R-net: no two of one sample within R
        ep, es = _t(pts)[extra], _t(inds)[extra]
        dmat = torch.cdist(ep.double(), ep.double()) + torch.eye(len(extra), device=_dev()) * 10
        assert torch.all((dmat > tel["radius"]) | (es[:, None] != es[None, :]))
    # edge set = oracle radius search from the chosen centres
    centers = m.downsample_indices.long().cpu().numpy()
    oi, oj, _, _ = og.radius_search_sorted_grid8_segments(pts, pts[centers], tel["radius"], 5, 0.02, inds,
                                                          inds[centers], fma=True)
    n = len(pts)
    assert np.array_equal(np.sort(m.i.cpu().numpy().astype(np.int64) * n + m.j.cpu().numpy()),
                          np.sort(oi.astype(np.int64) * n + oj))
    go = torch.randn_like(y)
    y.backward(go)
    wn = conv.weight.detach().float().cpu().numpy().astype(np.float64)
    xn = x.detach().float().cpu().numpy().astype(np.float64)[:, None, :]
    gn = go.float().cpu().numpy().astype(np.float64)[:, None, :]
    i_, j_, k_ = (t.cpu().numpy() for t in (m.i, m.j, m.k))
    assert oso.rel_frobenius(y.detach().float().cpu().numpy(), oso.mvmr_f64(wn, k_, xn, j_, i_, len(centers))[:, 0]) < TOL[dtype]
    assert oso.rel_frobenius(conv.weight.grad.float().cpu().numpy(), oso.vvor_f64(xn, j_, gn, i_, k_, 125)) < TOL[dtype]
    assert oso.rel_frobenius(x.grad.float().cpu().numpy(),
                             oso.mvmr_f64(np.swapaxes(wn, 2, 3), k_, gn, i_, j_, n)[:, 0]) < TOL[dtype]


# ------------------------------------------------------- upsample, triplet cache
def test_upsample_fresh_search_and_cached_edges():
    from pointelligence_b200.layers import MetaData, PointConv3d, Upsample, conv_with_stride
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    torch.manual_seed(3)
    pts, inds, sizes = ragged_batch([indoor_scene(4000, 7), indoor_scene(2500, 8)])
    down = PointConv3d(16, 32, 3, bias=False, device=_dev())
    x = torch.randn(len(pts), 16, device=_dev())
    m = MetaData(points=_t(pts), sample_inds=_t(inds), sample_sizes=_t(sizes), grid_size=0.02)
    y, m = conv_with_stride(down, x, m, 2, receptive_field_scaler=2.5)
    coarse = m.points.cpu().numpy()
    coarse_s = m.sample_inds.cpu().numpy()
    yn = y.detach().cpu().numpy().astype(np.float64)[:, None, :]

    fresh = Upsample(32, 16, 3, bias=False, receptive_field_scaler=2.5).to(_dev())
    out, m_hi = fresh(y, m)
    assert out.shape == (len(pts), 16) and m_hi.num_points() == len(pts)
    rs = og.radius_scaler_for_kernel_size(3, 2.5)
    oi, oj, oseg, _ = og.radius_search_sorted_grid8_segments(coarse, pts, 0.04 * rs, 3, 0.04, coarse_s, inds, fma=True)
    ok = np.repeat(np.arange(27), np.diff(oseg))
    assert np.array_equal(m_hi.seg_offs.cpu().numpy(), oseg)
    assert np.array_equal(
        og.canonical_triplet_keys(m_hi.i.cpu().numpy(), m_hi.j.cpu().numpy(), m_hi.k.cpu().numpy(), len(pts), len(coarse)),
        og.canonical_triplet_keys(oi, oj, ok, len(pts), len(coarse)))
    wn = fresh.conv.weight.detach().cpu().numpy().astype(np.float64)
    assert oso.rel_frobenius(out.detach().cpu().numpy(), oso.mvmr_f64(wn, ok, yn, oj, oi, len(pts))[:, 0]) < 1e-5

    cached = Upsample(32, 16, 3, bias=False, straight_recover=True).to(_dev())
    out2, m2 = cached(y, m)
    assert torch.equal(m2.i, m.j) and torch.equal(m2.j, m.i) and torch.equal(m2.k, m.k)
    wn = cached.conv.weight.detach().cpu().numpy().astype(np.float64)
    ref = oso.mvmr_f64(wn, m.k.cpu().numpy(), yn, m.i.cpu().numpy(), m.j.cpu().numpy(), len(pts))[:, 0]
    assert oso.rel_frobenius(out2.detach().cpu().numpy(), ref) < 1e-5
    with pytest.raises(ValueError, match="Parent information"):
        fresh(x[:, :16].repeat(1, 2), MetaData(points=_t(pts), sample_inds=_t(inds), sample_sizes=_t(sizes), grid_size=0.02))


def test_triplet_cache_scope_reuses_rulebooks():
    from pointelligence_b200.internals.triplet_cache import triplet_cache_scope
    from pointelligence_b200.layers.triplets import build_triplets_segmented

    pts = _t(np.random.default_rng(0).random((3000, 3)).astype(np.float32))
    s = torch.zeros(3000, dtype=torch.int64, device=_dev())
    n = torch.tensor([3000], device=_dev())
    a = build_triplets_segmented(pts, s, n, 0.1, 3, radius_scaler=2.0)
    b = build_triplets_segmented(pts, s, n, 0.1, 3, radius_scaler=2.0)
    assert a[0] is not b[0] and torch.equal(a[0], b[0])          # no scope: rebuilt, same result
    with triplet_cache_scope():
        c = build_triplets_segmented(pts, s, n, 0.1, 3, radius_scaler=2.0)
        d = build_triplets_segmented(pts, s, n, 0.1, 3, radius_scaler=2.0)
        e = build_triplets_segmented(pts, s, n, 0.12, 3, radius_scaler=2.0)
        assert c[0] is d[0] and c[3] is d[3]
        assert e[0] is not c[0]
    f = build_triplets_segmented(pts, s, n, 0.1, 3, radius_scaler=2.0)
    assert f[0] is not c[0] and torch.equal(f[0], c[0])
