"""The CPU oracle against golden vectors produced by the reference itself
(tests/golden/make_golden.py) and against the known answers of the
reference's unit tests.  No GPU needed."""
import math

import numpy as np
import pytest

from oracle import geometry as og
from oracle import sparse_ops as os_


def _case_names(z):
    return sorted({k.split(".")[0] for k in z.files})


def _query_major_keys(neighbors, counts, num_points):
    q = np.repeat(np.arange(len(counts)), counts)
    return np.sort(q.astype(np.int64) * num_points + neighbors.astype(np.int64))


def test_downsample_matches_reference(golden):
    z = golden("downsample")
    for name in _case_names(z):
        si = z[f"{name}.sample_inds"] if f"{name}.sample_inds" in z.files else None
        p, s, idx, mapping = og.grid_sample_center_nearest(
            z[f"{name}.points"], float(z[f"{name}.cell"]), si, return_mapping=True)
        assert np.array_equal(idx, z[f"{name}.out_indices"]), name
        assert np.array_equal(p, z[f"{name}.out_points"]), name
        assert np.array_equal(mapping, z[f"{name}.out_mapping"]), name
        if si is not None:
            assert np.array_equal(s, z[f"{name}.out_sample_inds"]), name


def test_downsample_tie_picks_lower_index(golden):
    z = golden("downsample")
    # tests/unittest/test_grid_sample_selector.py:75-108
    assert z["tie_dense.out_indices"][0] in (0, 1)
    _, _, idx, _ = og.grid_sample_center_nearest(
        z["tie_dense.points"], 1.0, z["tie_dense.sample_inds"])
    first_cell = idx[np.isin(idx, [0, 1])]
    assert first_cell.tolist() == [0]


def test_radius_search_matches_reference(golden):
    z = golden("radius")
    for name in _case_names(z):
        pts, q = z[f"{name}.points"], z[f"{name}.queries"]
        si = z[f"{name}.sample_inds"] if f"{name}.sample_inds" in z.files else None
        qsi = z[f"{name}.query_sample_inds"] if si is not None else None
        nb, cnt, dist = og.radius_search_sorted_grid8(
            pts, q, float(z[f"{name}.radius"]), si, qsi, return_distances=True)
        assert np.array_equal(cnt, z[f"{name}.num_neighbors"]), name
        ref_keys = _query_major_keys(z[f"{name}.neighbors"], z[f"{name}.num_neighbors"], len(pts))
        assert np.array_equal(_query_major_keys(nb, cnt, len(pts)), ref_keys), name
        # distances, compared pair by pair
        rq = np.repeat(np.arange(len(cnt)), z[f"{name}.num_neighbors"])
        order = np.lexsort((z[f"{name}.neighbors"], rq))
        assert np.array_equal(dist, z[f"{name}.distances"][order]), name


def test_tap_segments_match_reference(golden):
    z = golden("radius")
    for name in _case_names(z):
        pts, q = z[f"{name}.points"], z[f"{name}.queries"]
        si = z[f"{name}.sample_inds"] if f"{name}.sample_inds" in z.files else None
        qsi = z[f"{name}.query_sample_inds"] if si is not None else None
        K = int(z[f"{name}.kernel_size"])
        i, j, seg, cnt = og.radius_search_sorted_grid8_segments(
            pts, q, float(z[f"{name}.radius"]), K, float(z[f"{name}.kernel_grid_size"]), si, qsi)
        assert np.array_equal(seg, z[f"{name}.seg_offs"]), name
        assert np.array_equal(cnt, z[f"{name}.seg_num_neighbors"]), name
        k = np.repeat(np.arange(K ** 3), np.diff(seg))
        rk = np.repeat(np.arange(K ** 3), np.diff(z[f"{name}.seg_offs"]))
        assert np.array_equal(
            og.canonical_triplet_keys(i, j, k, len(q), len(pts)),
            og.canonical_triplet_keys(z[f"{name}.i"], z[f"{name}.j"], rk, len(q), len(pts))), name


def test_boundary_inclusion_known_answers(golden):
    # tests/unittest/test_grid_lookup_bounds.py:19-54: dist == R kept, R + 8 eps dropped
    z = golden("radius")
    nb, cnt = og.radius_search_sorted_grid8(
        z["alias_bounds.points"], z["alias_bounds.queries"], 1.0,
        z["alias_bounds.sample_inds"], z["alias_bounds.query_sample_inds"])
    assert cnt.tolist() == [3, 3]
    assert sorted(nb.tolist()) == [0, 1, 2, 4, 5, 6]


def test_division_is_correctly_rounded():
    # tests/unittest/test_radius_search_sorted_grid.py:314-343: 0.09/0.02 -> dx=+5
    k = og.voxelize_3d(15, np.array([[0.09, 0.0, 0.0]], np.float32), 0.02)
    assert k.tolist() == [(12 * 15 + 7) * 15 + 7]


def test_voxelize_matches_reference(golden):
    z = golden("voxelize")
    for ks in (1, 3, 5, 7, 15):
        assert np.array_equal(og.voxelize_3d(ks, z["offsets"], 0.02), z[f"k{ks}"])


def test_scalar_formulas(golden):
    z = golden("voxelize")
    got = [og.radius_scaler_for_kernel_size(3), og.radius_scaler_for_kernel_size(3, 2.5),
           og.radius_scaler_for_kernel_size(5, 2.5), og.radius_scaler_for_kernel_size(3, 1.0, "cube"),
           og.radius_scaler_for_kernel_size((1, 3, 5), 2.0)]
    assert np.allclose(got, z["radius_scaler"], rtol=0, atol=0)
    # tests/unittest/test_full_cover_strided.py:44-49
    s = og.full_cover_radius_scaler(8, 1e-2)
    assert s == pytest.approx(6.99748526, rel=1e-7)
    assert 0.05 * s == pytest.approx(0.34987426, rel=1e-7)
    assert og.minimum_full_cover_kernel_size(s) == 15
    assert og.minimum_full_cover_kernel_size(og.full_cover_radius_scaler(2)) == 5
    assert og.full_cover_radius_scaler(2) == pytest.approx(math.sqrt(3) * 1.01)


def test_empty_inputs():
    # tests/unittest/test_radius_search_sorted_grid.py:89-99,276-285
    for P, Q in ((0, 0), (0, 3), (3, 0)):
        nb, cnt = og.radius_search_sorted_grid8(np.zeros((P, 3)), np.zeros((Q, 3)), 1.0)
        assert nb.size == 0 and cnt.shape == (Q,)
        i, j, seg, cnt = og.radius_search_sorted_grid8_segments(
            np.zeros((P, 3)), np.zeros((Q, 3)), 0.2, 3, 0.2)
        assert i.size == 0 and j.size == 0 and np.array_equal(seg, np.zeros(28, np.int64))


def test_sparse_c_restatement_is_bit_exact_with_reference(golden):
    z = golden("sparse")
    for name in _case_names(z):
        a, b, go = z[f"{name}.a"], z[f"{name}.b"], z[f"{name}.go"]
        ai, bi, oi = z[f"{name}.a_idx"], z[f"{name}.b_idx"], z[f"{name}.o_idx"]
        n_o = int(z[f"{name}.n_o"])
        assert np.array_equal(os_.mvmr_c(a, ai, b, bi, oi, n_o), z[f"{name}.mvmr"]), name
        assert np.array_equal(os_.vvor_c(b, bi, go, oi, ai, a.shape[0]), z[f"{name}.vvor"]), name
        assert os_.rel_frobenius(os_.mvmr_f64(a, ai, b, bi, oi, n_o), z[f"{name}.mvmr"]) < 1e-6
        assert os_.rel_frobenius(os_.vvor_f64(b, bi, go, oi, ai, a.shape[0]), z[f"{name}.vvor"]) < 1e-6


def test_reference_cpu_ops_when_built(golden):
    if not os_.reference_ops_available():
        pytest.skip("reference CPU operators not built")
    z = golden("sparse")
    name = "c32"
    out = os_.mvmr_ref(z[f"{name}.a"], z[f"{name}.a_idx"], z[f"{name}.b"],
                       z[f"{name}.b_idx"], z[f"{name}.o_idx"], int(z[f"{name}.n_o"]))
    assert np.array_equal(out, z[f"{name}.mvmr"])


def _segment_cases(z, prefix):
    return sorted({k.split(".")[1] for k in z.files if k.startswith(prefix + ".")})


def test_segment_reduce_oracle_matches_reference_golden(golden):
    """oracle/segment_ops.py against the reference's Triton kernels (run under the
    interpreter): forward values and autograd gradients of both reductions."""
    from oracle import segment_ops as seg

    z = golden("segment")
    for name in _segment_cases(z, "large"):
        x, lengths, go = z[f"large.{name}.x"], z[f"large.{name}.lengths"], z[f"large.{name}.go"]
        for op in ("sum", "mean", "max", "min"):
            want = z[f"large.{name}.{op}"]
            got = seg.large_segment_reduce(x, lengths, op)
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5, err_msg=f"{name} {op}")
            grad = seg.large_segment_reduce_grad(go, x, want, lengths, op)
            np.testing.assert_allclose(grad, z[f"large.{name}.{op}.grad"], rtol=1e-5, atol=1e-6, err_msg=f"{name} {op}")
    for name in _segment_cases(z, "indexed"):
        x, idx = z[f"indexed.{name}.x"], z[f"indexed.{name}.indices"]
        lengths, go = z[f"indexed.{name}.lengths"], z[f"indexed.{name}.go"]
        for op in ("sum", "mean", "max", "min"):
            want = z[f"indexed.{name}.{op}"]
            got = seg.indexed_segment_reduce(x, idx, lengths, op)
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5, equal_nan=True, err_msg=f"{name} {op}")
            grad = seg.indexed_segment_reduce_grad(go, x, want, idx, lengths, op, len(x))
            np.testing.assert_allclose(grad, z[f"indexed.{name}.{op}.grad"], rtol=1e-5, atol=1e-6,
                                       err_msg=f"{name} {op}")


def test_ragged_norm_oracle_matches_reference_golden(golden):
    from oracle import segment_ops as seg

    z = golden("segment")
    for kind in ("layer", "instance", "group"):
        got = seg.ragged_norm(z["norm.x"], z["norm.lengths"], kind, num_groups=4, weight=z["norm.weight"],
                              bias=z["norm.bias"])
        np.testing.assert_allclose(got, z[f"norm.{kind}"], rtol=1e-4, atol=1e-5, err_msg=kind)
