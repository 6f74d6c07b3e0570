"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE.

Usage (only where a checkout of the reference is importable; the produced
``.npz`` files are committed and are all the tests need):

    python tests/golden/make_golden.py --reference <checkout>

What runs, per file:

``downsample.npz``   ``internals.grid_sample.grid_sample_filter(...,
    center_nearest_impl="torch")`` on CPU tensors (the reference's own
    selector twin), inputs shaped like tests/unittest/
    test_grid_sample_selector.py:37-108 and test_grid_sample_regression.py.
``radius.npz``       ``internals.neighbors.radius_search_sorted_grid8`` and
    ``radius_search_sorted_grid8_segments`` -- the reference's Triton kernels
    executed by Triton's CPU interpreter (``TRITON_INTERPRET=1``).  The
    interpreter has no libdevice, so ``libdevice.div_rn`` / ``libdevice.rint``
    are mapped to numpy's IEEE fp32 divide and round-half-even, which is
    their definition.  Inputs follow tests/unittest/
    test_radius_search_sorted_grid.py:55-86,150-232,235-273,314-343 and
    test_grid_lookup_bounds.py:19-54.
``voxelize.npz``     ``layers.triplets.voxelize_3d`` and the scalar formulas.
``sparse.npz``       the reference's CPU MVMR / VVOR operators compiled from
    its C++ sources (oracle/build_ref.py).
``full_cover.npz``   ``layers.triplets.build_full_cover_strided_rulebook`` on CPU tensors.  Its body is
    plain torch except for ``radius_search`` (a Triton launch); that one name is pointed at the
    numpy restatement of the search (``oracle/geometry.py``, one rounding per operation like the
    interpreter), everything else -- centre choice, residual R-net selector, ordering, taps -- is
    the reference's own code.  Inputs: the fixture of tests/unittest/test_full_cover_strided.py:52-120
    and a two-sample synthetic scene with enough uncovered points to need the residual selector.
``segment.npz``      ``sparse_engines.ops.large_segment_reduce`` and
    ``indexed_segment_reduce`` (Triton kernels under the interpreter, forward
    and autograd backward) and ``layers.norm.Ragged{Layer,Instance,Group}Norm``
    (plain torch on CPU).

Inputs are stored next to the outputs so that no random-number generator has
to agree between machines.
"""
import argparse
import itertools
import math
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _patch_libdevice():
    import triton.language as tl
    from triton.language.extra import libdevice
    from triton.runtime.interpreter import TensorHandle

    def _np(x):
        return x.handle.data if hasattr(x, "handle") else np.float32(x)

    def div_rn(x, y):
        out = np.divide(_np(x).astype(np.float32), np.float32(_np(y))).astype(np.float32)
        return tl.tensor(TensorHandle(out, tl.float32), x.type)

    def rint(x):
        out = np.rint(_np(x)).astype(np.float32)
        return tl.tensor(TensorHandle(out, tl.float32), x.type)

    libdevice.div_rn = div_rn
    libdevice.rint = rint


def gen_downsample(torch, out):
    from internals.grid_sample import grid_sample_filter

    cases = {}
    g = torch.Generator().manual_seed(31)
    pts = torch.randn((6000, 3), generator=g) * 3.0
    si = torch.arange(pts.shape[0]) % 4
    cases["neg_multibatch"] = (pts, 0.2, si)
    g = torch.Generator().manual_seed(47)
    dense = torch.rand((1025, 3), generator=g) * 0.98 + 0.01
    tie = torch.tensor([[0.25, 0.5, 0.5], [0.75, 0.5, 0.5]])
    pts = torch.cat((tie, dense + 2.0, -dense - 2.0), dim=0)
    si = torch.cat((torch.zeros(tie.shape[0] + dense.shape[0]),
                    torch.ones(dense.shape[0]))).to(torch.long)
    cases["tie_dense"] = (pts, 1.0, si)
    pts = torch.tensor([[-1e-4, 0.25, 0.25], [-0.75, 0.25, 0.25], [1e-4, 0.25, 0.25]])
    cases["half_open_zero"] = (pts, 1.0, None)
    # points one ulp below / at / above cell multiples: floor-division corner cases
    n = torch.arange(1, 2001, dtype=torch.float32)
    edge = n * torch.tensor(0.04, dtype=torch.float32)
    x = torch.cat((torch.nextafter(edge, torch.zeros_like(edge)), edge,
                   torch.nextafter(edge, edge + 1), -edge,
                   torch.nextafter(-edge, torch.zeros_like(edge))))
    pts = torch.stack((x, x.flip(0) * 0.5, torch.zeros_like(x)), dim=1)
    cases["cell_edges"] = (pts, 0.04, None)
    g = torch.Generator().manual_seed(5)
    pts = torch.rand((5000, 3), generator=g) * torch.tensor([6.0, 6.0, 3.0])
    si = torch.sort(torch.randint(0, 3, (5000,), generator=g)).values
    cases["indoor_like"] = (pts, 0.04, si)
    for name, (pts, cell, si) in cases.items():
        p_f, si_f, idx, mapping = grid_sample_filter(
            pts, cell, sample_inds=si, reduction="center_nearest",
            return_mapping=True, center_nearest_impl="torch")
        out[f"{name}.points"] = pts.numpy()
        out[f"{name}.cell"] = np.float64(cell)
        if si is not None:
            out[f"{name}.sample_inds"] = si.numpy().astype(np.int64)
            out[f"{name}.out_sample_inds"] = si_f.numpy().astype(np.int64)
        out[f"{name}.out_points"] = p_f.numpy()
        out[f"{name}.out_indices"] = idx.numpy().astype(np.int64)
        out[f"{name}.out_mapping"] = mapping.numpy().astype(np.int64)


def gen_radius(torch, out):
    from internals.neighbors import (radius_search_sorted_grid8,
                                     radius_search_sorted_grid8_segments)

    eps = float(np.finfo(np.float32).eps)
    cases = {}
    # boundary + batches (test_radius_search_sorted_grid.py:55-86)
    radius = 1.0
    offs = torch.tensor(list(itertools.product((-1.0, 0.0, 1.0), repeat=3)))
    p0 = torch.cat((offs * (radius - 8 * eps), torch.tensor([
        [radius, 0, 0], [radius + 8 * eps, 0, 0],
        [-radius, 0, 0], [-radius - 8 * eps, 0, 0]])))
    pts = torch.cat((p0, p0))
    q = torch.zeros((2, 3))
    s = torch.cat((torch.zeros(p0.shape[0], dtype=torch.long),
                   torch.ones(p0.shape[0], dtype=torch.long)))
    cases["boundary_batches"] = dict(points=pts, queries=q, radius=radius,
                                     sample_inds=s, query_sample_inds=torch.arange(2),
                                     kernel_size=3, kernel_grid_size=0.75)
    # key aliasing (test_grid_lookup_bounds.py:19-54)
    one = torch.tensor([[-1.0, 0, 0], [0, 0, 0], [1.0, 0, 0], [1.0 + 8 * eps, 0, 0]])
    cases["alias_bounds"] = dict(points=torch.cat((one, one)), queries=torch.zeros((2, 3)),
                                 radius=1.0,
                                 sample_inds=torch.repeat_interleave(torch.arange(2), 4),
                                 query_sample_inds=torch.arange(2),
                                 kernel_size=3, kernel_grid_size=1.0)
    # two ragged samples, separate query set (…sorted_grid.py:150-232), K=3 and K=15
    for ks, rad, kg in ((3, 0.05, 0.05), (15, math.sqrt(3) * 0.2 * 1.01, 0.05)):
        g = torch.Generator().manual_seed(29 + ks)
        n0, n1, m0, m1 = (700, 500, 90, 70) if ks == 3 else (260, 180, 40, 30)
        pp = [torch.rand(n0, 3, generator=g) * 1.8 - 0.9, torch.rand(n1, 3, generator=g) * 1.4 - 0.5]
        qq = [torch.rand(m0, 3, generator=g) * 1.8 - 0.9, torch.rand(m1, 3, generator=g) * 1.4 - 0.5]
        if ks == 3:  # denser so that R=0.05 finds neighbours
            pp = [x * 0.25 for x in pp]
            qq = [x * 0.25 for x in qq]
        cases[f"ragged_k{ks}"] = dict(
            points=torch.cat(pp), queries=torch.cat(qq), radius=rad,
            sample_inds=torch.cat([torch.full((x.shape[0],), b, dtype=torch.int32)
                                   for b, x in enumerate(pp)]),
            query_sample_inds=torch.cat([torch.full((x.shape[0],), b, dtype=torch.int32)
                                         for b, x in enumerate(qq)]),
            kernel_size=ks, kernel_grid_size=kg)
    # round-half-even ties (…sorted_grid.py:235-273)
    cases["tap_ties"] = dict(points=torch.tensor([
        [-0.75, 0, 0], [-0.25, 0, 0], [0.25, 0, 0], [0.75, 0, 0],
        [0, -0.75, 0.25], [0, 0.75, -0.25]]), queries=torch.zeros((1, 3)), radius=1.0,
        sample_inds=None, query_sample_inds=None, kernel_size=5, kernel_grid_size=0.5)
    # correctly rounded division (…sorted_grid.py:314-343)
    cases["div_rn"] = dict(points=torch.tensor([[0.09, 0.0, 0.0]]), queries=torch.zeros((1, 3)),
                           radius=0.1, sample_inds=None, query_sample_inds=None,
                           kernel_size=15, kernel_grid_size=0.02)
    # self query, single sample, surface-like slab
    g = torch.Generator().manual_seed(3)
    pts = torch.rand(900, 3, generator=g) * torch.tensor([0.6, 0.6, 0.02]) - 0.1
    cases["self_slab"] = dict(points=pts, queries=pts, radius=0.05, sample_inds=None,
                              query_sample_inds=None, kernel_size=3, kernel_grid_size=0.02)
    for name, c in cases.items():
        pts, q = c["points"].float(), c["queries"].float()
        nb, cnt, dist = radius_search_sorted_grid8(
            pts, q, c["radius"], c["sample_inds"], c["query_sample_inds"],
            return_distances=True)
        i, j, seg, cnt2 = radius_search_sorted_grid8_segments(
            pts, q, c["radius"], c["kernel_size"], c["kernel_grid_size"],
            c["sample_inds"], c["query_sample_inds"])
        out[f"{name}.points"] = pts.numpy()
        out[f"{name}.queries"] = q.numpy()
        out[f"{name}.radius"] = np.float64(c["radius"])
        out[f"{name}.kernel_size"] = np.int64(c["kernel_size"])
        out[f"{name}.kernel_grid_size"] = np.float64(c["kernel_grid_size"])
        if c["sample_inds"] is not None:
            out[f"{name}.sample_inds"] = c["sample_inds"].numpy().astype(np.int64)
            out[f"{name}.query_sample_inds"] = c["query_sample_inds"].numpy().astype(np.int64)
        out[f"{name}.neighbors"] = nb.numpy().astype(np.int64)
        out[f"{name}.num_neighbors"] = cnt.numpy().astype(np.int64)
        out[f"{name}.distances"] = dist.numpy()
        out[f"{name}.i"] = i.numpy().astype(np.int32)
        out[f"{name}.j"] = j.numpy().astype(np.int32)
        out[f"{name}.seg_offs"] = seg.numpy().astype(np.int64)
        out[f"{name}.seg_num_neighbors"] = cnt2.numpy().astype(np.int64)
        print(name, "edges", nb.numel(), "taps used", int((seg.diff() > 0).sum()))


def gen_voxelize(torch, out):
    from layers.triplets import (full_cover_radius_scaler, minimum_full_cover_kernel_size,
                                 radius_scaler_for_kernel_size, voxelize_3d)

    g = torch.Generator().manual_seed(11)
    offs = (torch.rand(4000, 3, generator=g) - 0.5) * 0.2
    ties = torch.tensor([[0.01, -0.01, 0.03], [0.05, -0.05, 0.07], [0.09, 0.0, 0.0],
                         [-0.03, 0.03, -0.09], [0.5, -0.5, 0.0]])
    offs = torch.cat((offs, ties))
    out["offsets"] = offs.numpy()
    for ks in (1, 3, 5, 7, 15):
        out[f"k{ks}"] = voxelize_3d(ks, offs, torch.tensor(0.02)).numpy().astype(np.int32)
    out["radius_scaler"] = np.array([
        radius_scaler_for_kernel_size(3), radius_scaler_for_kernel_size(3, 2.5),
        radius_scaler_for_kernel_size(5, 2.5), radius_scaler_for_kernel_size(3, 1.0, "cube"),
        radius_scaler_for_kernel_size((1, 3, 5), 2.0)])
    out["full_cover"] = np.array([full_cover_radius_scaler(8, 1e-2), full_cover_radius_scaler(2),
                                  float(minimum_full_cover_kernel_size(full_cover_radius_scaler(8, 1e-2))),
                                  float(minimum_full_cover_kernel_size(full_cover_radius_scaler(2)))])


def gen_sparse(torch, out):
    sys.path.insert(0, ROOT)
    from oracle import sparse_ops

    rng = np.random.default_rng(7)
    for name, (K, G, C, M, Nb, No, T) in {
        "c32": (27, 1, 32, 32, 300, 280, 4000),
        "c5_m20": (27, 1, 5, 20, 120, 120, 900),
        "c1": (8, 1, 1, 16, 64, 64, 300),
        "g2": (27, 2, 12, 8, 150, 140, 1500),
        "c40": (5, 1, 40, 24, 90, 70, 600),
    }.items():
        a = rng.standard_normal((K, G, C, M)).astype(np.float32)
        b = rng.standard_normal((Nb, G, C)).astype(np.float32)
        go = rng.standard_normal((No, G, M)).astype(np.float32)
        ai = np.sort(rng.integers(0, K, T)).astype(np.int32)
        bi = rng.integers(0, Nb, T).astype(np.int32)
        oi = rng.integers(0, No, T).astype(np.int32)
        out[f"{name}.a"], out[f"{name}.b"], out[f"{name}.go"] = a, b, go
        out[f"{name}.a_idx"], out[f"{name}.b_idx"], out[f"{name}.o_idx"] = ai, bi, oi
        out[f"{name}.n_o"] = np.int64(No)
        out[f"{name}.mvmr"] = sparse_ops.mvmr_ref(a, ai, b, bi, oi, No)
        # weight gradient as the reference composes it (mvmr_triton.py:286-296)
        out[f"{name}.vvor"] = sparse_ops.vvor_ref(b, bi, go, oi, ai, K)


def gen_full_cover(torch, out):
    sys.path.insert(0, ROOT)
    import layers.triplets as rt
    from oracle import geometry as og
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    def restated_radius_search(points, query_points, radius, sample_inds=None, query_sample_inds=None, **_):
        nb, counts = og.radius_search_sorted_grid8(
            points.numpy(), query_points.numpy(), float(radius),
            None if sample_inds is None else sample_inds.numpy(),
            None if query_sample_inds is None else query_sample_inds.numpy())
        return torch.from_numpy(nb), torch.from_numpy(counts)

    rt.radius_search = restated_radius_search
    p0 = torch.tensor([[0.001, 0.001, 0.001], [0.399, 0.399, 0.399], [0.401, 0.001, 0.001], [0.799, 0.399, 0.399]])
    cases = {"fixture": (torch.cat([p0, p0 + torch.tensor([2.0, 0.0, 0.0])]),
                         torch.cat([torch.zeros(4, dtype=torch.long), torch.ones(4, dtype=torch.long)]), 8, 0.05, 15)}
    pts, inds, _ = ragged_batch([indoor_scene(3000, 5), indoor_scene(2000, 6)])
    cases["scene"] = (torch.from_numpy(pts), torch.from_numpy(inds).long(), 2, 0.02, 5)
    # a slab whose points avoid the middle of every stride cell: the initial centres sit off-centre,
    # their balls miss the far corners, thousands of points stay uncovered and the residual selector
    # runs for several rounds (past its 2048-point dense branch, i.e. through radius_search)
    g = torch.Generator().manual_seed(9)
    slab = torch.rand(40000, 3, generator=g) * torch.tensor([2.0, 2.0, 0.16])
    cell = 8 * 0.02
    off = slab[:, :2] - (torch.floor(slab[:, :2] / cell) + 0.5) * cell
    slab = slab[off.norm(dim=1) > 0.07]
    cases["hollow_cells"] = (slab, (torch.arange(slab.shape[0]) >= slab.shape[0] // 2).long(), 8, 0.02, 15)
    for name, (points, sample, stride, grid, ks) in cases.items():
        rb = rt.build_full_cover_strided_rulebook(points, sample, torch.bincount(sample), stride=stride,
                                                  input_grid_size=grid, kernel_size=ks)
        n, nc = points.shape[0], rb.points.shape[0]
        out[f"{name}.points"], out[f"{name}.sample_inds"] = points.numpy(), sample.numpy()
        out[f"{name}.stride"], out[f"{name}.grid"], out[f"{name}.kernel_size"] = np.float64(stride), np.float64(grid), np.int64(ks)
        for f in ("center_source_indices", "initial_center_source_indices", "additional_center_source_indices",
                  "point_to_initial_center", "num_neighbors", "coverage_per_input", "initial_center_counts",
                  "additional_center_counts", "sample_sizes"):
            out[f"{name}.{f}"] = getattr(rb, f).numpy().astype(np.int64)
        out[f"{name}.radius"] = np.float64(rb.radius)
        out[f"{name}.rounds"] = np.int64(rb.selector_round_count)
        # edges in canonical order (the order inside a tap is unspecified)
        key = (rb.k.long() * nc + rb.i.long()) * n + rb.j.long()
        out[f"{name}.edges"] = torch.sort(key).values.numpy()
        key = (rb.k_upsample.long() * n + rb.i_upsample.long()) * nc + rb.j_upsample.long()
        out[f"{name}.edges_upsample"] = torch.sort(key).values.numpy()
        print(name, "centres", nc, "initial", rb.initial_center_source_indices.numel(), "added",
              rb.additional_center_source_indices.numel(), "rounds", rb.selector_round_count, "edges", rb.i.numel())


def gen_segment(torch, out):
    """Segment reductions (Triton kernels under the interpreter, forward and
    autograd backward) and the ragged norm layers (plain torch on CPU)."""
    # interpreted kernels are plain callables: torch's wrapper (which only accepts compiled
    # kernels) is bypassed before the reference modules import it
    import torch.library

    torch.library.wrap_triton = lambda kernel: kernel
    from layers.norm import RaggedGroupNorm, RaggedInstanceNorm, RaggedLayerNorm
    from sparse_engines.ops import indexed_segment_reduce, large_segment_reduce
    import sparse_engines.indexed_segment_reduce_triton as isr

    # the forward kernel is wrapped in an autotuner (launch parameters only), which wants
    # a GPU to time its candidates: run the kernel it wraps
    isr.indexed_segment_reduce_fwd_kernel = isr.indexed_segment_reduce_fwd_kernel.fn

    rng = np.random.default_rng(11)
    with torch.enable_grad():
        for name, (lengths, C) in {
            "ragged": ([70, 0, 5, 130, 1, 64], 20),      # boundaries inside and at block edges, an empty segment
            "single": ([200], 33),
            "wide": ([3, 90, 40], 96),
        }.items():
            n = int(sum(lengths))
            x = np.round(rng.standard_normal((n, C)) * 4).astype(np.float32) / 4   # ties for max / min
            go = rng.standard_normal((len(lengths), C)).astype(np.float32)
            out[f"large.{name}.x"], out[f"large.{name}.lengths"], out[f"large.{name}.go"] = x, np.asarray(lengths), go
            for op in ("sum", "mean", "max", "min"):
                xt = torch.from_numpy(x).requires_grad_(True)
                y = large_segment_reduce(xt, op, lengths=torch.tensor(lengths))
                y.backward(torch.from_numpy(go))
                out[f"large.{name}.{op}"] = y.detach().numpy()
                out[f"large.{name}.{op}.grad"] = xt.grad.numpy()
        for name, (lengths, n_x, C) in {
            "pool": ([3, 1, 4, 2, 0, 7, 1], 12, 16),
            "wide": ([5, 5, 9, 1], 30, 70),
        }.items():
            E = int(sum(lengths))
            x = np.round(rng.standard_normal((n_x, C)) * 4).astype(np.float32) / 4
            idx = rng.integers(0, n_x, E).astype(np.int64)
            go = rng.standard_normal((len(lengths), C)).astype(np.float32)
            out[f"indexed.{name}.x"], out[f"indexed.{name}.indices"] = x, idx
            out[f"indexed.{name}.lengths"], out[f"indexed.{name}.go"] = np.asarray(lengths), go
            for op in ("sum", "mean", "max", "min"):
                xt = torch.from_numpy(x).requires_grad_(True)
                y = indexed_segment_reduce(xt, op, torch.from_numpy(idx), lengths=torch.tensor(lengths))
                y.backward(torch.from_numpy(go))
                out[f"indexed.{name}.{op}"] = y.detach().numpy()
                out[f"indexed.{name}.{op}.grad"] = xt.grad.numpy()
    lengths = [40, 7, 90]
    x = rng.standard_normal((sum(lengths), 24)).astype(np.float32)
    w = rng.standard_normal(24).astype(np.float32)
    b = rng.standard_normal(24).astype(np.float32)
    out["norm.x"], out["norm.lengths"], out["norm.weight"], out["norm.bias"] = x, np.asarray(lengths), w, b
    for kind, layer in (("layer", RaggedLayerNorm(24)), ("instance", RaggedInstanceNorm(24, affine=True)),
                        ("group", RaggedGroupNorm(4, 24))):
        layer.weight.data = torch.from_numpy(w)
        layer.bias.data = torch.from_numpy(b)
        out[f"norm.{kind}"] = layer(torch.from_numpy(x), torch.tensor(lengths)).detach().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("POINTELLIGENCE_REFERENCE",
                                                           os.path.join(os.path.dirname(ROOT), "reference")))
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import torch

    _patch_libdevice()
    gens = dict(downsample=gen_downsample, radius=gen_radius, voxelize=gen_voxelize,
                sparse=gen_sparse, segment=gen_segment, full_cover=gen_full_cover)
    for name, fn in gens.items():
        if args.only and name not in args.only.split(","):
            continue
        out = {}
        with torch.no_grad():
            fn(torch, out)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
        print("wrote", name, len(out), "arrays")


if __name__ == "__main__":
    main()
