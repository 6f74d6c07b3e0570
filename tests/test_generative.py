"""Generative rulebooks on the CPU: the stamp-and-deduplicate builder against a brute-force set
computation, the closed-form subdivision generator, the contracts they ship and the
at-least-one-contributor check."""
import numpy as np
import pytest
import torch

from pointelligence_b200.layers.generative import (CoordinateGenerator, GeneratedSites, KernelStampGenerator,
                                                   SubdivisionGenerator, build_generative_triplets)
from pointelligence_b200.layers.metadata import MetaData


def _cloud(n=200, seed=0):
    g = torch.Generator().manual_seed(seed)
    pts = torch.rand(n, 3, generator=g) * 0.5 - 0.1
    smp = (torch.arange(n) >= int(0.6 * n)).long()
    return pts, smp, torch.bincount(smp)


def test_stamp_rulebook_against_brute_force():
    pts, smp, sizes = _cloud()
    n, K, fine = pts.shape[0], 27, 0.05
    s = build_generative_triplets(pts, smp, sizes, 0.1, (3, 3, 3), 2.0)
    s.validate()
    assert s.i.numel() == n * K and s.uniform_seg_len == n and s.grid_size == fine
    assert s.i.dtype == torch.int32 and bool((s.k[1:] >= s.k[:-1]).all())
    voxel = np.floor_divide(pts.numpy().astype(np.float32), np.float32(fine)).astype(np.int64)
    stencil = np.array([(a - 1, b - 1, c - 1) for a in range(3) for b in range(3) for c in range(3)])
    cell = lambda j, k: (int(smp[j]),) + tuple((voxel[j] + stencil[k])[::-1].tolist())   # (sample, z, y, x)
    cells = sorted({cell(j, k) for j in range(n) for k in range(K)})
    assert len(cells) == s.n_out and not s.exact_cover_out
    row = {c: r for r, c in enumerate(cells)}
    for t in range(n * K):
        assert row[cell(int(s.j[t]), int(s.k[t]))] == int(s.i[t])
    centres = (np.array([[c[3], c[2], c[1]] for c in cells]) + 0.5) * fine
    assert np.allclose(s.points.numpy(), centres, atol=1e-6)
    assert np.array_equal(s.sample_inds.numpy(), np.array([c[0] for c in cells]))
    assert s.sample_sizes.tolist() == np.bincount([c[0] for c in cells], minlength=2).tolist()
    by_row = build_generative_triplets(pts, smp, sizes, 0.1, (3, 3, 3), 2.0, sort_by="i")
    assert bool((by_row.i[1:] >= by_row.i[:-1]).all()) and by_row.uniform_seg_len is None
    key = lambda g: sorted(zip(g.i.tolist(), g.j.tolist(), g.k.tolist()))
    assert key(by_row) == key(s)
    with pytest.raises(ValueError):
        build_generative_triplets(pts, smp, sizes, 0.1, sort_by="j")


def test_custom_stencil_empty_input_and_contracts():
    pts, smp, sizes = _cloud(50, seed=1)
    stencil = torch.tensor([[0, 0, 0], [1, 0, 0], [0, 0, -1]])
    gen = KernelStampGenerator(3, expansion=1.0, stencil=stencil)
    assert isinstance(gen, CoordinateGenerator) and gen.kernel_taps == 3
    m = MetaData(points=pts, sample_inds=smp, sample_sizes=sizes, grid_size=0.1, auto_build_triplets=False)
    s = gen(m)
    assert s.i.numel() == 150 and s.to_contract().uniform_seg_len == 50 and s.to_contract().k_sorted
    out = s.to_metadata(parent=m)
    assert out.parent is m and out.points.shape[0] == s.n_out and out.contract == s.to_contract()
    empty = build_generative_triplets(pts[:0], smp[:0], sizes, 0.1)
    assert empty.n_out == 0 and empty.i.numel() == 0 and empty.sample_sizes.tolist() == [0, 0]
    empty.validate()
    with pytest.raises(ValueError):
        KernelStampGenerator(3, expansion=0.5)
    broken = GeneratedSites(points=torch.zeros(3, 3), sample_inds=torch.zeros(3, dtype=torch.long),
                            sample_sizes=torch.tensor([3]), grid_size=1.0, i=torch.tensor([0, 0, 2]),
                            j=torch.tensor([0, 1, 2]), k=torch.tensor([0, 0, 0]))
    with pytest.raises(RuntimeError):
        broken.validate()


def test_subdivision_is_closed_form_and_injective():
    pts, smp, sizes = _cloud(64, seed=2)
    grid = 0.1
    centred = (torch.div(pts, grid, rounding_mode="floor") + 0.5) * grid     # voxel-centred input
    m = MetaData(points=centred, sample_inds=smp, sample_sizes=sizes, grid_size=grid, auto_build_triplets=False)
    s = SubdivisionGenerator(2)(m)
    s.validate()
    n = 64
    assert s.n_out == 8 * n and s.exact_cover_out and s.uniform_seg_len == n and s.grid_size == grid / 2
    assert torch.equal(s.i.long(), torch.arange(8 * n)) and torch.equal(s.j.long(), torch.arange(n).repeat(8))
    parent_voxel = torch.div(s.points, grid, rounding_mode="floor")
    assert torch.equal(parent_voxel, torch.div(centred, grid, rounding_mode="floor")[s.j.long()])   # children tile the parent
    rows = lambda p, b: torch.unique(torch.cat([p, b.unsqueeze(1).to(p.dtype)], 1), dim=0).shape[0]
    assert rows(s.points, s.sample_inds) == 8 * rows(centred, smp)      # distinct parents have distinct children
    with pytest.raises(ValueError):
        SubdivisionGenerator(1.5)
    assert SubdivisionGenerator(3).kernel_taps == 27
