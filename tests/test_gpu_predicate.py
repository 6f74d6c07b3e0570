"""The library's default radius predicate against the compiled form of the reference's expression.

The reference decides membership with ``tl.sqrt(dx*dx + dy*dy + dz*dz) <= radius``
(sparse_engines/strided_grid_radius_triton_kernel.py:25-31,127); what that means on a GPU is
whatever Triton's compiler makes of it (it contracts the sum into fused multiply-adds).  A Triton
kernel written here evaluates exactly that expression on 1,048,576 (query, point) pairs placed
within 3 ulp of the radius -- the only place where the rounding of the sum can change the answer --
and the per-query neighbour counts must equal those of the library's default predicate ("fma")
on every query.  The one-rounding-per-operation form ("ieee", what Triton's CPU interpreter and
numpy compute, used for the golden vectors) is counted too, to show the shell is not empty.
Skipped when Triton is not installed.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

triton = pytest.importorskip("triton")
tl = pytest.importorskip("triton.language")


@triton.jit
def _count_kernel(q_ptr, p_ptr, out_ptr, radius, per: tl.constexpr):
    qi = tl.program_id(0)
    lane = tl.arange(0, per)
    qx = tl.load(q_ptr + qi * 3 + 0)
    qy = tl.load(q_ptr + qi * 3 + 1)
    qz = tl.load(q_ptr + qi * 3 + 2)
    base = (qi * per + lane) * 3
    px = tl.load(p_ptr + base + 0)
    py = tl.load(p_ptr + base + 1)
    pz = tl.load(p_ptr + base + 2)
    dx = qx - px
    dy = qy - py
    dz = qz - pz
    dist = tl.sqrt(dx * dx + dy * dy + dz * dz)
    tl.store(out_ptr + qi, tl.sum((dist <= radius).to(tl.int32), axis=0))


def _shell_inputs(n_queries=4096, per=256, radius=0.05):
    rng = np.random.default_rng(0)
    q = (rng.random((n_queries, 3)) * 50).astype(np.float32)  # queries far apart: no cross pairs
    d = rng.standard_normal((n_queries, per, 3))
    d /= np.linalg.norm(d, axis=-1, keepdims=True)
    scale = radius * (1 + rng.integers(-3, 4, (n_queries, per, 1)) * 2.0 ** -24)
    p = (q[:, None, :].astype(np.float64) + d * scale).astype(np.float32).reshape(-1, 3)
    return q, p, radius


def test_default_predicate_equals_compiled_reference_expression():
    from pointelligence_b200.internals.neighbors import radius_predicate, radius_search_sorted_grid8

    q, p, radius = _shell_inputs()
    dev = torch.device("cuda:0")
    qt, pt = torch.from_numpy(q).to(dev), torch.from_numpy(p).to(dev)
    expect = torch.zeros(len(q), dtype=torch.int32, device=dev)
    _count_kernel[(len(q),)](qt, pt, expect, float(radius), per=256)
    expect = expect.cpu().numpy().astype(np.int64)
    assert 0 < expect.sum() < len(p)                       # the shell straddles the radius

    _, counts = radius_search_sorted_grid8(pt, qt, radius)  # library default
    assert np.array_equal(counts.cpu().numpy(), expect)
    with radius_predicate("fma"):
        _, counts = radius_search_sorted_grid8(pt, qt, radius)
    assert np.array_equal(counts.cpu().numpy(), expect)
    with radius_predicate("ieee"):
        _, counts = radius_search_sorted_grid8(pt, qt, radius)
    differ = int((counts.cpu().numpy() != expect).sum())
    assert differ > 0, "the boundary shell no longer separates the two roundings"
