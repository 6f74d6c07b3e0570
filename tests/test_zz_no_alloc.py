"""The workspace-free weight-gradient entry point, through the C ABI.

``pcx_vvor_static_scratch`` serves embedders that cannot allocate device
memory where they need the gradient (allocator callbacks, regions where
cudaMalloc is off limits, plugins that own nothing but the tensors passed in):
its scratch is a fixed array inside the library.  The test calls it twice in a
row on different inputs -- the second call must not see the first call's sums
-- and compares each result with the regular ``pcx_vvor`` entry point.  It is
collected last so that a stop-at-first-failure run has already executed every
other test, and it does not depend on anything another test left behind.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 2e-2}


def _inputs(seed, dtype, K, C, M, n_in, n_out, T):
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(seed)
    k = np.sort(rng.integers(0, K, T))
    i = rng.integers(0, n_out, T)
    order = np.lexsort((i, k))
    t = lambda x, d: torch.as_tensor(x).to(dev).to(d)
    return (t(rng.standard_normal((n_in, 1, C)), dtype), t(rng.integers(0, n_in, T), torch.int32),
            t(rng.standard_normal((n_out, 1, M)), dtype), t(i[order], torch.int32), t(k, torch.int32))


@pytest.mark.parametrize("dtype,C,M", [(torch.bfloat16, 64, 64), (torch.float32, 24, 40)])
def test_static_scratch_matches_workspace_entry_point_twice(dtype, C, M):
    from pointelligence_b200 import _cabi

    K = 27
    for call, seed in enumerate((11, 12)):
        x, j, go, i, k = _inputs(seed, dtype, K, C, M, 500, 450, 6000 + 500 * call)
        seg = _cabi.seg_offs_from_sorted(k, K)
        expected = _cabi.vvor(x, j, go, i, seg, None, K)
        out = torch.full((K, 1, C, M), float("nan"), dtype=dtype, device=x.device)
        before = torch.cuda.memory_allocated()
        _cabi.vvor_static_scratch(x, j, go, i, seg, out)
        assert torch.cuda.memory_allocated() == before          # the call allocated nothing through torch
        torch.cuda.synchronize()
        err = (out.float() - expected.float()).norm() / expected.float().norm()
        assert float(err) < TOL[dtype], (call, float(err))
        # and against the fp64 oracle, so that the entry point has a pin of its own
        from oracle import sparse_ops as oso

        ref = oso.vvor_f64(x.float().cpu().numpy(), j.cpu().numpy(), go.float().cpu().numpy(), i.cpu().numpy(),
                           k.cpu().numpy(), K)
        assert oso.rel_frobenius(out.float().cpu().numpy(), ref) < TOL[dtype], call
    assert _cabi.device_status() == 0


def test_static_scratch_rejects_oversized_outputs():
    from pointelligence_b200 import _cabi

    dev = torch.device("cuda:0")
    limit = _cabi.lib().pcx_vvor_static_scratch_max_elements()
    K, C = 27, 512                                              # 27 * 512 * 512 > 2^21
    assert K * C * C > limit
    x = torch.zeros((4, 1, C), dtype=torch.bfloat16, device=dev)
    idx = torch.zeros(2, dtype=torch.int32, device=dev)
    seg = torch.full((K + 1,), 2, dtype=torch.int64, device=dev)
    seg[0] = 0
    out = torch.empty((K, 1, C, C), dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        _cabi.vvor_static_scratch(x, idx, x, idx, seg, out)
