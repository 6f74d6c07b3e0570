"""CPU-only tests: the C-ABI library loads and exports what the header
declares, host-side logic, loud failure without CUDA, data-parallel plumbing
over gloo with two ranks."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import ctypes

    from pointelligence_b200 import _cabi, build

    build.build()
    header = open(os.path.join(ROOT, "include", "pointelligence_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(pcx_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 16
    handle = ctypes.CDLL(_cabi.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared but not exported"
        assert name in _cabi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_cabi.SIGNATURES) == declared
    assert _cabi.lib().pcx_version() >= 10000


def test_operators_fail_loudly_without_cuda():
    from pointelligence_b200.internals.grid_sample import grid_sample_filter
    from pointelligence_b200.internals.neighbors import radius_search
    from pointelligence_b200.sparse_engines.ops import sparse_matrix_vector_multiplication_reduction as mvmr

    p = torch.rand(10, 3)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        radius_search(p, p, 0.5)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        grid_sample_filter(p, 0.1)
    a = torch.rand(3, 1, 4, 4)
    b = torch.rand(5, 1, 4)
    idx = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mvmr(a, idx, b, idx, idx, 5, torch.tensor([0, 2, 2, 2]))


def test_dispatch_and_precision_modes():
    from pointelligence_b200.sparse_engines._dispatch_override import (current_engine, current_mode,
                                                                       current_precision, dispatch_mode,
                                                                       precision_mode, resolve_input_precision)

    assert current_mode() == "auto" and current_engine() == 0
    with dispatch_mode("force_pt"):
        assert current_mode() == "force_pt" and current_engine() == 1
        with dispatch_mode("force_fgs"):
            assert current_mode() == "force_fused_gather_sum"
    assert current_mode() == "auto"
    with pytest.raises(ValueError, match="renamed"):
        with dispatch_mode("force_smig"):
            pass
    with pytest.raises(ValueError, match="unknown dispatch mode"):
        with dispatch_mode("nope"):
            pass
    assert resolve_input_precision(torch.bfloat16) == "tf32"
    with precision_mode("ieee"):
        assert current_precision() == "ieee" and resolve_input_precision(torch.float32) == "ieee"
    with pytest.raises(ValueError):
        with precision_mode("fp8"):
            pass


def test_host_formulas_and_voxelize(golden):
    from pointelligence_b200.layers import (full_cover_radius_scaler, minimum_full_cover_kernel_size,
                                            radius_scaler_for_kernel_size, voxelize_3d)

    z = golden("voxelize")
    got = [radius_scaler_for_kernel_size(3), radius_scaler_for_kernel_size(3, 2.5),
           radius_scaler_for_kernel_size(5, 2.5), radius_scaler_for_kernel_size(3, 1.0, "cube"),
           radius_scaler_for_kernel_size((1, 3, 5), 2.0)]
    assert np.array_equal(np.array(got), z["radius_scaler"])
    assert full_cover_radius_scaler(8, 1e-2) == pytest.approx(6.99748526, rel=1e-7)
    assert minimum_full_cover_kernel_size(full_cover_radius_scaler(8, 1e-2)) == 15
    offs = torch.from_numpy(z["offsets"])
    for ks in (1, 3, 5, 7, 15):
        assert np.array_equal(voxelize_3d(ks, offs, torch.tensor(0.02)).numpy(), z[f"k{ks}"])


def test_pointconv3d_parameters_and_legacy_checkpoint():
    from pointelligence_b200.layers import PointConv3d, TripletContract

    torch.manual_seed(0)
    conv = PointConv3d(8, 12, 3, groups=2, bias=True)
    assert conv.weight.shape == (27, 2, 4, 6) and conv.bias.shape == (12,)
    bound = 1.0 / np.sqrt(6 * 27)
    assert float(conv.weight.abs().max()) <= bound
    legacy = torch.randn(8, 6, 27)
    conv.load_state_dict({"weight": legacy, "bias": torch.zeros(12)})
    expect = legacy.reshape(2, 4, 6, 27).permute(3, 0, 1, 2)
    assert torch.equal(conv.weight.data, expect)
    c = TripletContract.submanifold()
    assert c.k_sorted and not c.exact_cover_out and c.uniform_seg_len is None
    with pytest.raises(ValueError):
        PointConv3d(7, 12, 3, groups=2)


def test_synthetic_generators_are_deterministic():
    from pointelligence_b200.synthetic import indoor_scene, lidar_sweep, ragged_batch

    a, b = indoor_scene(5000, 3), indoor_scene(5000, 3)
    assert a.dtype == np.float32 and a.shape == (5000, 3) and np.array_equal(a, b)
    cells = np.floor(a / np.float32(0.02)).astype(np.int64)
    assert len(np.unique(cells, axis=0)) == 5000          # voxel de-duplicated
    l = lidar_sweep(100)
    assert 80000 < len(l) < 131072 and np.array_equal(l, lidar_sweep(100))
    pts, inds, sizes = ragged_batch([a, l[:100]])
    assert pts.shape == (5100, 3) and sizes.tolist() == [5000, 100] and inds[-1] == 1


def test_partition_scenes_balances_and_covers():
    from pointelligence_b200.dist import partition_scenes

    rng = np.random.default_rng(1000)
    sizes = rng.integers(80000, 200001, 16).tolist()
    for world in (1, 2, 4, 8):
        owned = partition_scenes(sizes, world)
        assert sorted(s for o in owned for s in o) == list(range(16))
        loads = [sum(sizes[s] for s in o) for o in owned]
        assert max(loads) <= sum(sizes) / world + max(sizes)
    assert partition_scenes(sizes, 2) == partition_scenes(sizes, 2)


_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from pointelligence_b200.dist import allreduce_gradients, partition_scenes
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%s" % sys.argv[2],
                        rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
torch.manual_seed(0)
params = [torch.nn.Parameter(torch.zeros(27, 1, 8, 8)), torch.nn.Parameter(torch.zeros(8)),
          torch.nn.Parameter(torch.zeros(3, 3))]
params[0].grad = torch.full_like(params[0], float(rank + 1))
params[1].grad = torch.arange(8.0) * (rank + 1)
# params[2] has no gradient on rank 1 only
if rank == 0:
    params[2].grad = torch.ones(3, 3)
allreduce_gradients(params, average=True, bucket_bytes=4096)
assert torch.allclose(params[0].grad, torch.full_like(params[0], 1.5))
assert torch.allclose(params[1].grad, torch.arange(8.0) * 1.5)
assert torch.allclose(params[2].grad, torch.full((3, 3), 0.5))
owned = partition_scenes([5, 9, 7, 3], 2)
assert sorted(owned[0] + owned[1]) == [0, 1, 2, 3]
# the reducer that overlaps with backward: a small network whose ranks see different data, one
# parameter unused on rank 1, two steps through the same reducer, against a plain all-reduce
from pointelligence_b200.dist import OverlappedGradientReducer
torch.manual_seed(1)
net = torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.ReLU(), torch.nn.Linear(16, 16), torch.nn.ReLU(),
                          torch.nn.Linear(16, 3))
extra = torch.nn.Parameter(torch.ones(4))
params = list(net.parameters()) + [extra]
reducer = OverlappedGradientReducer(params, average=True, bucket_bytes=600)
assert len(reducer.buckets) >= 3
for step in range(2):
    for p in params:
        p.grad = None
    x = torch.randn(5, 6, generator=torch.Generator().manual_seed(10 * step + rank))
    loss = net(x).square().sum() + (extra.sum() * (rank == 0))
    loss.backward()
    local = [None if p.grad is None else p.grad.clone() for p in params]
    reducer.finish()
    for p, g in zip(params, local):
        want = torch.zeros_like(p) if g is None else g
        dist.all_reduce(want)
        assert torch.allclose(p.grad, want / 2, atol=1e-6), (step, p.shape)
reducer.remove()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_gradient_allreduce_two_ranks_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert f"rank {r} ok" in o


def test_radius_predicate_switch_is_scoped():
    from pointelligence_b200 import _cabi
    from pointelligence_b200.internals.neighbors import radius_predicate

    lib = _cabi.lib()
    default = lib.pcx_get_radius_predicate()
    assert default in (0, 1, 2)
    with radius_predicate("ieee"):
        assert lib.pcx_get_radius_predicate() == 0
        with radius_predicate("fma"):
            assert lib.pcx_get_radius_predicate() == 1
        assert lib.pcx_get_radius_predicate() == 0
    assert lib.pcx_get_radius_predicate() == default
    with pytest.raises(ValueError):
        with radius_predicate("exact"):
            pass


def test_bench_reference_arm_prints_the_contract_line():
    import json

    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "Gtriplets/s" and line["value"] > 0
    assert line["cpu_baseline"]["cores"] == 1 and line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    assert line["config"]["workload"].startswith("indoor150k_c64_bf16") and line["vs_baseline"] is None


def test_block_layers_construct_on_cpu_and_fail_loudly_without_cuda():
    """The norm / pooling layers and the benchmark backbone are host code over the CUDA
    library: they construct anywhere, keep the reference's parameter layout, and raise
    instead of computing on the CPU."""
    import torch

    from pointelligence_b200.backbone import ResUNet
    from pointelligence_b200.layers import (GlobalPool, RaggedBatchNorm, RaggedGroupNorm, RaggedInstanceNorm,
                                            RaggedLayerNorm)
    from pointelligence_b200.sparse_engines.ops import indexed_segment_reduce, large_segment_reduce

    ln = RaggedLayerNorm(24)
    assert ln.weight.shape == (24,) and ln.bias.shape == (24,) and ln.eps == 1e-5
    assert RaggedInstanceNorm(8).weight is None              # affine=False by default, as in the reference
    assert RaggedGroupNorm(4, 24).num_groups == 4
    with pytest.raises(ValueError):
        RaggedGroupNorm(5, 24)
    x, lengths = torch.randn(10, 24), torch.tensor([4, 6])
    with pytest.raises(ValueError):
        ln(x)                                                 # lengths are required
    for call in (lambda: ln(x, lengths), lambda: large_segment_reduce(x, "mean", lengths=lengths),
                 lambda: indexed_segment_reduce(x, "max", torch.tensor([0, 1, 2]), lengths=torch.tensor([1, 2])),
                 lambda: GlobalPool("max")(x, lengths)):
        with pytest.raises(RuntimeError, match="CUDA"):
            call()
    with pytest.raises(ValueError):
        large_segment_reduce(x, "median", lengths=lengths)
    assert RaggedBatchNorm(24)(x).shape == x.shape            # nn.BatchNorm1d, as in the reference
    net = ResUNet(in_channels=3, num_classes=20)
    assert sum(p.numel() for p in net.parameters()) == 22_834_100
    assert net.conv1.weight.shape == (125, 1, 3, 32) and net.final_conv.weight.shape == (1, 1, 96, 20)


def test_size_products_that_would_wrap_are_rejected_before_any_launch():
    """n_o * G * Ma * Cb is checked factor by factor: a product that wraps around 2^64 must not
    pass for a small one (the static-scratch entry would then write far past its built-in array).
    The check comes before any CUDA call, so it runs without a GPU; the pointers are never read."""
    import ctypes

    from pointelligence_b200 import _cabi

    L = _cabi.lib()
    fake = ctypes.c_void_p(4096)
    big = 1 << 21                                   # 4095 * 2^63 wraps to a multiple of 2^63 modulo 2^64
    rc = L.pcx_vvor_static_scratch(None, None, None, None, fake, fake, 0, 0, 0, 4095, big, big, big, _cabi.PCX_BF16, None)
    assert rc == -4 and b"exceeds the built-in scratch" in L.pcx_last_error_string()
    assert L.pcx_vvor_workspace_bytes(4095, big, big, big, _cabi.PCX_BF16) == 0
    assert L.pcx_mvmr_workspace_bytes(1 << 40, 27, big, big, big, 0, _cabi.PCX_BF16) == 0
    rc = L.pcx_vvor(None, None, None, None, fake, None, fake, 0, 0, 0, 4095, big, big, big, _cabi.PCX_BF16, 0, fake, 256,
                    None)
    assert rc == -4


def test_reference_style_imports_and_operator_namespace():
    """After ``compat.install()`` the reference's import lines resolve to this library and the
    three operators exist under ``sparse_engines::`` with the reference's schemas
    (sparse_engines/tig.py:1508-1515, mvmr_triton.py:145-152, vvor_triton.py:113-120).  Runs in
    a child interpreter: the aliases are process-wide."""
    code = r"""
import torch
import pointelligence_b200.compat as compat
compat.install(); compat.install()
from sparse_engines.ops import (sparse_matrix_vector_multiplication_reduction,
                                sparse_vector_vector_outer_product_reduction)
from sparse_engines.tig import TigIndex, tig_forward, tig_grad_input, tig_grad_weight, tig_mvmr
from sparse_engines._dispatch_override import current_mode, dispatch_mode, precision_mode
from layers import (MetaData, PointConv3d, TripletContract, build_triplets, build_triplets_segmented,
                    conv_with_stride, conv_with_stride_full_cover, radius_scaler_for_kernel_size, voxelize_3d)
from layers.downsample import downsample
from internals.neighbors import radius_search, radius_search_sorted_grid8, radius_search_sorted_grid8_segments
from internals.grid_sample import grid_sample_filter
from internals.two_phase import ForceFused, GeometryScheduler, TwoPhaseOp
from layers.two_phase_conv import ConvOp
from layers.generative import GeneratedSites, KernelStampGenerator, SubdivisionGenerator, build_generative_triplets
from layers.conv import GenerativePointConv3d, conv_with_stride_disjoint
from layers.triplets import handle_stride_disjoint_and_build_triplets
from layers.norm import RaggedGroupNorm, RaggedInstanceNorm, RaggedLayerNorm
import pointelligence_b200.layers as ours, layers
assert layers is ours and layers.PointConv3d is ours.PointConv3d
import sparse_engines.tig, pointelligence_b200.sparse_engines.tig as t
assert sparse_engines.tig is t
s = str(torch.ops.sparse_engines.tig_mvmr.default._schema)
assert s == ("sparse_engines::tig_mvmr(Tensor weight, Tensor feat, Tensor flat_i, Tensor flat_j, Tensor flat_seg, "
             "SymInt n_out, SymInt n_in, SymInt num_kernel_offsets, bool exact_cover_out, bool exact_cover_in, "
             "SymInt uniform_seg_len, str input_precision) -> Tensor"), s
for name in ("sparse_matrix_vector_multiplication_reduction", "sparse_vector_vector_outer_product_reduction"):
    s = str(getattr(torch.ops.sparse_engines, name).default._schema)
    assert s == (f"sparse_engines::{name}(Tensor a, Tensor a_idx, Tensor b, Tensor b_idx, Tensor o_idx, SymInt n_o, "
                 "Tensor? seg_offs=None) -> Tensor"), s
# shape-only fake kernels: traceable leaves
from torch._subclasses.fake_tensor import FakeTensorMode
with FakeTensorMode():
    w = torch.empty(27, 1, 16, 32); x = torch.empty(50, 16); idx = torch.empty(400, dtype=torch.int32)
    seg = torch.empty(28, dtype=torch.int64)
    y = torch.ops.sparse_engines.tig_mvmr(w, x, idx, idx, seg, 40, 50, 27, False, False, -1, "ieee")
    assert y.shape == (40, 32)
    o = torch.ops.sparse_engines.sparse_matrix_vector_multiplication_reduction(w, idx, x.view(50, 1, 16), idx, idx, 40)
    assert o.shape == (40, 1, 32)
print("ok")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-3000:]
