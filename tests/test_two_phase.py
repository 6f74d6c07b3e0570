"""Two-phase scheduler on the CPU with toy ops (what ``tests/unittest/test_two_phase_scheduler.py``
of the reference checks): hoisted builds give the interleaved result, geometry threads through the
builds, ``ForceFused`` changes only the order, a feature-dependent op cuts the sequence and its
geometry reaches the builds behind it; plus ``prepare`` (phase 1 once, phase 2 many times) and the
eager fall-backs of the CUDA-graph compiler."""
import pytest
import torch

from pointelligence_b200.internals.two_phase import (ForceFused, FusedOp, GeometryScheduler, Segment, TwoPhaseOp,
                                                     cuda_graph_compiler)


class Shift:
    """Separable: the bundle is the geometry counter at build time; apply adds it."""
    separable = True

    def __init__(self, log=None):
        self.seen = None
        self.log = log if log is not None else []

    def build_indices(self, geom):
        self.seen = geom
        self.log.append(("build", geom))

        class Bundle:
            pass

        b = Bundle()
        b.amount, b.next_geom = float(geom), geom + 1
        return b

    def apply(self, x, b):
        self.log.append(("apply", b.amount))
        return x + b.amount


class Reorder:
    """Not separable: its permutation depends on the features; it also moves the geometry."""
    separable = False

    def forward(self, x, geom):
        return x[torch.argsort(x.sum(dim=1))], geom + 100


def _interleaved(ops, x, geom):
    for op in ops:
        if op.separable:
            b = op.build_indices(geom)
            x, geom = op.apply(x, b), b.next_geom
        else:
            x, geom = op.forward(x, geom)
    return x


def test_protocols_and_hoisting_order():
    assert isinstance(Shift(), TwoPhaseOp) and isinstance(Reorder(), FusedOp)
    log = []
    x = torch.arange(6.0).reshape(3, 2)
    got = GeometryScheduler().run([Shift(log), Shift(log), Shift(log)], x.clone(), geom=0)
    assert torch.equal(got, _interleaved([Shift(), Shift(), Shift()], x.clone(), 0))
    assert torch.equal(got, x + 3.0)                                   # builds saw 0, 1, 2
    assert [kind for kind, _ in log] == ["build"] * 3 + ["apply"] * 3  # every build before any apply


def test_force_fused_is_the_interleaved_order_with_the_same_result():
    log = []
    x = torch.arange(6.0).reshape(3, 2)
    plain = GeometryScheduler().run([Shift(), Shift()], x.clone(), geom=0)
    forced = GeometryScheduler().run([ForceFused(Shift(log)), ForceFused(Shift(log))], x.clone(), geom=0)
    assert torch.equal(plain, forced)
    assert [kind for kind, _ in log] == ["build", "apply", "build", "apply"]


def test_feature_dependent_op_cuts_the_sequence():
    x = torch.tensor([[3.0, 0.0], [1.0, 0.0], [2.0, 0.0]])
    tail = Shift()
    compiled = []

    def counting(fn):
        compiled.append(fn)
        return fn

    out = GeometryScheduler().run([Shift(), Reorder(), tail], x.clone(), geom=0, compile_segments=True,
                                  compiler=counting)
    assert len(compiled) == 2 and tail.seen == 101           # 0 -> 1 (head) -> 101 (seam)
    assert torch.equal(out, _interleaved([Shift(), Reorder(), Shift()], x.clone(), 0))
    # a seam first and last, and an empty sequence
    assert torch.equal(GeometryScheduler().run([Reorder()], x.clone(), geom=0), x[torch.argsort(x.sum(dim=1))])
    assert torch.equal(GeometryScheduler().run([], x.clone(), geom=0), x)


def test_prepare_builds_once_and_applies_many_times():
    log = []
    body = GeometryScheduler().prepare([Shift(log), Shift(log)], geom=5)
    assert [kind for kind, _ in log] == ["build", "build"]
    for scale in (1.0, 2.0):
        x = torch.ones(2, 2) * scale
        assert torch.equal(body(x), x + 11.0)
    assert [kind for kind, _ in log].count("build") == 2
    with pytest.raises(ValueError):
        GeometryScheduler().prepare([Shift(), Reorder()], geom=0)
    seg = Segment([Shift()])
    assert seg.prepare(7) == 8 and torch.equal(seg.body(torch.zeros(1)), torch.full((1,), 7.0))


def test_graph_compiler_runs_eagerly_off_the_gpu():
    calls = []

    def fn(x):
        calls.append(x.shape)
        return x * 2

    run = cuda_graph_compiler(fn)
    x = torch.ones(3)
    assert torch.equal(run(x), x * 2) and torch.equal(run(x.requires_grad_()), x * 2)
    assert len(calls) == 2
