"""Geometry / feature two-phase execution (interface of ``internals/two_phase.py:24-97``).

An op that can prepare its indices from geometry alone (``separable = True``) exposes
``build_indices(geom) -> bundle`` and ``apply(x, bundle) -> x``; a bundle may carry ``next_geom``,
the geometry the following op sees.  An op whose indices depend on the features
(``separable = False``) exposes ``forward(x, geom) -> (x, geom)`` and cuts the op sequence.
``GeometryScheduler.run`` cuts the sequence at those ops into ``Segment`` objects; a segment first
prepares every bundle under one triplet-cache scope -- each build ends with its host hand-over, so
all of them happen before any feature kernel -- and then runs the ``apply`` chain, which contains
no hand-over.  ``ForceFused`` turns a separable op back into the interleaved order (the parity
reference of the hoisted one).

Where the reference hands the ``apply`` chain of a segment to ``torch.compile``, the default
"compiler" here is ``cuda_graph_compiler``: the chain is captured once into a CUDA graph and
replayed for later feature tensors of the same shape on the same bundles (inference only; under
autograd, on the CPU, or for a changed input shape the chain runs eagerly).
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional, Protocol, Sequence, Tuple, runtime_checkable

import torch

from .triplet_cache import triplet_cache_scope


@runtime_checkable
class TwoPhaseOp(Protocol):
    separable: bool

    def build_indices(self, geom: Any) -> Any: ...

    def apply(self, x: torch.Tensor, bundle: Any) -> torch.Tensor: ...


@runtime_checkable
class FusedOp(Protocol):
    separable: bool

    def forward(self, x: torch.Tensor, geom: Any) -> Tuple[torch.Tensor, Any]: ...


def _advance(geom, bundle):
    nxt = getattr(bundle, "next_geom", None)
    return geom if nxt is None else nxt


class ForceFused:
    """A separable op run at its own position: build, then apply, nothing hoisted."""

    separable = False

    def __init__(self, inner: TwoPhaseOp):
        self.inner = inner

    def forward(self, x, geom):
        bundle = self.inner.build_indices(geom)
        return self.inner.apply(x, bundle), _advance(geom, bundle)


class Segment:
    """A maximal run of separable ops: ``prepare`` builds every bundle, ``body`` applies them."""

    def __init__(self, ops: Sequence[TwoPhaseOp]):
        self.ops: List[TwoPhaseOp] = list(ops)
        self.bundles: List[Any] = []

    def prepare(self, geom):
        self.bundles = []
        with triplet_cache_scope():
            for op in self.ops:
                bundle = op.build_indices(geom)
                self.bundles.append(bundle)
                geom = _advance(geom, bundle)
        return geom

    def body(self, x):
        for op, bundle in zip(self.ops, self.bundles):
            x = op.apply(x, bundle)
        return x


def cuda_graph_compiler(fn: Callable[[torch.Tensor], torch.Tensor]) -> Callable[[torch.Tensor], torch.Tensor]:
    """Capture ``fn`` (a chain of kernels with no host hand-over) into a CUDA graph on first use.

    The returned callable copies its argument into the graph's static input, replays, and returns
    a clone of the static output.  It falls back to calling ``fn`` when autograd is recording, the
    input is not a CUDA tensor, or the input's shape or dtype differs from the captured one.
    """
    state = {}

    def run(x: torch.Tensor) -> torch.Tensor:
        if not (isinstance(x, torch.Tensor) and x.is_cuda) or (torch.is_grad_enabled() and x.requires_grad):
            return fn(x)
        if "graph" not in state:
            with torch.no_grad():
                static_in = x.clone()
                side = torch.cuda.Stream(device=x.device)
                side.wait_stream(torch.cuda.current_stream(x.device))
                with torch.cuda.stream(side):   # warm-up: lazy plans, workspaces and tensor maps exist before capture
                    fn(static_in)
                torch.cuda.current_stream(x.device).wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    static_out = fn(static_in)
            state.update(graph=graph, static_in=static_in, static_out=static_out)
        static_in = state["static_in"]
        if x.shape != static_in.shape or x.dtype != static_in.dtype:
            with torch.no_grad():
                return fn(x)
        static_in.copy_(x)
        state["graph"].replay()
        return state["static_out"].clone()

    return run


class GeometryScheduler:
    """Cuts ``ops`` at the non-separable ones and runs segment by segment."""

    def prepare(self, ops: Sequence[TwoPhaseOp], geom: Any, *, compile_segments: bool = False,
                compiler: Optional[Callable[[Callable], Callable]] = None) -> Callable[[torch.Tensor], torch.Tensor]:
        """Phase 1 once, phase 2 many times: builds the bundles of an all-separable sequence and
        returns the ``apply`` chain as a callable for any number of feature tensors on this
        geometry (with ``compile_segments`` one CUDA graph serves all of them)."""
        if not all(getattr(op, "separable", True) for op in ops):
            raise ValueError("prepare() needs separable ops only: a feature-dependent op has no feature-free build")
        seg = Segment(ops)
        seg.prepare(geom)
        return (compiler or cuda_graph_compiler)(seg.body) if compile_segments else seg.body

    def run(self, ops: Sequence[Any], x: torch.Tensor, geom: Any, *, compile_segments: bool = False,
            compiler: Optional[Callable[[Callable], Callable]] = None) -> torch.Tensor:
        compiler = compiler or cuda_graph_compiler

        def flush(pending, x, geom):
            if not pending:
                return x, geom
            seg = Segment(pending)
            geom = seg.prepare(geom)
            body = compiler(seg.body) if compile_segments else seg.body
            return body(x), geom

        pending: List[Any] = []
        for op in ops:
            if getattr(op, "separable", True):
                pending.append(op)
                continue
            x, geom = flush(pending, x, geom)
            pending = []
            x, geom = op.forward(x, geom)
        x, geom = flush(pending, x, geom)
        return x
