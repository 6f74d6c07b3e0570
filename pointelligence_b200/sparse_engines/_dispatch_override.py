"""Global engine selection and fp32 precision knobs.

Mirror of the reference's ``sparse_engines/_dispatch_override.py:100-243``:
same function names, same accepted mode strings, same "not thread-safe
module-global" semantics.  The reference multiplexes ~10 kernel tiers; here
there is one backend with two engines, so the modes collapse:

* ``"force_pt"``                 -> CUDA-core engine (IEEE fp32 FMA, any shape)
* every other accepted mode      -> automatic choice (tcgen05 tensor engine
                                    when dtype/shape allow, else CUDA cores)

fp32 operands are always multiplied in IEEE fp32 (the reference's ``"ieee"``
default); ``precision_mode("tf32")`` is accepted and keeps IEEE arithmetic.
"""
from __future__ import annotations

import os
import warnings
from contextlib import contextmanager

_MODES = (
    "auto", "force_fsg", "force_pt",
    "force_fsg_wmma_vvor", "force_fsg_wmma_coop_vvor", "force_fsg_wmma_mvmr",
    "force_fsg_cutlass_vvor", "force_fsg_cutlass_mvmr",
    "force_fsg_cutlass_mvmr_vvor", "force_fsg_fused",
    "force_tig", "force_fused_gather_sum", "force_fgs",
)
_RENAMED = {
    "force_grouped": "force_fsg",
    "force_per_triplet": "force_pt",
    "force_grouped_wmma_vvor": "force_fsg_wmma_vvor",
    "force_grouped_cutlass_vvor": "force_fsg_cutlass_vvor",
    "force_grouped_cutlass_mvmr": "force_fsg_cutlass_mvmr",
    "force_grouped_cutlass_mvmr_vvor": "force_fsg_cutlass_mvmr_vvor",
    "force_fused_conv": "force_fsg_fused",
    "force_smig": "force_tig",
}


def _normalize(mode):
    return "force_fused_gather_sum" if mode == "force_fgs" else mode


_state = {"mode": _normalize(os.environ.get("PNT_DISPATCH_MODE", "auto")), "precision": "default"}


def current_mode():
    return _state["mode"]


def current_engine():
    """C-ABI engine code for the current mode (0 automatic, 1 CUDA cores)."""
    return 1 if _state["mode"] == "force_pt" else 0


def current_precision():
    p = _state["precision"]
    if p in ("ieee", "tf32"):
        return p
    import torch

    return "tf32" if torch.backends.cuda.matmul.allow_tf32 else "ieee"


def resolve_input_precision(dtype):
    import torch

    return "tf32" if dtype != torch.float32 else current_precision()


@contextmanager
def dispatch_mode(mode):
    if mode not in _MODES:
        if mode in _RENAMED:
            raise ValueError(f"dispatch mode {mode!r} was renamed to {_RENAMED[mode]!r}")
        raise ValueError(f"unknown dispatch mode: {mode!r}")
    prev = _state["mode"]
    _state["mode"] = _normalize(mode)
    try:
        yield
    finally:
        _state["mode"] = prev


@contextmanager
def precision_mode(mode):
    if mode not in ("default", "ieee", "tf32"):
        raise ValueError(f"unknown precision mode: {mode!r}")
    prev = _state["precision"]
    _state["precision"] = mode
    try:
        yield
    finally:
        _state["precision"] = prev


_SEEN = set()


def warn_pt_fallback(site, reason, **ctx):
    """One warning per (site, shape) when ``auto`` lands on the per-triplet
    CUDA-core kernel (unsorted triplets)."""
    key = (site, tuple(sorted(ctx.items())))
    if key in _SEEN:
        return
    _SEEN.add(key)
    detail = ", ".join(f"{k}={v}" for k, v in sorted(ctx.items()))
    warnings.warn(f"[{site}] 'auto' routed to the per-triplet fallback engine ({reason}; {detail}). "
                  "Correct but slow: tap-sorted triplets engage the tiled engines.",
                  RuntimeWarning, stacklevel=3)
