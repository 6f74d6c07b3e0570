"""CPU restatements of MVMR / VVOR (TEST INFRASTRUCTURE).

Three checkers of increasing fidelity to the reference's own CPU path:

``mvmr_f64`` / ``vvor_f64``
    fp64 ``einsum + add.at`` formulation, the shape used by the reference's
    unit tests (tests/unittest/test_tig_forward.py:27-38,
    tests/unittest/test_sparse_linalg.py:12-51).  Tolerance oracle.
``mvmr_c`` / ``vvor_c``
    the plain-C restatement of the reference's fp32 loops
    (extensions/sparse_engines_cuda/csrc/spare_mvmr.cpp:12-75,
    sparse_vvor.cpp:12-53) loaded from ``_ref/liboracle_sparse.so``.
``mvmr_ref`` / ``vvor_ref``
    the reference's operators themselves, compiled from its sources into
    ``_ref/libsparse_engines_ref_cpu.so`` (``torch.ops.sparse_engines_cuda``).

Semantics (sparse_engines/mvmr_triton.py:148-254, vvor_triton.py:116-223):

    MVMR  o[o_idx[t], g, :]    += b[b_idx[t], g, :] @ a[a_idx[t], g, :, :]
          a (K,G,C,M)  b (Nb,G,C)  ->  o (n_o,G,M)
    VVOR  o[o_idx[t], g, m, c] += a[a_idx[t], g, m] * b[b_idx[t], g, c]
          a (Na,G,M)   b (Nb,G,C)  ->  o (n_o,G,M,C)
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build_ref

_lib = None
_ref_loaded = False


def _c_lib():
    global _lib
    if _lib is None:
        path = build_ref.ORACLE_SO
        if not os.path.exists(path):
            build_ref.build_oracle_c()
        _lib = ctypes.CDLL(path)
        i32p = ctypes.POINTER(ctypes.c_int32)
        f32p = ctypes.POINTER(ctypes.c_float)
        for name in ("oracle_mvmr_f32", "oracle_vvor_f32"):
            fn = getattr(_lib, name)
            fn.restype = None
            fn.argtypes = [f32p, i32p, f32p, i32p, i32p, f32p, ctypes.c_int64,
                           ctypes.c_int, ctypes.c_int, ctypes.c_int]
    return _lib


def _f32(x):
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


def _i32(x):
    return np.ascontiguousarray(np.asarray(x, dtype=np.int32))


def _p(arr, ct):
    return arr.ctypes.data_as(ctypes.POINTER(ct))


def mvmr_f64(a, a_idx, b, b_idx, o_idx, n_o):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    K, G, C, M = a.shape
    o = np.zeros((n_o, G, M), np.float64)
    T = len(a_idx)
    step = 1 << 16
    for s in range(0, T, step):
        sl = slice(s, min(T, s + step))
        prod = np.einsum("tgc,tgcm->tgm", b[np.asarray(b_idx[sl])], a[np.asarray(a_idx[sl])])
        np.add.at(o, np.asarray(o_idx[sl]), prod)
    return o


def vvor_f64(a, a_idx, b, b_idx, o_idx, n_o):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    G, M, C = a.shape[1], a.shape[2], b.shape[2]
    o = np.zeros((n_o, G, M, C), np.float64)
    T = len(a_idx)
    step = 1 << 14
    for s in range(0, T, step):
        sl = slice(s, min(T, s + step))
        prod = np.einsum("tgm,tgc->tgmc", a[np.asarray(a_idx[sl])], b[np.asarray(b_idx[sl])])
        np.add.at(o, np.asarray(o_idx[sl]), prod)
    return o


def mvmr_f64_taps(a, seg_offs, b, b_idx, o_idx, n_o, rows=None):
    """MVMR in fp64 for TAP-SORTED triplets (``seg_offs`` = K+1 segment offsets), one group:
    per tap one dense product of the gathered rows with ``a[k]`` and a sparse-matrix sum into
    the output rows.  Same result as ``mvmr_f64`` (it is the same sum in another order) but
    affordable at benchmark sizes.  With ``rows`` (sorted unique output rows) only those rows
    are computed and returned, in that order.  a (K,1,C,M) or (K,C,M); b (Nb,C) -> (n_o, M).
    """
    import scipy.sparse as sp

    a = np.asarray(a, np.float64)
    a = a.reshape(a.shape[0], a.shape[-2], a.shape[-1])
    b = np.asarray(b, np.float64).reshape(len(b), -1)
    b_idx, o_idx, seg = np.asarray(b_idx), np.asarray(o_idx), np.asarray(seg_offs)
    if rows is not None:
        rows = np.asarray(rows)
        keep = np.isin(o_idx, rows)
        slot = np.searchsorted(rows, o_idx)
        n_res = len(rows)
    else:
        keep, slot, n_res = None, o_idx, n_o
    out = np.zeros((n_res, a.shape[2]), np.float64)
    for k in range(a.shape[0]):
        lo, hi = int(seg[k]), int(seg[k + 1])
        if hi <= lo:
            continue
        sel = np.arange(lo, hi) if keep is None else lo + np.flatnonzero(keep[lo:hi])
        if len(sel) == 0:
            continue
        prod = b[b_idx[sel]] @ a[k]
        scatter = sp.csr_matrix((np.ones(len(sel)), (slot[sel], np.arange(len(sel)))), shape=(n_res, len(sel)))
        out += scatter @ prod
    return out


def vvor_f64_taps(a, a_idx, b, b_idx, seg_offs, taps=None):
    """VVOR in fp64 for TAP-SORTED triplets, one group: ``out[k] = a[a_idx[seg k]]^T @ b[b_idx[seg k]]``.
    With ``taps`` only those taps are computed (result (len(taps), Ma, Cb))."""
    a = np.asarray(a, np.float64).reshape(len(a), -1)
    b = np.asarray(b, np.float64).reshape(len(b), -1)
    a_idx, b_idx, seg = np.asarray(a_idx), np.asarray(b_idx), np.asarray(seg_offs)
    taps = range(len(seg) - 1) if taps is None else taps
    out = np.zeros((len(taps), a.shape[1], b.shape[1]), np.float64)
    for n, k in enumerate(taps):
        lo, hi = int(seg[k]), int(seg[k + 1])
        if hi > lo:
            out[n] = a[a_idx[lo:hi]].T @ b[b_idx[lo:hi]]
    return out


def mvmr_c(a, a_idx, b, b_idx, o_idx, n_o):
    a, b = _f32(a), _f32(b)
    ai, bi, oi = _i32(a_idx), _i32(b_idx), _i32(o_idx)
    K, G, C, M = a.shape
    o = np.zeros((n_o, G, M), np.float32)
    _c_lib().oracle_mvmr_f32(_p(a, ctypes.c_float), _p(ai, ctypes.c_int32),
                             _p(b, ctypes.c_float), _p(bi, ctypes.c_int32),
                             _p(oi, ctypes.c_int32), _p(o, ctypes.c_float),
                             len(ai), G, C, M)
    return o


def vvor_c(a, a_idx, b, b_idx, o_idx, n_o):
    a, b = _f32(a), _f32(b)
    ai, bi, oi = _i32(a_idx), _i32(b_idx), _i32(o_idx)
    G, M, C = a.shape[1], a.shape[2], b.shape[2]
    o = np.zeros((n_o, G, M, C), np.float32)
    _c_lib().oracle_vvor_f32(_p(a, ctypes.c_float), _p(ai, ctypes.c_int32),
                             _p(b, ctypes.c_float), _p(bi, ctypes.c_int32),
                             _p(oi, ctypes.c_int32), _p(o, ctypes.c_float),
                             len(ai), G, M, C)
    return o


def reference_ops_available():
    return os.path.exists(build_ref.REF_SO) or build_ref.build_reference_cpu_ops() is not None


def _ref_ops():
    global _ref_loaded
    import torch

    if not _ref_loaded:
        path = build_ref.build_reference_cpu_ops()
        if path is None:
            raise RuntimeError("reference CPU operators are not built and the "
                               "reference sources are not available")
        torch.ops.load_library(path)
        _ref_loaded = True
    return torch.ops.sparse_engines_cuda


def mvmr_ref(a, a_idx, b, b_idx, o_idx, n_o):
    """The reference's own CPU MVMR (fp32 tensors, int32 indices)."""
    import torch

    t = lambda x, d: torch.as_tensor(np.asarray(x)).to(d).contiguous()
    out = _ref_ops().sparse_matrix_vector_multiplication_reduction(
        t(a, torch.float32), t(a_idx, torch.int32), t(b, torch.float32),
        t(b_idx, torch.int32), t(o_idx, torch.int32), int(n_o))
    return out.numpy()


def vvor_ref(a, a_idx, b, b_idx, o_idx, n_o):
    """The reference's own CPU VVOR (fp32 tensors, int32 indices)."""
    import torch

    t = lambda x, d: torch.as_tensor(np.asarray(x)).to(d).contiguous()
    out = _ref_ops().sparse_vector_vector_outer_product_reduction(
        t(a, torch.float32), t(a_idx, torch.int32), t(b, torch.float32),
        t(b_idx, torch.int32), t(o_idx, torch.int32), int(n_o))
    return out.numpy()


def rel_frobenius(x, ref):
    """tests/unittest/test_tig_forward.py:41-43."""
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.linalg.norm(x - ref) / max(np.linalg.norm(ref), 1e-30))
