"""Tap-segment bookkeeping (mirror of ``sparse_engines/_seg_offs.py:21-185``)."""
from __future__ import annotations

import weakref

import torch

from .. import _cabi

_SORTED = {}
_COVER = {}
_SEG = {}
_MAX = 256


def kernel_offset_segments(idx_sorted, num_kernel_offsets):
    """``seg[k]`` = first position whose value is >= k; (K+1,) int64, no host sync."""
    return _cabi.seg_offs_from_sorted(idx_sorted, int(num_kernel_offsets))


def kernel_offset_segments_cached(idx_sorted, num_kernel_offsets):
    try:
        ver = idx_sorted._version
    except RuntimeError:
        return kernel_offset_segments(idx_sorted, num_kernel_offsets)
    key = (idx_sorted.data_ptr(), ver, idx_sorted.numel(), int(num_kernel_offsets))
    hit = _SEG.get(key)
    if hit is not None:
        src, seg = hit
        alive = src()
        if alive is not None and alive._version == ver and alive.data_ptr() == key[0]:
            return seg
        del _SEG[key]
    seg = kernel_offset_segments(idx_sorted, num_kernel_offsets)
    if len(_SEG) >= 64:
        _SEG.pop(next(iter(_SEG)))
    _SEG[key] = (weakref.ref(idx_sorted), seg)
    return seg


def _memo(cache, key, idx, compute):
    """Verdict memo keyed by (address, version, ...) and guarded by a weak
    reference to the tensor, so a new tensor at a recycled address re-checks."""
    hit = cache.get(key)
    if hit is not None:
        ref, verdict = hit
        if ref() is idx:
            return verdict
        del cache[key]
    verdict = compute()
    if len(cache) >= _MAX:
        cache.pop(next(iter(cache)))
    cache[key] = (weakref.ref(idx), verdict)
    return verdict


def is_sorted_cached(idx):
    """Memoised non-decreasing check (one device reduction + host sync per new tensor)."""
    key = (idx.data_ptr(), idx._version, idx.numel())
    return _memo(_SORTED, key, idx,
                 lambda: bool((idx[1:] >= idx[:-1]).all().item()) if idx.numel() > 1 else True)


def exact_cover_cached(idx, n):
    """True iff ``idx`` is a permutation of ``[0, n)``."""
    if idx.numel() != n:
        return False
    key = (idx.data_ptr(), idx._version, n)
    return _memo(_COVER, key, idx,
                 lambda: bool((torch.bincount(idx.long(), minlength=n).max() <= 1).item()) if n else True)
