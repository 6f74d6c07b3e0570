"""Forward-scoped triplet cache (mirror of ``internals/triplet_cache.py:34-110``).

Triplets are a pure function of the point sets, the radius, the kernel and the
sort order, and the same combination recurs inside one forward pass (U-Net
encoder/decoder, residual blocks).  ``with triplet_cache_scope():`` installs a
per-thread dictionary that the triplet builders consult; outside a scope
nothing is cached.  ``POINTELLIGENCE_DISABLE_TRIPLET_CACHE=1`` turns it off.
"""
from __future__ import annotations

import functools
import os
import threading
import weakref
from contextlib import contextmanager

_local = threading.local()
_DISABLED = os.environ.get("POINTELLIGENCE_DISABLE_TRIPLET_CACHE", "0") == "1"


def _active_cache():
    return getattr(_local, "cache", None)


@contextmanager
def triplet_cache_scope():
    """Re-entrant: a nested scope shares the enclosing scope's dictionary."""
    if _DISABLED:
        yield None
        return
    outer = _active_cache()
    if outer is not None:
        yield outer
        return
    _local.cache = {}
    try:
        yield _local.cache
    finally:
        _local.cache = None


def _indexer_identity(kernel_indexer):
    """Hashable identity of a ``functools.partial`` tap indexer, else None (not cacheable)."""
    if not isinstance(kernel_indexer, functools.partial):
        return None
    try:
        ident = (getattr(kernel_indexer.func, "__qualname__", repr(kernel_indexer.func)),
                 tuple(kernel_indexer.args), tuple(sorted(kernel_indexer.keywords.items())))
        hash(ident)
    except TypeError:
        return None
    return ident


def triplet_key(points, query_points, neighbor_radius, radius_scaler, sort_by, return_num_neighbors,
                sample_inds, query_sample_inds, kernel_indexer):
    """Everything the builders' output depends on, by tensor identity; None = do not cache."""
    ident = _indexer_identity(kernel_indexer)
    if ident is None:
        return None
    self_query = query_points is points
    return (points.data_ptr(), int(points.shape[0]), sample_inds.data_ptr(),
            "self" if self_query else query_points.data_ptr(),
            "self" if self_query else query_sample_inds.data_ptr(),
            round(float(neighbor_radius), 9),
            None if radius_scaler is None else round(float(radius_scaler), 9),
            sort_by, bool(return_num_neighbors), ident)


def cache_get(key):
    cache = _active_cache()
    if cache is None or key is None:
        return None
    hit = cache.get(key)
    if hit is None:
        return None
    value, alive = hit
    return value if alive() is not None else None   # a dead owner means the address may have been recycled


def cache_put(key, value, owner):
    cache = _active_cache()
    if cache is not None and key is not None:
        cache[key] = (value, weakref.ref(owner))
