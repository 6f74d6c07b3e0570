"""TEST INFRASTRUCTURE ONLY -- CPU restatement (numpy, float64) of the reference's
segment reductions; never imported by the product path.

``large_segment_reduce``     follows sparse_engines/large_segment_reduce_triton.py:25-77,
                             :180-188 and its kernel (large_segment_reduce_triton_kernel.py:4-140)
``large_segment_reduce_grad``  :94-166 and the two backward kernels (:141-230 of the kernel file)
``indexed_segment_reduce``   follows sparse_engines/indexed_segment_reduce_triton.py:25-63,
                             :147-173 and its kernel (indexed_segment_reduce_triton_kernel.py:18-84)
``indexed_segment_reduce_grad``  the backward kernel (:89-170 of the kernel file)
``ragged_norm``              follows layers/norm.py:59-130

Pinned by tests/golden/segment.npz, produced by running the reference's Triton
kernels under Triton's CPU interpreter (tests/golden/make_golden.py).
"""
import numpy as np

_NEUTRAL = {"sum": 0.0, "mean": 0.0, "max": -np.inf, "min": np.inf}


def _fold(rows, reduce):
    if reduce in ("sum", "mean"):
        return rows.sum(axis=0)
    return rows.max(axis=0) if reduce == "max" else rows.min(axis=0)


def large_segment_reduce(x, lengths, reduce):
    x = np.asarray(x, np.float64)
    lengths = np.asarray(lengths, np.int64)
    offs = np.concatenate([[0], np.cumsum(lengths)])
    out = np.full((len(lengths), x.shape[1]), _NEUTRAL[reduce])
    for s, n in enumerate(lengths):
        if n > 0:
            out[s] = _fold(x[offs[s]:offs[s + 1]], reduce)
        if reduce == "mean":
            out[s] = out[s] / max(int(n), 1)
    return out


def large_segment_reduce_grad(grad_out, x, out, lengths, reduce):
    grad_out = np.asarray(grad_out, np.float64)
    lengths = np.asarray(lengths, np.int64)
    seg = np.repeat(np.arange(len(lengths)), lengths)
    g = grad_out[seg]
    if reduce == "mean":
        g = g / np.maximum(lengths, 1)[seg, None]
    if reduce in ("max", "min"):
        g = np.where(np.asarray(x) == np.asarray(out)[seg], g, 0.0)
    return g


def indexed_segment_reduce(x, indices, lengths, reduce):
    x = np.asarray(x, np.float64)
    lengths = np.asarray(lengths, np.int64)
    offs = np.concatenate([[0], np.cumsum(lengths)])
    out = np.full((len(lengths), x.shape[1]), _NEUTRAL[reduce])
    for k, n in enumerate(lengths):
        if n > 0:
            out[k] = _fold(x[indices[offs[k]:offs[k + 1]]], reduce)
        if reduce == "mean":
            with np.errstate(invalid="ignore", divide="ignore"):
                out[k] = out[k] / np.float64(n)
    return out


def indexed_segment_reduce_grad(grad_y, x, y, indices, lengths, reduce, n_x):
    grad_y = np.asarray(grad_y, np.float64)
    lengths = np.asarray(lengths, np.int64)
    seg = np.repeat(np.arange(len(lengths)), lengths)
    g = grad_y[seg]
    if reduce == "mean":
        g = g / lengths[seg, None]
    if reduce in ("max", "min"):
        g = np.where(np.asarray(x)[indices] == np.asarray(y)[seg], g, 0.0)
    out = np.zeros((n_x, grad_y.shape[1]))
    np.add.at(out, indices, g)
    return out


def ragged_norm(x, lengths, norm_type, num_groups=1, eps=1e-5, weight=None, bias=None):
    x = np.asarray(x, np.float64)
    lengths = np.asarray(lengths, np.int64)
    seg = np.repeat(np.arange(len(lengths)), lengths)

    def seg_mean(v):
        return large_segment_reduce(v, lengths, "mean")[seg]

    if norm_type == "instance":
        c = x - seg_mean(x)
        out = c / np.sqrt(seg_mean(c ** 2) + eps)
    elif norm_type == "layer":
        c = x - seg_mean(x.mean(axis=1, keepdims=True))
        out = c / np.sqrt(seg_mean((c ** 2).mean(axis=1, keepdims=True)) + eps)
    elif norm_type == "group":
        xg = x.reshape(len(x), num_groups, -1)
        c = xg - seg_mean(xg.mean(axis=2))[:, :, None]
        out = (c / np.sqrt(seg_mean((c ** 2).mean(axis=2)) + eps)[:, :, None]).reshape(x.shape)
    else:
        raise ValueError(norm_type)
    if weight is not None:
        out = out * np.asarray(weight, np.float64) + np.asarray(bias, np.float64)
    return out
