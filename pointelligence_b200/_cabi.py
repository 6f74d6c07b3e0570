"""ctypes binding of ``libpointelligence_b200.so`` (see
``include/pointelligence_b200.h``) and the marshalling helpers used by the
host-side mirrors of the reference modules.

The library is mandatory: if it cannot be loaded every operator raises
``RuntimeError`` -- there is no CPU or PyTorch fallback.  Tensors are passed as
raw device pointers; outputs and workspaces are allocated here with PyTorch so
the caching allocator and the caller's current stream stay in charge.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_double, c_int, c_int64, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libpointelligence_b200.so")

PCX_F32, PCX_F16, PCX_BF16 = 0, 1, 2
ENGINE_AUTO, ENGINE_CUDA_CORE, ENGINE_TENSOR = 0, 1, 2
ENGINE_FLAG_FAN_IN_ONE = 0x100   # OR-ed into an engine: every output row occurs in exactly one triplet
PCX_E_CAPACITY = -4

_DTYPES = {torch.float32: PCX_F32, torch.float16: PCX_F16, torch.bfloat16: PCX_BF16}

_STATUS_EXC = {
    -1: ValueError,          # PCX_E_ARG
    -2: TypeError,           # PCX_E_DTYPE
    -3: ValueError,          # PCX_E_ALIGN
    -4: RuntimeError,        # PCX_E_CAPACITY
    -5: RuntimeError,        # PCX_E_LAUNCH
    -6: NotImplementedError, # PCX_E_UNSUPPORTED
    -7: RuntimeError,        # PCX_E_DEVICE
}

# name -> (restype, argtypes); every symbol declared in the header
SIGNATURES = {
    "pcx_version": (c_int, []),
    "pcx_last_error_string": (ctypes.c_char_p, []),
    "pcx_device_status": (c_int, [c_void_p, c_int, c_void_p]),
    "pcx_launch_count": (ctypes.c_longlong, [c_int]),
    "pcx_profile_enable": (c_int, [c_int]),
    "pcx_profile_count": (c_int, []),
    "pcx_profile_get": (c_int, [c_int, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_float)]),
    "pcx_mvmr_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int, c_int, c_int]),
    "pcx_mvmr": (c_int, [c_void_p] * 7 + [c_int64] * 3 + [c_int] * 7 + [c_void_p, c_size_t, c_void_p]),
    "pcx_mvmr_plan_group_blocks": (c_int, [c_int]),
    "pcx_mvmr_plan_bytes": (c_size_t, [c_int64, c_int64, c_int, c_int]),
    "pcx_mvmr_plan_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int, c_int]),
    "pcx_mvmr_plan_build": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_int64, c_int, c_void_p, c_size_t, c_void_p,
                                    c_size_t, c_void_p]),
    "pcx_mvmr_plan_multi_buckets": (c_int, [c_void_p, ctypes.POINTER(c_int64), c_void_p]),
    "pcx_mvmr_planned_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "pcx_mvmr_planned": (c_int, [c_void_p] * 3 + [c_size_t, c_void_p] + [c_int64] * 3 + [c_int] * 6
                         + [c_int64, c_void_p, c_size_t, c_void_p]),
    "pcx_debug_wait_runs_out": (c_int, [ctypes.c_ulonglong, c_void_p]),
    "pcx_vvor_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int]),
    "pcx_vvor": (c_int, [c_void_p] * 7 + [c_int64] * 4 + [c_int] * 5 + [c_void_p, c_size_t, c_void_p]),
    "pcx_vvor_static_scratch_max_elements": (c_size_t, []),
    "pcx_vvor_static_scratch": (c_int, [c_void_p] * 6 + [c_int64] * 4 + [c_int] * 4 + [c_void_p]),
    "pcx_segment_reduce_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "pcx_segment_reduce": (c_int, [c_void_p] * 3 + [c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_size_t,
                                                   c_void_p]),
    "pcx_segment_reduce_backward": (c_int, [c_void_p] * 5 + [c_int64, c_int64, c_int, c_int, c_int, c_void_p,
                                                            c_size_t, c_void_p]),
    "pcx_indexed_segment_reduce_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int, c_int, c_int]),
    "pcx_indexed_segment_reduce": (c_int, [c_void_p] * 4 + [c_int64] * 3 + [c_int] * 3 + [c_void_p, c_size_t,
                                                                                         c_void_p]),
    "pcx_indexed_segment_reduce_backward": (c_int, [c_void_p] * 6 + [c_int64] * 3 + [c_int] * 3
                                            + [c_void_p, c_size_t, c_void_p]),
    "pcx_ragged_layer_norm_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "pcx_ragged_layer_norm": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int, c_double, c_int, c_int, c_void_p,
                                                      c_size_t, c_void_p]),
    "pcx_ragged_layer_norm_backward": (c_int, [c_void_p] * 11 + [c_int64, c_int64, c_int, c_int, c_int, c_void_p,
                                                                c_size_t, c_void_p]),
    "pcx_ragged_group_norm_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "pcx_ragged_group_norm": (c_int, [c_void_p] * 7 + [c_int64, c_int64, c_int, c_int, c_double, c_int, c_void_p,
                                                      c_size_t, c_void_p]),
    "pcx_ragged_group_norm_backward": (c_int, [c_void_p] * 9 + [c_int64, c_int64, c_int, c_int, c_int, c_void_p,
                                                               c_size_t, c_void_p]),
    "pcx_rnet_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "pcx_rnet_far": (c_int, [c_void_p] * 3 + [c_int64, c_void_p, c_void_p]),
    "pcx_rnet_rounds": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_void_p, c_void_p, ctypes.POINTER(ctypes.c_int32),
                                c_void_p, c_size_t, c_void_p]),
    "pcx_seg_offs": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "pcx_expand_taps": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "pcx_set_radius_predicate": (c_int, [c_int]),
    "pcx_get_radius_predicate": (c_int, []),
    "pcx_radius_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "pcx_radius_fill_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "pcx_radius_count": (c_int, [c_void_p] * 4 + [c_int64, c_int64, c_double, c_int, c_int, c_double]
                         + [c_void_p] * 3 + [c_void_p, c_size_t, c_void_p]),
    "pcx_radius_fill": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_double, c_int, c_int, c_double,
                                c_int64] + [c_void_p] * 5 + [c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "pcx_radius_taps_supported": (c_int, [c_int]),
    "pcx_radius_taps_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "pcx_radius_taps_count": (c_int, [c_void_p] * 4 + [c_int64, c_int64, c_double, c_int, c_int, c_double]
                              + [c_void_p] * 2 + [c_void_p, c_size_t, c_void_p]),
    "pcx_radius_taps_total": (c_int, [c_int64, c_int64, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "pcx_radius_taps_fill": (c_int, [c_void_p] * 3 + [c_int64, c_int64, c_double, c_int, c_int, c_double, c_int64]
                             + [c_void_p] * 4 + [c_void_p, c_size_t, c_void_p]),
    "pcx_grid_sample_workspace_bytes": (c_size_t, [c_int64]),
    "pcx_grid_sample_count": (c_int, [c_void_p, c_void_p, c_int64, c_double, c_void_p, c_void_p, c_size_t,
                                      c_void_p]),
    "pcx_grid_sample_select": (c_int, [c_void_p, c_void_p, c_int64, c_double, c_int64] + [c_void_p] * 4
                               + [c_void_p, c_size_t, c_void_p]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m pointelligence_b200.build` "
                "(the operators have no fallback implementation)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    if rc == 0:
        return
    msg = lib().pcx_last_error_string().decode("utf-8", "replace")
    raise _STATUS_EXC.get(rc, RuntimeError)(f"{msg} [pcx status {rc}]")


def dtype_code(dtype):
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"unsupported feature dtype {dtype}; expected float32, float16 or bfloat16")


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "pointelligence_b200 operators run on CUDA tensors only (no CPU fallback); "
                f"got a tensor on {t.device}")


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


# ---------------------------------------------------- geometry beside the features ----
_SIDE_STREAMS = {}
_overlap = threading.local()


def _side_stream(device):
    """The high-priority stream geometry runs on inside a ``geometry_overlap`` scope, else None."""
    active = getattr(_overlap, "devices", None)
    index = device.index if device.index is not None else torch.cuda.current_device()
    if not active or index not in active:
        return None
    return _SIDE_STREAMS[index]


class geometry_overlap:
    """Scope in which the index-building calls of this module (radius search, grid sampling, plan
    building) run on a stream of their own, so that their host hand-overs wait for the geometry
    kernels only and the feature kernels already queued on the caller's stream keep the GPU busy
    meanwhile.  Results are handed to the caller's stream with an event, never with a host wait.

    Contract: inside the scope, every tensor handed to those calls was either complete before the
    scope was entered or is itself the result of one of them (point clouds, sample ids, index
    arrays) -- true for a network that derives its geometry from the input cloud alone.  The side
    stream waits for the caller's stream once, on entry; the caller's stream waits for the side
    stream on exit.  Not re-entrant across devices; nested use on one device is a no-op."""

    def __init__(self, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.owner = False

    def __enter__(self):
        if self.device.type != "cuda" or os.environ.get("PCX_GEOMETRY_OVERLAP", "1") == "0":
            return self
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        active = getattr(_overlap, "devices", None)
        if active is None:
            active = _overlap.devices = set()
        if index in active:
            return self
        if index not in _SIDE_STREAMS:
            _SIDE_STREAMS[index] = torch.cuda.Stream(device=index, priority=-1)
        _SIDE_STREAMS[index].wait_stream(torch.cuda.current_stream(index))
        active.add(index)
        self.owner, self.index = True, index
        return self

    def __exit__(self, *exc):
        if self.owner:
            _overlap.devices.discard(self.index)
            torch.cuda.current_stream(self.index).wait_stream(_SIDE_STREAMS[self.index])
            self.owner = False
        return False


def on_geometry_stream(fn):
    """Decorator of an index-building function (no feature arithmetic inside): when its device is
    inside a ``geometry_overlap`` scope the whole body runs on the side stream, and every tensor it
    returns -- also inside tuples and geometry records such as ``MetaData`` and its parents -- is
    made known to the caller's stream (event wait, allocator bookkeeping)."""
    import functools

    def device_of(values):
        for v in values:
            if isinstance(v, torch.Tensor):
                if v.is_cuda:
                    return v.device
            elif hasattr(v, "points") and isinstance(getattr(v, "points"), torch.Tensor) and v.points.is_cuda:
                return v.points.device
        return None

    def hand_over(value, main, depth=0):
        if isinstance(value, torch.Tensor):
            if value.is_cuda:
                value.record_stream(main)
        elif isinstance(value, (tuple, list)):
            for v in value:
                hand_over(v, main, depth)
        elif isinstance(value, MvmrPlan):
            value.buffer.record_stream(main)
        elif hasattr(value, "__dataclass_fields__") and depth < 8:
            for v in vars(value).values():
                if isinstance(v, (torch.Tensor, tuple, list)) or hasattr(v, "__dataclass_fields__"):
                    hand_over(v, main, depth + 1)

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        dev = device_of(list(args) + list(kwargs.values()))
        side = _side_stream(dev) if dev is not None else None
        if side is None:
            return fn(*args, **kwargs)
        main = torch.cuda.current_stream(dev)
        if main == side:
            return fn(*args, **kwargs)
        with torch.cuda.stream(side):
            out = fn(*args, **kwargs)
        main.wait_stream(side)
        hand_over(out, main)
        return out

    return wrapper


def as_i32(t):
    if t is None:
        return None
    return t.contiguous() if t.dtype == torch.int32 else t.to(torch.int32).contiguous()


def device_status(clear=True):
    """Status word set by kernels whose bounded waits ran out (0 = healthy)."""
    out = ctypes.c_uint(0)
    check(lib().pcx_device_status(ctypes.byref(out), 1 if clear else 0, stream_ptr()))
    return int(out.value)


def raise_if_device_reported():
    """Raise ``RuntimeError`` (PCX_E_DEVICE) if a kernel of the library gave up on one of its bounded
    waits since the last check; its result is incomplete.  Called where the host synchronises
    anyway (the geometry hand-overs), so that such a result cannot go unnoticed for long."""
    status = device_status(clear=True)
    if status:
        raise RuntimeError(f"a kernel of the library gave up on a bounded wait (device status word {status:#x}): "
                           "results computed since the last check are incomplete [pcx status -7]")


def launch_count(reset=False):
    """Kernels launched by the library so far (optionally resetting the counter)."""
    return int(lib().pcx_launch_count(1 if reset else 0))


def profile_enable(on=True):
    check(lib().pcx_profile_enable(1 if on else 0))


def profile_records():
    """[(kernel label, milliseconds)] recorded since ``profile_enable(True)``."""
    L = lib()
    out = []
    for i in range(L.pcx_profile_count()):
        name, ms = ctypes.c_char_p(), ctypes.c_float()
        check(L.pcx_profile_get(i, ctypes.byref(name), ctypes.byref(ms)))
        out.append((name.value.decode(), float(ms.value)))
    return out


# ---------------------------------------------------------------- sparse ----
# Engine choice of ``mvmr`` with the automatic engine.  The output-stationary kernel
# (``pcx_mvmr_planned``: accumulators in tensor memory across all taps, every output row written
# once) needs a plan of the rulebook, built once per rulebook and direction and remembered by the
# identity of the index tensors.  Measured on B200 it beats the scatter kernel of ``pcx_mvmr``
#   - for dense neighbourhoods (a dozen triplets per output row and more: the deeper levels of a
#     U-Net, dense scans), at every width, and
#   - from four triplets per row on once the scatter kernel's fp32 accumulator (n_out x width x 4
#     bytes) outgrows half of the 126 MB L2 and its reductions start to go to HBM: wide layers and
#     large clouds (on the residual U-Net of the benchmark: 282 ms per step on the scatter kernel
#     alone, 203 ms with this rule).
# Sparse rulebooks over small accumulators and single-tap rulebooks (nothing to keep across taps)
# stay on the scatter kernel.  So do rulebooks that are thin in tap space (fewer than 0.18 triplets
# per output row and tap): their 128-row tiles are mostly padding.  The 125-tap stem of the benchmark
# (16.5 triplets per row, 0.13 per row and tap, 16 input channels) takes 1.03 ms on the scatter kernel
# against 2.56 ms plus its plan; the 27-tap layers of the finest level (0.23) stay planned.
ENGINE_PLANNED = 3
_PLANNED_DENSE_RATIO = float(os.environ.get("PCX_PLANNED_DENSE_RATIO", "12"))   # triplets per output row: always planned
_PLANNED_MIN_RATIO = float(os.environ.get("PCX_PLANNED_MIN_RATIO", "4"))        # ... planned when the accumulator is large
_PLANNED_MIN_ACC_BYTES = int(os.environ.get("PCX_PLANNED_MIN_ACC_BYTES", str(64 << 20)))
_PLANNED_MIN_TAP_FILL = float(os.environ.get("PCX_PLANNED_MIN_TAP_FILL", "0.18"))  # triplets per output row and tap
_PLANNED_ENABLED = os.environ.get("PCX_PLANNED", "1") != "0"


def _planned_pays(T, n_out, outw, K):
    if not _PLANNED_ENABLED or K <= 1 or n_out <= 0:
        return False
    ratio = T / n_out
    if ratio / K < _PLANNED_MIN_TAP_FILL:
        return False
    return ratio >= _PLANNED_DENSE_RATIO or (ratio >= _PLANNED_MIN_RATIO and n_out * outw * 4 >= _PLANNED_MIN_ACC_BYTES)


class MvmrPlan:
    """A rulebook regrouped for the output-stationary MVMR kernel (``pcx_mvmr_plan_build``).

    Holds the device buffer and the sizes it was built for.  A plan belongs to one rulebook,
    one direction (which index is scattered) and one ``group_blocks`` value.
    """

    __slots__ = ("buffer", "T", "K", "n_out", "group_blocks", "multi_buckets", "__weakref__")

    def __init__(self, buffer, T, K, n_out, group_blocks, multi_buckets):
        self.buffer, self.T, self.K, self.n_out, self.group_blocks = buffer, T, K, n_out, group_blocks
        self.multi_buckets = multi_buckets   # (row, tap) buckets with several triplets

    def views(self):
        """The plan's arrays as tensors (for tests): perm, tile_offs, entries (T, 2), group_order."""
        nblocks = (self.n_out + 127) // 128
        ngroups = (nblocks + self.group_blocks - 1) // self.group_blocks

        def up(n):
            return (n + 255) // 256 * 256

        buf, off, out = self.buffer, 0, {}
        for name, count, dtype, width in (("ctrl", 64, torch.int32, 4), ("perm", nblocks * 128, torch.int32, 4),
                                          ("tile_offs", nblocks * self.K + 1, torch.int32, 4),
                                          ("entries", max(self.T, 1) * 2, torch.int32, 4),
                                          ("group_order", max(ngroups, 1), torch.int32, 4),
                                          ("tile_rows", nblocks * self.K * 128, torch.int32, 4),
                                          ("buckets", (self.T // 2 + 1) * 2, torch.int32, 4)):
            out[name] = buf[off:off + count * width].view(dtype)
            off += up(count * width)
        out["entries"] = out["entries"][: self.T * 2].view(-1, 2)
        out["group_order"] = out["group_order"][:ngroups]
        out["tile_rows"] = out["tile_rows"].view(-1, 128)
        out["buckets"] = out["buckets"].view(-1, 2)[: self.multi_buckets]
        return out


def plan_group_blocks(out_width):
    """Blocks of 128 output rows that share the weight tiles they stream, for rows of ``out_width`` channels."""
    return int(lib().pcx_mvmr_plan_group_blocks(int(out_width)))


def planned_supported(weight, feat, gather, scatter, seg_offs, n_out, transpose):
    """Whether the output-stationary kernel takes this call (fp16 / bf16, one group, tap-sorted
    int32 triplets, channel counts that are multiples of 16, output rows of at most 256 channels)."""
    K, G, C, M = weight.shape
    inw, outw = (M, C) if transpose else (C, M)
    if G != 1 or seg_offs is None or feat.dtype not in (torch.float16, torch.bfloat16) or n_out <= 0:
        return False
    if inw % 16 or outw % 16 or outw > 256 or inw > 1024 or K > 512:
        return False
    T = gather.numel()
    nblocks = (int(n_out) + 127) // 128
    return T < 2 ** 31 and nblocks * K * 128 <= 2 ** 32


@on_geometry_stream
def mvmr_plan(scatter, gather, seg_offs, K, n_out, group_blocks):
    """Build the plan of a tap-sorted rulebook: ``scatter`` indexes the rows that are summed
    into (n_out of them), ``gather`` the rows that are read."""
    require_cuda(scatter, gather, seg_offs)
    scatter, gather = as_i32(scatter), as_i32(gather)
    seg_offs = seg_offs.to(torch.int64).contiguous()
    dev, T, n_out, K, G = scatter.device, scatter.numel(), int(n_out), int(K), int(group_blocks)
    L = lib()
    nbytes = L.pcx_mvmr_plan_bytes(T, n_out, K, G)
    if nbytes == 0:
        raise NotImplementedError(f"no output-stationary plan for T={T} n_out={n_out} K={K} group={G}")
    with torch.cuda.device(dev):
        buf = workspace(nbytes, dev)
        ws = workspace(L.pcx_mvmr_plan_workspace_bytes(T, n_out, K, G), dev)
        check(L.pcx_mvmr_plan_build(ptr(scatter), ptr(gather), ptr(seg_offs), T, K, n_out, G, ptr(buf), buf.numel(),
                                    ptr(ws), ws.numel(), stream_ptr()))
        multi = c_int64(0)
        check(L.pcx_mvmr_plan_multi_buckets(ptr(buf), ctypes.byref(multi), stream_ptr()))
    return MvmrPlan(buf, T, K, n_out, G, int(multi.value))


_PLAN_CACHE = {}
_PLAN_CACHE_MAX = 64
_SYMMETRIC = {}


def mark_symmetric(i, j):
    """Record that the rulebook ``(i, j, k)`` these index tensors belong to is its own mirror image:
    with ``(i, j, k)`` it holds ``(j, i, K - 1 - k)``.  True for a self-search (queries are the points):
    the distance is symmetric and the tap of the opposite offset is the mirrored tap.  The input
    gradient of such a layer is then a forward pass over the SAME rulebook with the taps of the
    weight reversed, so it needs no plan of its own (``tig_grad_input``).  Remembered by tensor
    identity, like the plans."""
    import weakref

    for key in [key for key, (refs, _) in _SYMMETRIC.items() if any(r() is None for r in refs)]:
        _SYMMETRIC.pop(key, None)
    _SYMMETRIC[(i.data_ptr(), j.data_ptr(), i.numel())] = ((weakref.ref(i), weakref.ref(j)), (i._version, j._version))


def is_symmetric(i, j):
    hit = _SYMMETRIC.get((i.data_ptr(), j.data_ptr(), i.numel()))
    if hit is None or os.environ.get("PCX_SYMMETRIC_DGRAD", "1") == "0":
        return False
    refs, stamp = hit
    return refs[0]() is i and refs[1]() is j and stamp == (i._version, j._version)


def cached_mvmr_plan(scatter, gather, seg_offs, K, n_out, group_blocks):
    """``mvmr_plan`` remembered by the identity (and version) of the index tensors, so that every
    layer and every step that shares a rulebook builds its plan once."""
    import weakref

    key = (scatter.data_ptr(), gather.data_ptr(), seg_offs.data_ptr(), scatter.numel(), int(K), int(n_out),
           int(group_blocks))
    stamp = (scatter._version, gather._version, seg_offs._version)
    hit = _PLAN_CACHE.get(key)
    if hit is not None:
        refs, old_stamp, value = hit
        if old_stamp == stamp and all(r() is t for r, t in zip(refs, (scatter, gather, seg_offs))):
            return value
    value = mvmr_plan(scatter, gather, seg_offs, K, n_out, group_blocks)
    for k in [k for k, (refs, _, _) in _PLAN_CACHE.items() if any(r() is None for r in refs)]:
        _PLAN_CACHE.pop(k, None)
    if len(_PLAN_CACHE) >= _PLAN_CACHE_MAX:
        for k in list(_PLAN_CACHE)[: _PLAN_CACHE_MAX // 2]:
            _PLAN_CACHE.pop(k, None)
    _PLAN_CACHE[key] = (tuple(weakref.ref(t) for t in (scatter, gather, seg_offs)), stamp, value)
    return value


def mvmr_planned(weight, feat, plan, transpose):
    """``out[scatter[t]] += feat[gather[t]] @ W[tap(t)]`` for the rulebook of ``plan``
    (``transpose``: use W^T); returns (plan.n_out, out_width) in feat.dtype."""
    require_cuda(weight, feat)
    K, G, C, M = weight.shape
    assert G == 1 and K == plan.K and weight.dtype == feat.dtype, (weight.shape, plan.K, weight.dtype, feat.dtype)
    weight, feat = weight.contiguous(), feat.contiguous()
    inw, outw = (M, C) if transpose else (C, M)
    out = torch.empty((plan.n_out, outw), dtype=feat.dtype, device=feat.device)
    L = lib()
    with torch.cuda.device(feat.device):
        ws = workspace(L.pcx_mvmr_planned_workspace_bytes(plan.multi_buckets, inw), feat.device)
        check(L.pcx_mvmr_planned(ptr(weight), ptr(feat), ptr(plan.buffer), plan.buffer.numel(), ptr(out), plan.T,
                                 feat.shape[0], plan.n_out, K, C, M, int(bool(transpose)), dtype_code(feat.dtype),
                                 plan.group_blocks, plan.multi_buckets, ptr(ws), ws.numel(), stream_ptr()))
    return out


def debug_wait_runs_out(limit_ns=1_000_000):
    """Launch the test kernel whose bounded wait runs out after ``limit_ns``."""
    check(lib().pcx_debug_wait_runs_out(int(limit_ns), stream_ptr()))


def mvmr(weight, feat, gather, scatter, seg_offs, tap_idx, n_out, transpose, engine=ENGINE_AUTO):
    """``out[scatter[t]] += feat[gather[t]] @ W[tap(t)]`` (``transpose``: use W^T).

    weight (K,G,C,M); feat (n_feat, G*inw); returns (n_out, G*outw) in feat.dtype.  With the
    automatic engine, wide rows and dense neighbourhoods take the output-stationary kernel
    (``ENGINE_PLANNED`` forces it), everything else the scatter engines of ``pcx_mvmr``.
    """
    require_cuda(weight, feat, gather, scatter, seg_offs, tap_idx)
    K, G, C, M = weight.shape
    code = dtype_code(feat.dtype)
    assert weight.dtype == feat.dtype, (weight.dtype, feat.dtype)
    weight, feat = weight.contiguous(), feat.contiguous()
    n_out = int(n_out)
    if engine in (ENGINE_AUTO, ENGINE_PLANNED):
        fits = planned_supported(weight, feat, gather, scatter, seg_offs, n_out, transpose)
        if engine == ENGINE_PLANNED and not fits:
            raise NotImplementedError("the output-stationary engine needs fp16/bf16 features, one group, tap-sorted "
                                      "triplets, channel counts that are multiples of 16 and rows of at most 256 channels")
        outw = C if transpose else M
        if fits and (engine == ENGINE_PLANNED or _planned_pays(gather.numel(), n_out, outw, K)):
            plan = cached_mvmr_plan(scatter, gather, seg_offs, K, n_out, plan_group_blocks(outw))
            return mvmr_planned(weight, feat, plan, transpose)
        engine = ENGINE_AUTO
    gather, scatter, tap_idx = as_i32(gather), as_i32(scatter), as_i32(tap_idx)
    if seg_offs is not None:
        seg_offs = seg_offs.to(torch.int64).contiguous()
    outw = C if transpose else M
    out = torch.empty((n_out, G * outw), dtype=feat.dtype, device=feat.device)
    L = lib()
    with torch.cuda.device(feat.device):
        nbytes = L.pcx_mvmr_workspace_bytes(n_out, K, G, C, M, int(bool(transpose)), code)
        ws = workspace(nbytes, feat.device)
        check(L.pcx_mvmr(ptr(weight), ptr(feat), ptr(gather), ptr(scatter), ptr(seg_offs), ptr(tap_idx),
                         ptr(out), gather.numel(), feat.shape[0], n_out, K, G, C, M,
                         int(bool(transpose)), code, engine, ptr(ws), ws.numel(), stream_ptr()))
    return out


def prepare_mvmr(weight, gather, scatter, seg_offs, n_out, transpose=False):
    """Build (and cache) now what ``mvmr`` with the automatic engine would build on its first call
    for this rulebook -- the plan of the output-stationary kernel, whose construction ends with a
    host hand-over -- so that the feature pass itself is kernels only.  Returns True when a plan
    was prepared, False when the policy keeps the scatter engines (which need no preparation)."""
    K, G, C, M = weight.shape
    n_out = int(n_out)
    outw = C if transpose else M
    if not (gather is not None and gather.is_cuda and planned_supported(weight, weight, gather, scatter, seg_offs,
                                                                        n_out, transpose)):
        return False
    if not _planned_pays(gather.numel(), n_out, outw, K):
        return False
    cached_mvmr_plan(scatter, gather, seg_offs, K, n_out, plan_group_blocks(outw))
    return True


def vvor(a, a_idx, b, b_idx, seg_offs, o_idx, n_o, engine=ENGINE_AUTO):
    """``out[o[t], g, m, c] += a[a_idx[t], g, m] * b[b_idx[t], g, c]``.

    a (n_a, G, Ma); b (n_b, G, Cb); returns (n_o, G, Ma, Cb) in a.dtype.
    """
    require_cuda(a, b, a_idx, b_idx, seg_offs, o_idx)
    code = dtype_code(a.dtype)
    assert a.dtype == b.dtype, (a.dtype, b.dtype)
    a, b = a.contiguous(), b.contiguous()
    G, Ma, Cb = a.shape[1], a.shape[2], b.shape[2]
    a_idx, b_idx, o_idx = as_i32(a_idx), as_i32(b_idx), as_i32(o_idx)
    if seg_offs is not None:
        seg_offs = seg_offs.to(torch.int64).contiguous()
    n_o = int(n_o)
    out = torch.empty((n_o, G, Ma, Cb), dtype=a.dtype, device=a.device)
    L = lib()
    with torch.cuda.device(a.device):
        ws = workspace(L.pcx_vvor_workspace_bytes(n_o, G, Ma, Cb, code), a.device)
        check(L.pcx_vvor(ptr(a), ptr(a_idx), ptr(b), ptr(b_idx), ptr(seg_offs), ptr(o_idx), ptr(out),
                         a_idx.numel(), a.shape[0], b.shape[0], n_o, G, Ma, Cb, code, engine,
                         ptr(ws), ws.numel(), stream_ptr()))
    return out


def vvor_static_scratch(a, a_idx, b, b_idx, seg_offs, out):
    """VVOR into the caller's ``out`` (n_o, G, Ma, Cb) using the library's built-in
    scratch array: nothing is allocated by the call, here or in the library.
    For embedders that cannot allocate device memory at the call site; see
    ``pcx_vvor_static_scratch`` in the header for the size limits and for the
    rule that calls must not overlap on the GPU."""
    require_cuda(a, b, a_idx, b_idx, seg_offs, out)
    code = dtype_code(a.dtype)
    for t in (a, b, out):
        assert t.is_contiguous() and t.dtype == a.dtype
    assert a_idx.dtype == torch.int32 and b_idx.dtype == torch.int32 and seg_offs.dtype == torch.int64
    n_o, G, Ma, Cb = out.shape
    with torch.cuda.device(a.device):
        check(lib().pcx_vvor_static_scratch(ptr(a), ptr(a_idx), ptr(b), ptr(b_idx), ptr(seg_offs), ptr(out),
                                            a_idx.numel(), a.shape[0], b.shape[0], n_o, G, Ma, Cb, code,
                                            stream_ptr()))
    return out


REDUCE_OPS = {"sum": 0, "mean": 1, "max": 2, "min": 3}


def segment_reduce(x, lengths, op):
    """``out[s] = op`` over the ``lengths[s]`` consecutive rows of segment s; x (N, C) -> (S, C)."""
    require_cuda(x, lengths)
    x = x.contiguous()
    lengths = lengths.to(torch.int64).contiguous()
    N, C = x.shape
    S = lengths.numel()
    out = torch.empty((S, C), dtype=x.dtype, device=x.device)
    L = lib()
    with torch.cuda.device(x.device):
        ws = workspace(L.pcx_segment_reduce_workspace_bytes(S, C), x.device)
        check(L.pcx_segment_reduce(ptr(x), ptr(lengths), ptr(out), N, S, C, op, dtype_code(x.dtype), ptr(ws),
                                   ws.numel(), stream_ptr()))
    return out


def segment_reduce_backward(grad_out, x, out, lengths, op, n_rows):
    require_cuda(grad_out, lengths)
    grad_out = grad_out.contiguous()
    if op >= 2:   # max / min compare x with out: both are read row-major in the gradient's element type
        assert x.dtype == grad_out.dtype and out.dtype == grad_out.dtype, (x.dtype, out.dtype, grad_out.dtype)
        x, out = x.contiguous(), out.contiguous()
    lengths = lengths.to(torch.int64).contiguous()
    S, C = grad_out.shape
    grad_x = torch.empty((n_rows, C), dtype=grad_out.dtype, device=grad_out.device)
    L = lib()
    with torch.cuda.device(grad_out.device):
        ws = workspace(L.pcx_segment_reduce_workspace_bytes(S, 1), grad_out.device)
        check(L.pcx_segment_reduce_backward(ptr(grad_out), ptr(x), ptr(out), ptr(lengths), ptr(grad_x), n_rows, S, C,
                                            op, dtype_code(grad_out.dtype), ptr(ws), ws.numel(), stream_ptr()))
    return grad_x


def indexed_segment_reduce(x, indices, lengths, op):
    """``y[k] = op`` over ``x[indices[e]]`` for the ``lengths[k]`` consecutive entries of list k."""
    require_cuda(x, indices, lengths)
    x = x.contiguous()
    indices = as_i32(indices)
    lengths = lengths.to(torch.int64).contiguous()
    n_x, C = x.shape
    K = lengths.numel()
    y = torch.empty((K, C), dtype=x.dtype, device=x.device)
    L = lib()
    code = dtype_code(x.dtype)
    with torch.cuda.device(x.device):
        ws = workspace(L.pcx_indexed_segment_reduce_workspace_bytes(K, n_x, C, code, 0), x.device)
        check(L.pcx_indexed_segment_reduce(ptr(x), ptr(indices), ptr(lengths), ptr(y), n_x, indices.numel(), K, C, op,
                                           code, ptr(ws), ws.numel(), stream_ptr()))
    return y


def indexed_segment_reduce_backward(grad_y, x, y, indices, lengths, op, n_x):
    require_cuda(grad_y, indices, lengths)
    grad_y = grad_y.contiguous()
    indices = as_i32(indices)
    lengths = lengths.to(torch.int64).contiguous()
    K, C = grad_y.shape
    grad_x = torch.empty((n_x, C), dtype=grad_y.dtype, device=grad_y.device)
    L = lib()
    code = dtype_code(grad_y.dtype)
    with torch.cuda.device(grad_y.device):
        ws = workspace(L.pcx_indexed_segment_reduce_workspace_bytes(K, n_x, C, code, 1), grad_y.device)
        check(L.pcx_indexed_segment_reduce_backward(ptr(grad_y), ptr(x), ptr(y), ptr(indices), ptr(lengths),
                                                    ptr(grad_x), n_x, indices.numel(), K, C, op, code, ptr(ws),
                                                    ws.numel(), stream_ptr()))
    return grad_x


def _f32_or_none(t):
    return None if t is None else t.detach().to(torch.float32).contiguous()


def ragged_layer_norm(x, lengths, weight, bias, residual, eps, relu):
    """Fused ``relu?(layer_norm_per_sample(x) * weight + bias (+ residual))``; returns ``(y, mean, rstd)``."""
    require_cuda(x, lengths, weight, bias, residual)
    x = x.contiguous()
    lengths = lengths.to(torch.int64).contiguous()
    weight, bias = _f32_or_none(weight), _f32_or_none(bias)
    residual = None if residual is None else residual.to(x.dtype).contiguous()
    N, C = x.shape
    S = lengths.numel()
    y = torch.empty_like(x)
    mean = torch.empty(S, dtype=torch.float32, device=x.device)
    rstd = torch.empty(S, dtype=torch.float32, device=x.device)
    L = lib()
    with torch.cuda.device(x.device):
        ws = workspace(L.pcx_ragged_layer_norm_workspace_bytes(N, S), x.device)
        check(L.pcx_ragged_layer_norm(ptr(x), ptr(lengths), ptr(weight), ptr(bias), ptr(residual), ptr(y), ptr(mean),
                                      ptr(rstd), N, S, C, float(eps), int(bool(relu)), dtype_code(x.dtype), ptr(ws),
                                      ws.numel(), stream_ptr()))
    return y, mean, rstd


def ragged_layer_norm_backward(grad_y, x, y, lengths, weight, mean, rstd, relu, want_affine, want_residual):
    """Returns ``(grad_x, grad_weight|None, grad_bias|None, grad_residual|None)`` (affine gradients in fp32)."""
    require_cuda(grad_y, x, lengths)
    grad_y, x = grad_y.contiguous(), x.contiguous()
    lengths = lengths.to(torch.int64).contiguous()
    weight = _f32_or_none(weight)
    N, C = x.shape
    S = lengths.numel()
    grad_x = torch.empty_like(x)
    gw = torch.empty(C, dtype=torch.float32, device=x.device) if want_affine else None
    gb = torch.empty(C, dtype=torch.float32, device=x.device) if want_affine else None
    gres = torch.empty_like(x) if want_residual else None
    L = lib()
    with torch.cuda.device(x.device):
        ws = workspace(L.pcx_ragged_layer_norm_workspace_bytes(N, S), x.device)
        check(L.pcx_ragged_layer_norm_backward(ptr(grad_y), ptr(x), ptr(y), ptr(lengths), ptr(weight), ptr(mean),
                                               ptr(rstd), ptr(grad_x), ptr(gw), ptr(gb), ptr(gres), N, S, C,
                                               int(bool(relu)), dtype_code(x.dtype), ptr(ws), ws.numel(),
                                               stream_ptr()))
    return grad_x, gw, gb, gres


def ragged_group_norm(x, lengths, weight, bias, groups, eps):
    """Group norm per sample (``groups`` blocks of consecutive channels; ``groups == C`` is the
    instance norm); returns ``(y, mean, rstd)`` with the statistics as (S * groups,) fp32."""
    require_cuda(x, lengths, weight, bias)
    x = x.contiguous()
    lengths = lengths.to(torch.int64).contiguous()
    weight, bias = _f32_or_none(weight), _f32_or_none(bias)
    N, C = x.shape
    S, G = lengths.numel(), int(groups)
    y = torch.empty_like(x)
    mean = torch.empty(S * G, dtype=torch.float32, device=x.device)
    rstd = torch.empty(S * G, dtype=torch.float32, device=x.device)
    L = lib()
    with torch.cuda.device(x.device):
        ws = workspace(L.pcx_ragged_group_norm_workspace_bytes(S, G), x.device)
        check(L.pcx_ragged_group_norm(ptr(x), ptr(lengths), ptr(weight), ptr(bias), ptr(y), ptr(mean), ptr(rstd),
                                      N, S, C, G, float(eps), dtype_code(x.dtype), ptr(ws), ws.numel(), stream_ptr()))
    return y, mean, rstd


def ragged_group_norm_backward(grad_y, x, lengths, weight, mean, rstd, groups, want_affine):
    """Returns ``(grad_x, grad_weight|None, grad_bias|None)`` (affine gradients in fp32)."""
    require_cuda(grad_y, x, lengths)
    grad_y, x = grad_y.contiguous(), x.contiguous()
    lengths = lengths.to(torch.int64).contiguous()
    weight = _f32_or_none(weight)
    N, C = x.shape
    S, G = lengths.numel(), int(groups)
    grad_x = torch.empty_like(x)
    gw = torch.empty(C, dtype=torch.float32, device=x.device) if want_affine else None
    gb = torch.empty(C, dtype=torch.float32, device=x.device) if want_affine else None
    L = lib()
    with torch.cuda.device(x.device):
        ws = workspace(L.pcx_ragged_group_norm_workspace_bytes(S, G), x.device)
        check(L.pcx_ragged_group_norm_backward(ptr(grad_y), ptr(x), ptr(lengths), ptr(weight), ptr(mean), ptr(rstd),
                                               ptr(grad_x), ptr(gw), ptr(gb), N, S, C, G, dtype_code(x.dtype), ptr(ws),
                                               ws.numel(), stream_ptr()))
    return grad_x, gw, gb


def seg_offs_from_sorted(idx_sorted, K):
    require_cuda(idx_sorted)
    idx = as_i32(idx_sorted)
    out = torch.empty(int(K) + 1, dtype=torch.int64, device=idx.device)
    with torch.cuda.device(idx.device):
        check(lib().pcx_seg_offs(ptr(idx), idx.numel(), int(K), ptr(out), stream_ptr()))
    return out


def expand_taps(seg_offs, K, T):
    require_cuda(seg_offs)
    out = torch.empty(int(T), dtype=torch.int32, device=seg_offs.device)
    with torch.cuda.device(seg_offs.device):
        check(lib().pcx_expand_taps(ptr(seg_offs), int(K), int(T), ptr(out), stream_ptr()))
    return out


def rnet_select(points, centres, centre_of, neighbors, offsets, source, rounds_per_call=4):
    """Residual R-net over ``points`` (n, 3): returns ``(chosen bool (n,), rounds)``.

    ``neighbors`` / ``offsets``: query-major neighbour lists within R (self included);
    ``centres[centre_of[v]]`` is the initial centre of v's stride cell; ``source`` breaks ties.
    The host sees the device once per ``rounds_per_call`` rounds."""
    require_cuda(points, centres, centre_of, neighbors, offsets, source)
    dev, n = points.device, points.shape[0]
    points, centres = points.contiguous().float(), centres.contiguous().float()
    centre_of, neighbors = centre_of.to(torch.int64).contiguous(), neighbors.to(torch.int64).contiguous()
    offsets, source = offsets.to(torch.int64).contiguous(), source.to(torch.int64).contiguous()
    far = torch.empty(n, dtype=torch.float32, device=dev)
    active = torch.ones(n, dtype=torch.uint8, device=dev)
    chosen = torch.zeros(n, dtype=torch.uint8, device=dev)
    L = lib()
    rounds = 0
    with torch.cuda.device(dev):
        check(L.pcx_rnet_far(ptr(points), ptr(centres), ptr(centre_of), n, ptr(far), stream_ptr()))
        ws = workspace(L.pcx_rnet_workspace_bytes(n, rounds_per_call), dev)
        remaining = (ctypes.c_int32 * rounds_per_call)()
        for _ in range(n + 1):           # every productive round retires at least one point
            check(L.pcx_rnet_rounds(ptr(neighbors), ptr(offsets), ptr(far), ptr(source), n, rounds_per_call,
                                    ptr(active), ptr(chosen), remaining, ptr(ws), ws.numel(), stream_ptr()))
            left = list(remaining)
            if 0 in left:
                rounds += left.index(0) + 1
                break
            rounds += rounds_per_call
        else:
            raise RuntimeError("full-cover R-net selector made no progress")
    return chosen.bool(), rounds


# -------------------------------------------------------------- geometry ----
@on_geometry_stream
def radius_search(points, queries, radius, point_sample, query_sample, distance_type,
                  kernel_size=0, kernel_grid_size=0.0, return_distances=False, want_k=False):
    """Sorted-grid fixed-radius search.

    ``kernel_size == 0``: returns ``(neighbors int64, num_neighbors int64, distances|None)``.
    ``kernel_size > 0``: returns ``(i int32, j int32, k int32|None, seg_offs int64, num_neighbors int64)``.
    Inputs must be non-empty fp32 (P,3)/(Q,3) CUDA tensors.
    """
    require_cuda(points, queries, point_sample, query_sample)
    dev = points.device
    points, queries = points.contiguous(), queries.contiguous()
    ps = as_i32(point_sample)
    qs = ps if query_sample is point_sample else as_i32(query_sample)
    P, Q = points.shape[0], queries.shape[0]
    L = lib()
    k3 = kernel_size ** 3
    if kernel_size > 0 and L.pcx_radius_taps_supported(kernel_size) and os.environ.get("PCX_RADIUS_TAPS", "1") != "0":
        return _radius_taps(points, queries, radius, ps, qs, distance_type, kernel_size, kernel_grid_size, want_k)
    with torch.cuda.device(dev):
        ws = workspace(L.pcx_radius_workspace_bytes(P, Q, kernel_size), dev)
        num_neighbors = torch.empty(Q, dtype=torch.int64, device=dev)
        seg = torch.empty(k3 + 1, dtype=torch.int64, device=dev) if kernel_size > 0 else None
        total = c_int64(0)
        check(L.pcx_radius_count(ptr(points), ptr(queries), ptr(ps), ptr(qs), P, Q, float(radius),
                                 distance_type, kernel_size, float(kernel_grid_size), ptr(num_neighbors),
                                 ptr(seg), ctypes.byref(total), ptr(ws), ws.numel(), stream_ptr()))
        total = int(total.value)
        raise_if_device_reported()   # the count above was a host hand-over: the stream is idle
        if kernel_size == 0:
            neighbors = torch.empty(total, dtype=torch.int64, device=dev)
            dist = torch.empty(total, dtype=torch.float32, device=dev) if return_distances else None
            check(L.pcx_radius_fill(ptr(points), ptr(queries), P, Q, float(radius), distance_type, 0, 0.0,
                                    total, ptr(neighbors), ptr(dist), None, None, None, ptr(ws), ws.numel(),
                                    None, 0, stream_ptr()))
            return neighbors, num_neighbors, dist
        if total > 2 ** 31 - 1:
            raise RuntimeError("prepared kernel-segment output currently requires fewer "
                               f"than 2^31 edges; got {total}")
        out_i = torch.empty(total, dtype=torch.int32, device=dev)
        out_j = torch.empty(total, dtype=torch.int32, device=dev)
        out_k = torch.empty(total, dtype=torch.int32, device=dev) if want_k else None
        ws2 = workspace(L.pcx_radius_fill_workspace_bytes(total, kernel_size), dev)
        check(L.pcx_radius_fill(ptr(points), ptr(queries), P, Q, float(radius), distance_type, kernel_size,
                                float(kernel_grid_size), total, None, None, ptr(out_i), ptr(out_j), ptr(out_k),
                                ptr(ws), ws.numel(), ptr(ws2), ws2.numel(), stream_ptr()))
    return out_i, out_j, out_k, seg, num_neighbors


# Largest pairs-per-query ratio seen per (kernel_size, distance_type, radius) -- one entry per level of a
# network: sizes the edge buffers of the next such search so that it needs one host hand-over, not two.
_TAPS_RATIO = {}


def _radius_taps(points, queries, radius, ps, qs, distance_type, kernel_size, kernel_grid_size, want_k):
    """Tap-segmented search through ``pcx_radius_taps_*``: the pairs are written into buffers sized
    from the density of earlier searches (exactly sized after a counted first call or when the
    estimate turns out too small) and returned as views of the first ``total`` entries."""
    dev = points.device
    P, Q = points.shape[0], queries.shape[0]
    L = lib()
    k3 = kernel_size ** 3
    with torch.cuda.device(dev):
        ws = workspace(L.pcx_radius_taps_workspace_bytes(P, Q, kernel_size), dev)
        num_neighbors = torch.empty(Q, dtype=torch.int64, device=dev)
        seg = torch.empty(k3 + 1, dtype=torch.int64, device=dev)
        check(L.pcx_radius_taps_count(ptr(points), ptr(queries), ptr(ps), ptr(qs), P, Q, float(radius),
                                      distance_type, kernel_size, float(kernel_grid_size), ptr(num_neighbors),
                                      ptr(seg), ptr(ws), ws.numel(), stream_ptr()))
        total = (c_int64 * 3)()
        ratio_key = (kernel_size, distance_type, float(radius))
        ratio = _TAPS_RATIO.get(ratio_key)
        if ratio is None:
            check(L.pcx_radius_taps_total(P, Q, kernel_size, total, ptr(ws), ws.numel(), stream_ptr()))
            capacity = int(total[0])
        else:
            capacity = min(int(ratio * Q * 1.25) + 4096, 2 ** 31 - 1)
        for attempt in range(2):
            out_i = torch.empty(capacity, dtype=torch.int32, device=dev)
            out_j = torch.empty(capacity, dtype=torch.int32, device=dev)
            out_k = torch.empty(capacity, dtype=torch.int32, device=dev) if want_k else None
            rc = L.pcx_radius_taps_fill(ptr(queries), ptr(ps), ptr(qs), P, Q, float(radius), distance_type,
                                        kernel_size, float(kernel_grid_size), capacity, ptr(out_i), ptr(out_j),
                                        ptr(out_k), total, ptr(ws), ws.numel(), stream_ptr())
            if rc == PCX_E_CAPACITY and attempt == 0 and int(total[0]) > capacity:
                capacity = int(total[0])   # the estimate was too small: exact size, fill pass only
                continue
            check(rc)
            break
        if total[2]:                 # the hand-over of the fill pass brought the status word along
            raise_if_device_reported()
        n = int(total[0])
        if len(_TAPS_RATIO) > 256:
            _TAPS_RATIO.clear()
        _TAPS_RATIO[ratio_key] = max(ratio or 0.0, n / Q)
        num_neighbors.pcx_queries_without_neighbor = int(total[1])   # spares the caller a pass over the counts
    return out_i[:n], out_j[:n], (out_k[:n] if want_k else None), seg, num_neighbors


@on_geometry_stream
def grid_sample_center_nearest(points, cell, sample, return_mapping):
    """Returns ``(indices int64 (S,), points_f (S,3), sample_f int32 (S,)|None, mapping int64|None)``."""
    require_cuda(points, sample)
    dev = points.device
    points = points.contiguous()
    smp = as_i32(sample)
    N = points.shape[0]
    L = lib()
    with torch.cuda.device(dev):
        ws = workspace(L.pcx_grid_sample_workspace_bytes(N), dev)
        ncells = c_int64(0)
        check(L.pcx_grid_sample_count(ptr(points), ptr(smp), N, float(cell), ctypes.byref(ncells), ptr(ws),
                                      ws.numel(), stream_ptr()))
        S = int(ncells.value)
        indices = torch.empty(S, dtype=torch.int64, device=dev)
        out_pts = torch.empty((S, 3), dtype=torch.float32, device=dev)
        out_smp = torch.empty(S, dtype=torch.int32, device=dev) if smp is not None else None
        mapping = torch.empty(N, dtype=torch.int64, device=dev) if return_mapping else None
        check(L.pcx_grid_sample_select(ptr(points), ptr(smp), N, float(cell), S, ptr(indices), ptr(out_pts),
                                       ptr(out_smp), ptr(mapping), ptr(ws), ws.numel(), stream_ptr()))
    return indices, out_pts, out_smp, mapping
