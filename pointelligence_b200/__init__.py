"""Blackwell (sm_100a) implementation of the point-convolution hot path of
PointCNN++ behind the reference's ``sparse_engines`` / ``layers`` /
``internals`` interfaces.

Sub-packages mirror the reference modules they stand in for:

    pointelligence_b200.sparse_engines   ops, tig, _dispatch_override, _seg_offs
    pointelligence_b200.internals        neighbors, grid_sample, grid_indexing, indexing
    pointelligence_b200.layers           conv, contract, metadata, triplets, downsample

All device work is done by hand-written CUDA kernels in
``lib/libpointelligence_b200.so`` (sources under ``csrc/``, C ABI in
``include/pointelligence_b200.h``).  There is no CPU fallback: calling an
operator without the library or without a CUDA tensor raises.
"""

__version__ = "0.1.0"
