"""CPU oracle for the point-convolution hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory.  The only callers are the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark, where the oracle
plays the role of the checker (or of the timed CPU baseline), never of the
product.

Contents
--------
``geometry``     numpy restatement of the reference's geometry stage: sorted
                 eight-cell fixed-radius search, tap-segmented triplet
                 emission, centre-nearest grid down-sampling.
``sparse_ops``   fp64 and fp32 restatements of MVMR / VVOR plus loaders for the
                 compiled C restatement (``mvmr_vvor.c``) and for the reference's
                 own CPU operators compiled from its sources (``_ref/``).
``build_ref``    build recipe for both shared objects.

Parity status: pinned.  Every function is checked in ``tests/`` against the
known-answer fixtures of the reference's own unit tests and against the
golden vectors under ``tests/golden/`` that were produced by running the
reference's Python code (CPU torch path, and its Triton geometry kernels under
Triton's CPU interpreter) in the build container.
"""
