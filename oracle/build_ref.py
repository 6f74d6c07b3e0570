"""Build recipe for the oracle's shared objects (TEST INFRASTRUCTURE).

Outputs go to ``oracle/_ref/`` only (git-ignored build artefacts):

``liboracle_sparse.so``
    ``gcc`` on ``oracle/mvmr_vvor.c`` -- the plain-C restatement.

``libsparse_engines_ref_cpu.so``
    ``g++`` on the reference's own CPU operator sources, compiled where they
    lie (``extensions/sparse_engines_cuda/csrc/{definitions,spare_mvmr,
    sparse_vvor,common}.cpp``) with the reference's flags (``-O3
    -DWITHOUT_CUDA``, as in ``extensions/setup.py:57-58,107-108``).  Only built
    when the reference checkout is present; the sources are never copied.
    Loading it registers ``torch.ops.sparse_engines_cuda.*`` for CPU tensors.

Run ``python -m oracle.build_ref`` (optionally ``--reference DIR``).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(OUT, "liboracle_sparse.so")
REF_SO = os.path.join(OUT, "libsparse_engines_ref_cpu.so")
# the reference checkout: POINTELLIGENCE_REFERENCE, else a directory "reference" beside this repository
DEFAULT_REFERENCE = os.environ.get("POINTELLIGENCE_REFERENCE",
                                   os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
_REF_SOURCES = ("definitions.cpp", "spare_mvmr.cpp", "sparse_vvor.cpp", "common.cpp")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle_c(force=False):
    src = os.path.join(HERE, "mvmr_vvor.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    os.makedirs(OUT, exist_ok=True)
    cmd = ["gcc", "-O3", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off",
           src, "-lm", "-o", ORACLE_SO]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_reference_cpu_ops(reference=DEFAULT_REFERENCE, force=False):
    """Returns the path of the built library, or None if the reference
    checkout is absent (then a previously built copy is used if it exists)."""
    csrc = os.path.join(reference, "extensions", "sparse_engines_cuda", "csrc")
    sources = [os.path.join(csrc, f) for f in _REF_SOURCES]
    if not all(os.path.exists(s) for s in sources):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, sources):
        return REF_SO
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT, exist_ok=True)
    cmd = ["g++", "-O3", "-DWITHOUT_CUDA", "-std=c++17", "-fPIC", "-shared",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-I", sysconfig.get_paths()["include"]]
    cmd += sources
    for lib in cpp_extension.library_paths():
        cmd += ["-L", lib, "-Wl,-rpath," + lib]
    cmd += ["-ltorch", "-ltorch_cpu", "-lc10", "-o", REF_SO]
    subprocess.run(cmd, check=True)
    return REF_SO


def build_all(reference=DEFAULT_REFERENCE, force=False):
    return build_oracle_c(force), build_reference_cpu_ops(reference, force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_all(a.reference, a.force))
