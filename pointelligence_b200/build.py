"""Build libpointelligence_b200.so in-tree with nvcc for sm_100a.

    python -m pointelligence_b200.build [--force]

One object per translation unit under ``csrc/`` (compiled in parallel), linked
into ``pointelligence_b200/lib/libpointelligence_b200.so`` against the shared
CUDA runtime so that the library and PyTorch use the same runtime instance.
nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "lib", "obj")
LIB = os.path.join(HERE, "lib", "libpointelligence_b200.so")
SOURCES = ("status.cu", "geometry.cu", "sparse_generic.cu", "sparse_tc.cu", "sparse_api.cu",
           "sparse_noalloc.cu", "segment_reduce.cu", "ragged_norm.cu", "mvmr_os.cu", "rnet.cu", "radius_taps.cu")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xptxas", "-v"] + os.environ.get("PCX_NVCC_EXTRA", "").split()


def _deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "pointelligence_b200.h"))
    return deps


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src):
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    log = obj + ".log"
    cmd = [NVCC, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stderr[-4000:]}")
    return obj


def build(force=False, verbose=False):
    deps = _deps()
    if not force and not _stale(LIB, deps):
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(_compile, SOURCES))
    rpaths = ["/usr/local/cuda/lib64"]
    try:
        import nvidia.cuda_runtime  # the runtime PyTorch loads

        rpaths.insert(0, os.path.join(list(nvidia.cuda_runtime.__path__)[0], "lib"))
    except Exception:
        pass
    cmd = [NVCC, "-shared", "-cudart", "shared", "-o", LIB, *objs]
    for r in rpaths:
        cmd += ["-Xlinker", "-rpath", "-Xlinker", r]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    if verbose:
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    build(force=a.force, verbose=True)
    sys.exit(0)
