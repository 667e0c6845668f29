"""Ahead-of-time build of the sm_100a kernels into one in-tree shared library.

`nvcc` compiles every `csrc/*.cu` for compute_100a/sm_100a only and links `libtileinfer_b200.so`
next to this file; a stamp with the hash of the sources and flags makes rebuilds a no-op.  There is
no JIT cache: the library is loaded with ctypes and its `extern "C"` launchers take raw device
pointers and a stream, so they can be captured into CUDA graphs.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libtileinfer_b200.so")
STAMP = os.path.join(BUILD, "stamp.txt")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-DTI_GEMV_WARPS=" + os.environ.get("TI_GEMV_WARPS", "16"),
              "-DTI_GEMV_TPS=" + os.environ.get("TI_GEMV_TPS", "8"),
              "-DTI_GEMM_RING_KB=" + os.environ.get("TI_GEMM_RING_KB", "192"),
              "-DTI_GEMV_PREFETCH_KB=" + os.environ.get("TI_GEMV_PREFETCH_KB", "0")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources() -> list:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _hash() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _hash()


# The checked variant: every peer-buffer / KV-page / workspace index that comes from run-time data goes through
# TI_CHECK (common.cuh), which records kStatusBounds in the status word and SKIPS the access instead of faulting;
# TI_JITTER adds random __nanosleep delays before packet sends and collects (stress of the flag protocols).
# Selected at run time with TI_DEBUG_LIB=1 (see lib.py).
DEBUG_FLAGS = ["-DTI_BOUNDS_CHECK", "-DTI_JITTER"]
LIB_DEBUG = os.path.join(HERE, "libtileinfer_b200_dbg.so")
BUILD_DEBUG = os.path.join(HERE, "build_dbg")


def build_debug(force: bool = False) -> str:
    """Compile the bounds-checked, jittered variant of the library (same sources, DEBUG_FLAGS)."""
    global LIB, BUILD, STAMP, NVCC_FLAGS
    keep = (LIB, BUILD, STAMP, NVCC_FLAGS)
    LIB, BUILD, STAMP = LIB_DEBUG, BUILD_DEBUG, os.path.join(BUILD_DEBUG, "stamp.txt")
    NVCC_FLAGS = keep[3] + DEBUG_FLAGS
    try:
        return build(force)
    finally:
        LIB, BUILD, STAMP, NVCC_FLAGS = keep


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile (if needed) and return the path of the shared library."""
    if not force and is_current():
        return LIB
    os.makedirs(BUILD, exist_ok=True)
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    build_dir, lib_path, stamp_path = BUILD, LIB, STAMP

    def one(src):
        obj = os.path.join(build_dir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(one, sources()))
    cmd = [nvcc, "-shared", "-o", lib_path, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(stamp_path, "w") as f:
        f.write(_hash())
    return lib_path


if __name__ == "__main__":
    if "--debug" in sys.argv:
        print(build_debug(force="--force" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
