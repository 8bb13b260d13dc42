"""Build ``libf2cgt_b200.so`` (the C-ABI library, include/f2cgt_b200.h) in-tree with plain nvcc.

The library has no torch, pybind or Python dependency: it is CUDA C++ compiled for sm_100a only and
linked against the static CUDA runtime.  ``python -m f2cgt_b200.build`` rebuilds what is stale;
``--force`` rebuilds everything; ``--verbose`` prints ptxas resource usage (-Xptxas -v).
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(PKG, "libf2cgt_b200.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "f2cgt_b200.h")

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc():
    return os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def _deps_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [HEADER]
    return max(os.path.getmtime(h) for h in hs)


def build(force=False, verbose=False, jobs=8):
    os.makedirs(OBJ, exist_ok=True)
    dep_t = _deps_mtime()
    units = [(s, os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")) for s in sources()]

    def compile_one(pair):
        src, obj = pair
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), dep_t):
            return 0, src, ""
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        return p.returncode, src, p.stderr

    with ThreadPoolExecutor(max_workers=jobs) as ex:
        results = list(ex.map(compile_one, units))
    for rc, src, err in results:
        if rc != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{err[-6000:]}")
        if verbose and err:
            print(f"== {os.path.basename(src)}\n{err}")
    objs = [o for _, o in units]
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, "-gencode", "arch=compute_100a,code=sm_100a"] + objs
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stderr[-4000:]}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
