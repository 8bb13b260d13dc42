"""TEST INFRASTRUCTURE ONLY.  Build the reference's own RAFT-free CUDA sources into a Python
extension ``oracle/_ref/f2cgt_ref*.so`` so that its kernels can be run next to ours on a B200.

The sources are compiled where they lie in the reference checkout (nothing is copied); the only
file of ours in the build is ``oracle/ref_binding.cu``.  Flags follow the reference's CMake build
(C++17, ``--expt-extended-lambda``, Release -O3, default math flags so FMA contraction and the
libdevice ``exp2f``/``log2f`` are the ones the reference ships) with the architecture fixed to
sm_100a.  ``src/kmeans.cu`` and ``src/pybind.cu`` need RAFT 23.10 headers that are fetched from the
network by the reference's CMake and are therefore left out.

Usage: ``python oracle/build_ref.py [--reference /path/to/F2CGT] [--jobs N]``.  A missing reference
checkout is not an error: the script prints a note and exits 0 (prebuilt files are used as is).
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REF_SOURCES = ["sq_quantization.cu", "vq_quantization.cu", "packbits.cu", "fusion_spmm.cu",
               "fusion_dropout.cu"]


def ext_suffix():
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def target_path():
    return os.path.join(OUT, "f2cgt_ref" + ext_suffix())


def build(reference, jobs=5, force=False, verbose=True):
    src_dir = os.path.join(reference, "src")
    if not os.path.isdir(src_dir):
        if verbose:
            print(f"[build_ref] no reference checkout at {reference}; keeping prebuilt files")
        return None
    os.makedirs(OUT, exist_ok=True)
    import torch
    from torch.utils import cpp_extension as ce
    import pybind11

    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    incs = ce.include_paths() + [sysconfig.get_paths()["include"], pybind11.get_include(), src_dir]
    common = [nvcc, "-std=c++17", "-O3", "--expt-extended-lambda", "--expt-relaxed-constexpr",
              "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
              "-DTORCH_EXTENSION_NAME=f2cgt_ref", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-w"]
    for i in incs:
        common += ["-isystem", i]

    units = [(os.path.join(src_dir, s), os.path.join(OUT, s.replace(".cu", ".o"))) for s in REF_SOURCES]
    units.append((os.path.join(HERE, "ref_binding.cu"), os.path.join(OUT, "ref_binding.o")))

    def stale(src, obj):
        return force or not os.path.exists(obj) or os.path.getmtime(obj) < os.path.getmtime(src)

    def compile_one(pair):
        src, obj = pair
        if not stale(src, obj):
            return 0, src, ""
        p = subprocess.run(common + ["-c", src, "-o", obj], capture_output=True, text=True)
        return p.returncode, src, p.stderr[-4000:]

    with ThreadPoolExecutor(max_workers=jobs) as ex:
        results = list(ex.map(compile_one, units))
    for rc, src, err in results:
        if rc != 0:
            raise RuntimeError(f"[build_ref] nvcc failed on {src}:\n{err}")
    tgt = target_path()
    objs = [o for _, o in units]
    if force or not os.path.exists(tgt) or any(os.path.getmtime(o) > os.path.getmtime(tgt) for o in objs):
        libdirs = ce.library_paths()
        link = [nvcc, "-shared", "-o", tgt] + objs
        for d in libdirs:
            link += ["-L" + d, "-Xlinker", "-rpath=" + d]
        link += ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-ltorch_python",
                 "-lcudart", "-lcurand"]
        p = subprocess.run(link, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"[build_ref] link failed:\n{p.stderr[-4000:]}")
    if verbose:
        print(f"[build_ref] ok: {tgt}")
    return tgt


def load():
    """Import the built reference extension (GPU box only: every op allocates CUDA tensors)."""
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    tgt = target_path()
    if not os.path.exists(tgt):
        raise FileNotFoundError(tgt)
    spec = importlib.util.spec_from_file_location("f2cgt_ref", tgt)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--reference", default=os.environ.get("F2CGT_REFERENCE") or os.path.join(os.path.dirname(here), "reference"),
                    help="checkout of gpzlx1/F2CGT (default: $F2CGT_REFERENCE, else a directory `reference` beside this repository)")
    ap.add_argument("--jobs", type=int, default=5)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    build(a.reference, a.jobs, a.force)
    sys.exit(0)
