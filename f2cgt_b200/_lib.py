"""ctypes binding of ``libf2cgt_b200.so`` (C ABI in include/f2cgt_b200.h).

The library is the only compute path of this package: if it is missing or fails to load, importing
this module raises - there is no CPU or PyTorch fallback.
"""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("F2CGT_B200_LIB") or os.path.join(_PKG, "libf2cgt_b200.so")  # override: another build of the same ABI

# dtype tags of include/f2cgt_b200.h
U8, I8, I16, I32, I64, F16, F32, F64 = range(8)
MEAN, SUM = 0, 1
L2, COSINE = 0, 1
SCORER_EXACT, SCORER_TENSOR = 0x100, 0x200
# f2c_kernel: kernel family of a fused aggregation call
KERNELS = {"auto": 0, "stream": 1, "prefetch": 2, "general": 3, "prefetch_arith": 4}

STATUS_NAMES = {1: "invalid argument", 2: "unsupported", 3: "CUDA error", 4: "size limit"}


class Epilogue(C.Structure):
    _fields_ = [("p", C.c_float), ("training", C.c_int), ("scale", C.c_int), ("seed", C.c_uint64),
                ("offset", C.c_uint64), ("kernel", C.c_int)]


class F2CError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m f2cgt_b200.build` (needs nvcc); "
            "f2cgt_b200 has no fallback path")
    return C.CDLL(LIB_PATH)


lib = _load()

p, i64, ci, u64, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_uint64, C.c_float
EP = C.POINTER(Epilogue)

# name -> argtypes; every function returns an int status except the ones listed in _RESTYPE
SIGNATURES = {
    "f2c_packbits": [p, p, i64, i64, ci, p],
    "f2c_unpackbits": [p, p, i64, i64, i64, ci, p],
    "f2c_sq_compress": [p, p, p, i64, i64, i64, ci, i64, p],
    "f2c_sq_decompress": [p, ci, p, i64, p, i64, i64, i64, ci, i64, p],
    "f2c_vq_decompress": [p, ci, p, ci, p, i64, i64, i64, i64, i64, p],
    "f2c_spmm_csr": [p, ci, p, p, ci, p, i64, i64, ci, p],
    "f2c_spmm_csr_backward": [p, p, p, ci, p, i64, i64, i64, ci, p],
    "f2c_sq_spmm_csr": [p, ci, p, i64, p, p, ci, p, i64, i64, i64, i64, ci, i64, ci, EP, p],
    "f2c_sq_spmm_csr_peer": [p, ci, i64, ci, p, i64, p, p, ci, p, i64, i64, i64, i64, ci, i64, ci, EP, p],
    "f2c_peer_hot_first_cold_id": [i64, i64],
    "f2c_sq_spmm_csr_peer_hot": [p, i64, p, ci, i64, ci, p, i64, p, p, ci, p, i64, i64, i64, i64, ci, i64, ci, EP, p],
    "f2c_shard_create": [p, i64, p, p, p],
    "f2c_shard_free": [p],
    "f2c_shard_open": [p, p],
    "f2c_shard_close": [p],
    "f2c_shard_copy": [p, p, i64, p],
    "f2c_vq_spmm_csr": [p, ci, p, p, p, ci, p, i64, i64, i64, i64, i64, ci, EP, p],
    "f2c_hybrid_decompress": [p, ci, p, i64, ci, i64, i64, i64, p, ci, p, i64, i64, i64, i64, p, i64, p],
    "f2c_hybrid_spmm_csr": [p, ci, p, i64, ci, i64, i64, p, ci, p, i64, i64, i64, p, i64, p, p, ci, p, i64, i64, ci, EP, p],
    "f2c_hybrid_spmm_csr_peer": [p, p, p, ci, i64, i64, i64, i64, ci, p, i64, ci, i64, i64, ci, p, i64, i64, i64, p, p, ci, p, i64, i64,
                                 ci, EP, p],
    "f2c_dropout": [p, i64, f32, ci, u64, u64, ci, p],
    "f2c_pairwise_distance": [p, p, p, i64, i64, i64, ci, p],
    "f2c_kmeans_assign_workspace": [i64, i64, i64],
    "f2c_kmeans_assign": [p, p, p, i64, i64, i64, ci, p, p],
    "f2c_kmeans_assign_static": [p, p, p, i64, i64, i64, ci, p],
    "f2c_kmeans_assign_static_status": [p, p, p],
    "f2c_device_status": [p, p],
    "f2c_check_csc": [p, p, ci, i64, i64, p, p],
    "f2c_relabel_capacity": [i64],
    "f2c_relabel_mark": [p, ci, i64, p, p, i64, p, p, p],
    "f2c_relabel_assign": [p, ci, i64, p, p, i64, p, p, p, p, p],
    "f2c_sample_degrees": [p, p, p, ci, i64, ci, p],
    "f2c_sample_neighbors": [p, p, p, p, p, i64, ci, i64, ci, u64, u64, p],
    "f2c_sample_block_workspace": [i64, ci, ci],
    "f2c_sample_block": [p, p, p, ci, i64, ci, u64, u64, p, p, p, p, p, p, i64, p],
    "f2c_last_error": [],
    "f2c_version": [],
}
_RESTYPE = {"f2c_last_error": C.c_char_p, "f2c_kmeans_assign_workspace": C.c_int64, "f2c_relabel_capacity": C.c_int64,
            "f2c_sample_block_workspace": C.c_int64, "f2c_peer_hot_first_cold_id": C.c_int64}

for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = header and library out of step
    _fn.argtypes = _args
    _fn.restype = _RESTYPE.get(_name, C.c_int)


def check(status):
    if status != 0:
        msg = lib.f2c_last_error().decode("utf-8", "replace")
        raise F2CError(f"f2cgt_b200: {STATUS_NAMES.get(status, status)}: {msg}")
