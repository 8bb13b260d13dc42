"""CPU: the C-ABI library loads and exports every entry point include/f2cgt_b200.h declares
(no kernel is launched here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "f2cgt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(f2c_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_surface():
    syms = declared_symbols()
    for name in ["f2c_packbits", "f2c_unpackbits", "f2c_sq_compress", "f2c_sq_decompress", "f2c_vq_decompress",
                 "f2c_spmm_csr", "f2c_sq_spmm_csr", "f2c_vq_spmm_csr", "f2c_hybrid_decompress", "f2c_hybrid_spmm_csr",
                 "f2c_dropout", "f2c_pairwise_distance", "f2c_kmeans_assign", "f2c_last_error"]:
        assert name in syms


def test_library_exports_every_declared_symbol():
    from f2cgt_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    # and the Python binding knows each of them
    for name in declared_symbols():
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_argument_validation_needs_no_gpu():
    # bad arguments are rejected before any CUDA call, so this runs on a CPU-only machine
    from f2cgt_b200 import _lib
    lib = _lib.lib
    rc = lib.f2c_packbits(None, None, 4, 8, 3, None)
    assert rc == 2 and b"target_bits" in lib.f2c_last_error()
    rc = lib.f2c_sq_decompress(None, _lib.I16, None, 1, None, 4, 16, 128, 4, 128, None)
    assert rc == 2  # packed codes cannot be an int16 tensor
    rc = lib.f2c_sq_decompress(None, _lib.U8, None, 1, None, 4, 16, 128, 4, 128, None)
    assert rc == 1 and b"exceeds" in lib.f2c_last_error()  # 16 bytes hold 32 4-bit elements, not 128
    rc = lib.f2c_sq_spmm_csr(None, _lib.U8, None, 5, None, None, _lib.I64, None, 4, 9, 64, 128, 4, 31, 0, None, None)
    assert rc == 1 and b"column_slice" in lib.f2c_last_error()
    rc = lib.f2c_vq_spmm_csr(None, _lib.U8, None, None, None, _lib.I16, None, 4, 4, 256, 32, 128, 0, None, None)
    assert rc == 2  # int16 indices
    rc = lib.f2c_dropout(None, 10, 1.5, 1, 0, 0, 0, None)
    assert rc == 1
    assert lib.f2c_kmeans_assign(None, None, None, 10, 0, 8, 0, None, None) == 1
    # hot-first numbering of a sharded table: the sharded rows' ids start at the next multiple of the shard size
    assert lib.f2c_peer_hot_first_cold_id(0, 100) == 0 and lib.f2c_peer_hot_first_cold_id(1, 100) == 100
    assert lib.f2c_peer_hot_first_cold_id(100, 100) == 100 and lib.f2c_peer_hot_first_cold_id(101, 100) == 200
    # ... and the replicated rows share the kernel's 16 pointer slots with the shards
    import ctypes as C
    fake = (C.c_void_p * 8)(*[0x1000] * 8)
    rc = lib.f2c_sq_spmm_csr_peer_hot(0x1000, 901, fake, 8, 100, _lib.U8, None, 1, None, None, _lib.I64, None, 4, 1700, 64, 128, 4, 128, 0, None, None)
    assert rc == 1 and b"16 slots" in lib.f2c_last_error()
    assert lib.f2c_sample_block_workspace(0, 12, _lib.I64) == 0 and lib.f2c_sample_block_workspace(1024, 12, _lib.I64) > 1024 * 13 * 12
    # zero-sized work is a no-op, not an error
    assert lib.f2c_packbits(None, None, 0, 8, 4, None) == 0
    assert lib.f2c_sq_spmm_csr(None, _lib.U8, None, 1, None, None, _lib.I64, None, 0, 9, 64, 128, 4, 128, 0, None, None) == 0


def test_python_surface_matches_reference_module():
    import inspect
    import F2CGTLib as capi
    # names and argument names of src/pybind.cu:8-28
    expect = {
        "packbits": ["unpack", "target_bits"],
        "unpackbits": ["pack", "target_bits", "unpack_dim"],
        "sq_compress": ["src", "codebooks", "target_bits", "column_slice"],
        "sq_decompress": ["compress_data", "codebooks", "target_bits", "column_slice", "feat_dim"],
        "vq_decompress": ["index_tensor", "codebooks", "feat_dim"],
        "pairwise_distance": ["x", "y", "metric"],
        "spmm_csr": ["feat", "indptr", "indices"],
        "vq_decompress_spmm_csr": ["compress_feat", "codebooks", "indptr", "indices", "feat_dim"],
        "sq_decompress_spmm_csr": ["compress_feat", "codebooks", "indptr", "indices", "target_bit", "column_slice", "feat_dim"],
    }
    for name, args in expect.items():
        params = list(inspect.signature(getattr(capi, name)).parameters)
        assert params[:len(args)] == args, name
    assert hasattr(capi, "KMeans") and hasattr(capi.KMeans, "fit") and hasattr(capi.KMeans, "predict") and hasattr(capi.KMeans, "get_centers")
    import torch
    import pytest
    with pytest.raises(RuntimeError):
        capi.packbits(torch.zeros(2, 8, dtype=torch.uint8), 4)  # CPU tensor is rejected, never silently computed
