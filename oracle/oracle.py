"""TEST INFRASTRUCTURE ONLY - numpy front end of the C restatement in ``oracle/f2c_oracle.c``.

Only ``tests/``, the smoke test and the benchmark's CPU legs may import this module; the product
package never does.  Inputs and outputs are numpy arrays; shapes and dtypes mirror the reference
operators (src/pybind.cu:8-28 of gpzlx1/F2CGT).  ``build()`` compiles the C file with gcc into
``oracle/liboracle.so`` (git-ignored) and is idempotent.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "f2c_oracle.c")
LIB = os.path.join(HERE, "liboracle.so")

DT = {np.dtype(np.uint8): 0, np.dtype(np.int8): 1, np.dtype(np.int16): 2, np.dtype(np.int32): 3,
      np.dtype(np.int64): 4, np.dtype(np.float16): 5, np.dtype(np.float32): 6, np.dtype(np.float64): 7}

_lib = None


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-o", LIB, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(LIB)
        _lib.orc_dropout_threshold.restype = C.c_uint32
        _lib.orc_dropout_threshold.argtypes = [C.c_float]
    return _lib


def _p(a):
    return C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(0)


def _c(a, dtype=None):
    a = np.ascontiguousarray(a)
    if dtype is not None and a.dtype != np.dtype(dtype):
        a = a.astype(dtype)
    return a


i64 = C.c_int64
ci = C.c_int


def packbits(unpack, bits):
    unpack = _c(unpack, np.uint8)
    rows, dim = unpack.shape
    per = 8 // bits
    out = np.empty((rows, (dim + per - 1) // per), np.uint8)
    lib().orc_packbits(_p(unpack), _p(out), i64(rows), i64(dim), ci(bits))
    return out


def unpackbits(pack, bits, unpack_dim):
    pack = _c(pack).view(np.uint8)
    rows, pdim = pack.shape
    out = np.empty((rows, unpack_dim), np.uint8)
    lib().orc_unpackbits(_p(pack), _p(out), i64(rows), i64(unpack_dim), i64(pdim), ci(bits))
    return out


def sq_compress(src, codebooks, bits, column_slice):
    src, codebooks = _c(src, np.float32), _c(codebooks, np.float32)
    out = np.empty_like(src)
    lib().orc_sq_compress(_p(src), _p(out), _p(codebooks), i64(src.shape[0]), i64(src.shape[1]), ci(bits),
                          i64(column_slice))
    return out


def sq_compress_prefloor(src, codebooks, bits, column_slice):
    src, codebooks = _c(src, np.float32), _c(codebooks, np.float32)
    out = np.empty_like(src)
    lib().orc_sq_compress_prefloor(_p(src), _p(out), _p(codebooks), i64(src.shape[0]), i64(src.shape[1]),
                                   ci(bits), i64(column_slice))
    return out


def sq_codes_to_storage(float_codes, bits):
    """What callers do with sq_compress output (examples/process_compress.py:131-139)."""
    if bits < 8:
        return packbits(float_codes.astype(np.uint8), bits)
    if bits == 8:
        return float_codes.astype(np.int8)
    return float_codes.astype(np.int16)


def sq_decompress(codes, codebooks, bits, column_slice, feat_dim):
    codes, codebooks = _c(codes), _c(codebooks, np.float32)
    out = np.empty((codes.shape[0], feat_dim), np.float32)
    lib().orc_sq_decompress(_p(codes), ci(DT[codes.dtype]), _p(out), _p(codebooks), i64(codes.shape[0]),
                            i64(codes.shape[1]), i64(feat_dim), ci(bits), i64(column_slice))
    return out


def vq_decompress(codes, codebooks, feat_dim):
    codes, codebooks = _c(codes), _c(codebooks)
    n_cb, K, cs = codebooks.shape
    out = np.empty((codes.shape[0], feat_dim), np.float32)
    lib().orc_vq_decompress(_p(codes), ci(DT[codes.dtype]), _p(codebooks), ci(DT[codebooks.dtype]), _p(out),
                            i64(codes.shape[0]), i64(n_cb), i64(K), i64(cs), i64(feat_dim))
    return out


def spmm_csr(feat, indptr, indices, reduce="mean"):
    feat, indptr, indices = _c(feat), _c(indptr), _c(indices)
    assert indptr.dtype == indices.dtype
    n_dst = indptr.shape[0] - 1
    out = np.empty((n_dst, feat.shape[1]), feat.dtype)
    fn = {np.dtype(np.float32): lib().orc_spmm_csr_f32, np.dtype(np.float64): lib().orc_spmm_csr_f64,
          np.dtype(np.float16): lib().orc_spmm_csr_f16}[feat.dtype]
    fn(_p(feat), _p(out), _p(indptr), _p(indices), ci(DT[indptr.dtype]), i64(n_dst), i64(feat.shape[1]),
       ci(0 if reduce == "mean" else 1))
    return out


def sq_decompress_spmm_csr(codes, codebooks, indptr, indices, bits, column_slice, feat_dim, reduce="mean",
                           acc64=False):
    codes, codebooks, indptr, indices = _c(codes), _c(codebooks, np.float32), _c(indptr), _c(indices)
    n_dst = indptr.shape[0] - 1
    out = np.empty((n_dst, feat_dim), np.float32)
    lib().orc_sq_spmm_csr(_p(codes), ci(DT[codes.dtype]), _p(codebooks), _p(indptr), _p(indices),
                          ci(DT[indptr.dtype]), _p(out), i64(n_dst), i64(codes.shape[1]), i64(feat_dim),
                          ci(bits), i64(column_slice), ci(0 if reduce == "mean" else 1), ci(int(acc64)))
    return out


def vq_decompress_spmm_csr(codes, codebooks, indptr, indices, feat_dim, reduce="mean", acc64=False):
    codes, codebooks, indptr, indices = _c(codes), _c(codebooks, np.float32), _c(indptr), _c(indices)
    n_cb, K, cs = codebooks.shape
    n_dst = indptr.shape[0] - 1
    out = np.empty((n_dst, feat_dim), np.float32)
    lib().orc_vq_spmm_csr(_p(codes), ci(DT[codes.dtype]), _p(codebooks), _p(indptr), _p(indices),
                          ci(DT[indptr.dtype]), _p(out), i64(n_dst), i64(n_cb), i64(K), i64(cs),
                          i64(feat_dim), ci(0 if reduce == "mean" else 1), ci(int(acc64)))
    return out


def fusion_decompress(sq_codes, sq_codebooks, bits, column_slice, vq_codes, vq_codebooks, feat_dim):
    sq_codes, sq_codebooks = _c(sq_codes), _c(sq_codebooks, np.float32)
    vq_codes, vq_codebooks = _c(vq_codes), _c(vq_codebooks, np.float32)
    n_cb, K, cs = vq_codebooks.shape
    out = np.empty((sq_codes.shape[0] + vq_codes.shape[0], feat_dim), np.float32)
    lib().orc_hybrid_decompress(_p(sq_codes), ci(DT[sq_codes.dtype]), _p(sq_codebooks), ci(bits),
                                i64(column_slice), i64(sq_codes.shape[0]), i64(sq_codes.shape[1]),
                                _p(vq_codes), ci(DT[vq_codes.dtype]), _p(vq_codebooks), i64(vq_codes.shape[0]),
                                i64(n_cb), i64(K), i64(cs), _p(out), i64(feat_dim))
    return out


def two_level_decompress_spmm_csr(sq_codes, sq_codebooks, bits, column_slice, vq_codes, vq_codebooks, slot,
                                  indptr, indices, feat_dim, reduce="mean", acc64=False):
    sq_codes, sq_codebooks = _c(sq_codes), _c(sq_codebooks, np.float32)
    vq_codes, vq_codebooks = _c(vq_codes), _c(vq_codebooks, np.float32)
    slot, indptr, indices = _c(slot, np.int32), _c(indptr), _c(indices)
    n_cb, K, cs = vq_codebooks.shape
    n_dst = indptr.shape[0] - 1
    out = np.empty((n_dst, feat_dim), np.float32)
    lib().orc_hybrid_spmm_csr(_p(sq_codes), ci(DT[sq_codes.dtype]), _p(sq_codebooks), ci(bits),
                              i64(column_slice), i64(sq_codes.shape[1]), _p(vq_codes), ci(DT[vq_codes.dtype]),
                              _p(vq_codebooks), i64(n_cb), i64(K), i64(cs), _p(slot), _p(indptr), _p(indices),
                              ci(DT[indptr.dtype]), _p(out), i64(n_dst), i64(feat_dim),
                              ci(0 if reduce == "mean" else 1), ci(int(acc64)))
    return out


def dropout(x, p, training=True, seed=0, offset=0, scale=False):
    x = _c(x, np.float32).copy()
    lib().orc_dropout(_p(x), i64(x.size), C.c_float(p), ci(int(training)), C.c_uint64(seed),
                      C.c_uint64(offset), ci(int(scale)))
    return x


_METRIC = {"cosine": 1}


def pairwise_distance(x, y, metric):
    x, y = _c(x, np.float32), _c(y, np.float32)
    out = np.empty((x.shape[0], y.shape[0]), np.float32)
    lib().orc_pairwise_distance(_p(x), _p(y), _p(out), i64(x.shape[0]), i64(y.shape[0]), i64(x.shape[1]),
                                ci(_METRIC.get(metric, 0)))
    return out


def kmeans_assign(x, centers, metric, with_margin=False):
    x, centers = _c(x, np.float32), _c(centers, np.float32)
    n = x.shape[0]
    labels = np.empty(n, np.int64)
    best = np.empty(n, np.float64)
    second = np.empty(n, np.float64)
    lib().orc_kmeans_assign(_p(x), _p(centers), _p(labels), _p(best), _p(second), i64(n), i64(centers.shape[0]),
                            i64(x.shape[1]), ci(_METRIC.get(metric, 0)))
    return (labels, best, second) if with_margin else labels


def sq_codebook_row(sample):
    """Codebook recipe [fmin, fmax, emin, emax, mean] of tests/test_sq.py:8-21 and
    examples/process_compress.py:55-68 (0.5 / 99.5 percentiles of |x|, log2 range, mean(|x|) + 0.1
    when below 0.1), evaluated in fp32 like the reference's torch code."""
    eps = 1e-5
    a = np.abs(np.asarray(sample, np.float32))
    fmin = np.float32(max(np.percentile(a, 0.5), eps))
    fmax = np.float32(max(np.percentile(a, 99.5), 2 * eps))
    emin = np.log2(fmin, dtype=np.float32)
    emax = np.float32(np.log2(fmax, dtype=np.float32) + np.float32(eps))
    mean = np.float32(a.mean(dtype=np.float32))
    if mean < 0.1:
        mean = np.float32(mean + np.float32(0.1))
    return np.array([fmin, fmax, emin, emax, mean], np.float32)


def sq_codebooks(data, column_slice):
    D = data.shape[1]
    n_cb = (D + column_slice - 1) // column_slice
    return np.stack([sq_codebook_row(data[:, i * column_slice:min((i + 1) * column_slice, D)])
                     for i in range(n_cb)])


def sample_neighbors(indptr, indices, seeds, num_pick, rng_seed=0, rng_offset=0):
    """CSC over ``seeds`` with at most ``num_pick`` uniformly chosen distinct in-neighbours each."""
    indptr, indices, seeds = _c(indptr, np.int64), _c(indices, np.int64), _c(seeds, np.int64)
    deg = np.minimum(indptr[seeds + 1] - indptr[seeds], num_pick)
    out_indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    out_indices = np.empty(int(out_indptr[-1]), np.int64)
    lib().orc_sample_neighbors(_p(indptr), _p(indices), _p(seeds), _p(out_indptr), _p(out_indices), i64(seeds.shape[0]),
                               ci(num_pick), C.c_uint64(rng_seed), C.c_uint64(rng_offset))
    return out_indptr, out_indices


def tensor_relabel(tensors):
    """Contract of the reference's ``tensor_relabel([seeds, sub_indices])`` as its call sites use it
    (examples/dataloader.py:176-177,289-290; examples/conv.py:48-49): distinct ids of the concatenation numbered in
    order of first occurrence (so distinct seeds keep positions 0..len(seeds)-1), every id replaced by its number."""
    arrs = [np.asarray(t).reshape(-1) for t in tensors]
    keys = np.concatenate(arrs) if arrs else np.zeros(0, np.int64)
    _, first_idx, inverse = np.unique(keys, return_index=True, return_inverse=True)
    order = np.argsort(first_idx, kind="stable")          # sorted-unique slots in order of first occurrence
    rank_of_slot = np.empty_like(order)
    rank_of_slot[order] = np.arange(order.size)
    unique = keys[np.sort(first_idx)]
    relabelled = rank_of_slot[inverse].astype(keys.dtype)
    out, off = [], 0
    for a in arrs:
        out.append(relabelled[off:off + a.size])
        off += a.size
    return unique, out
