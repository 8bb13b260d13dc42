"""The ``F2CGTLib`` operator surface (gpzlx1/F2CGT src/pybind.cu:7-47) over the B200 C-ABI library.

Same names, positional/keyword arguments and return conventions as the reference's pybind11 module:
inputs are CUDA tensors that are only borrowed, outputs are fresh tensors on the input's device.
Differences, all additive:
  * work is queued on the caller's current CUDA stream (the reference always uses the legacy
    default stream, e.g. src/fusion_spmm.cu:261);
  * bad arguments raise ``RuntimeError`` instead of aborting the process (src/common.h:29,51,64,80,102)
    or reading out of bounds;
  * operators the reference's callers use but its module does not bind: ``fusion_decompress``
    (tests/test_fusion_decompress.py:40), ``dropout_inplace`` (src/fusion_dropout.cu:21),
    ``two_level_decompress_spmm_csr`` and the ``reduce=`` / ``dropout=`` keywords.

torch is used for memory and streams only; every computation is a kernel of libf2cgt_b200.so.
"""
import torch

from . import _lib
from ._lib import lib, check, Epilogue

_DT = {torch.uint8: _lib.U8, torch.int8: _lib.I8, torch.int16: _lib.I16, torch.int32: _lib.I32,
       torch.int64: _lib.I64, torch.float16: _lib.F16, torch.float32: _lib.F32, torch.float64: _lib.F64}
_REDUCE = {"mean": _lib.MEAN, "sum": _lib.SUM}


def _metric(name):
    # src/kmeans.cu:107-112: "cosine" selects the cosine distance, any other string the squared L2
    return _lib.COSINE if name == "cosine" else _lib.L2


def _chk(t, name, dtypes=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise RuntimeError(f"{name} has unsupported dtype {t.dtype}")
    return t


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t):
    return t.data_ptr() if t is not None else 0


class _on:
    """Make the tensor's device current for the duration of a call (kernels launch on it)."""

    def __init__(self, t):
        self.g = torch.cuda.device(t.device)

    def __enter__(self):
        self.g.__enter__()

    def __exit__(self, *a):
        return self.g.__exit__(*a)


def _epilogue(dropout, kernel="auto"):
    """Per-call options: dropout = None or dict(p=..., seed=..., offset=0, training=True, scale=False); kernel = one of
    ``_lib.KERNELS`` ("auto" lets the library choose; the others pin a kernel family - same bits, for tests and timing)."""
    if dropout is None and kernel == "auto":
        return None
    if dropout is None:
        return Epilogue(0.0, 0, 0, 0, 0, _lib.KERNELS[kernel])
    return Epilogue(float(dropout["p"]), int(dropout.get("training", True)), int(dropout.get("scale", False)),
                    int(dropout.get("seed", 0)) & 0xFFFFFFFFFFFFFFFF, int(dropout.get("offset", 0)), _lib.KERNELS[kernel])


def _check_block(check, indptr, indices, n_src):
    """check=True: verify the CSC block on the device first (indptr non-decreasing from 0, every index in [0, n_src));
    the fused kernels trust ``indices`` like the reference does, so a debugging caller can ask."""
    if not check:
        return
    flag = torch.zeros(1, dtype=torch.int32, device=indptr.device)
    with _on(indptr):
        _lib.check(lib.f2c_check_csc(_ptr(indptr), _ptr(indices), _DT[indptr.dtype], indptr.numel() - 1, int(n_src), _ptr(flag),
                                     _stream(indptr)))
    code = int(flag.item())
    if code != 0:
        raise RuntimeError(f"invalid CSC block (code {code}): indptr must be non-decreasing from 0 and every index in [0, {n_src})")


def device_status(device=None):
    """0, or the code of a bounded wait that ran out inside a kernel since the last query (synchronises the current stream)."""
    import ctypes
    code = ctypes.c_int32(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        check(lib.f2c_device_status(ctypes.byref(code), torch.cuda.current_stream(dev).cuda_stream))
    return int(code.value)


# ------------------------------------------------------------------ bit packing
def packbits(unpack, target_bits):
    """src/packbits.cu:44-64.  unpack uint8 [rows, dim] -> uint8 [rows, ceil(dim*bits/8)]."""
    _chk(unpack, "unpack", (torch.uint8,))
    if unpack.dim() != 2:
        raise RuntimeError("unpack must be 2-D")
    if target_bits not in (1, 2, 4):
        raise RuntimeError(f"TARGET_BITS can only be [1,2,4] for packbits (got {target_bits})")
    per = 8 // target_bits
    rows, dim = unpack.shape
    pack = torch.empty((rows, (dim + per - 1) // per), dtype=torch.uint8, device=unpack.device)
    with _on(unpack):
        check(lib.f2c_packbits(_ptr(unpack), _ptr(pack), rows, dim, target_bits, _stream(unpack)))
    return pack


def unpackbits(pack, target_bits, unpack_dim):
    """src/packbits.cu:97-114."""
    _chk(pack, "pack", (torch.uint8, torch.int8))
    if pack.dim() != 2:
        raise RuntimeError("pack must be 2-D")
    unpack = torch.empty((pack.shape[0], unpack_dim), dtype=torch.uint8, device=pack.device)
    with _on(pack):
        check(lib.f2c_unpackbits(_ptr(pack), _ptr(unpack), pack.shape[0], pack.shape[1], unpack_dim, target_bits,
                                 _stream(pack)))
    return unpack


# ------------------------------------------------------------------ scalar quantisation
def sq_compress(src, codebooks, target_bits, column_slice):
    """src/sq_quantization.cu:65-83.  Returns float32 codes with the shape of ``src``; the caller casts
    (``.to(uint8)`` + packbits, ``.to(int8)`` or ``.to(int16)``, examples/process_compress.py:131-139)."""
    _chk(src, "src", (torch.float32,))
    _chk(codebooks, "codebooks", (torch.float32,))
    if src.dim() != 2 or codebooks.dim() != 2 or codebooks.shape[1] != 5:
        raise RuntimeError("src must be [rows, feat_dim] and codebooks [n, 5]")
    out = torch.empty_like(src)
    with _on(src):
        check(lib.f2c_sq_compress(_ptr(src), _ptr(out), _ptr(codebooks), codebooks.shape[0], src.shape[0], src.shape[1],
                                  target_bits, column_slice, _stream(src)))
    return out


def sq_decompress(compress_data, codebooks, target_bits, column_slice, feat_dim):
    """src/sq_quantization.cu:158-182.  Codes [rows, src_dim] -> float32 [rows, feat_dim]."""
    _chk(compress_data, "compress_data", (torch.uint8, torch.int8, torch.int16))
    _chk(codebooks, "codebooks", (torch.float32,))
    if compress_data.dim() != 2:
        raise RuntimeError("compress_data must be 2-D")
    rows, src_dim = compress_data.shape
    out = torch.empty((rows, feat_dim), dtype=torch.float32, device=compress_data.device)
    with _on(compress_data):
        check(lib.f2c_sq_decompress(_ptr(compress_data), _DT[compress_data.dtype], _ptr(codebooks), codebooks.shape[0],
                                    _ptr(out), rows, src_dim, feat_dim, target_bits, column_slice, _stream(compress_data)))
    return out


# ------------------------------------------------------------------ vector quantisation
def vq_decompress(index_tensor, codebooks, feat_dim):
    """src/vq_quantization.cu:35-60.  Codes [rows, n_cb], codebooks [n_cb, K, cs] (fp32/fp16) -> fp32."""
    _chk(index_tensor, "index_tensor", (torch.uint8, torch.int8, torch.int16))
    _chk(codebooks, "codebooks", (torch.float32, torch.float16))
    if index_tensor.dim() != 2 or codebooks.dim() != 3 or index_tensor.shape[1] != codebooks.shape[0]:
        raise RuntimeError("index_tensor must be [rows, n_codebooks] and codebooks [n_codebooks, length, column_slice]")
    rows = index_tensor.shape[0]
    n_cb, K, cs = codebooks.shape
    out = torch.empty((rows, feat_dim), dtype=torch.float32, device=index_tensor.device)
    with _on(index_tensor):
        check(lib.f2c_vq_decompress(_ptr(index_tensor), _DT[index_tensor.dtype], _ptr(codebooks), _DT[codebooks.dtype],
                                    _ptr(out), rows, n_cb, K, cs, feat_dim, _stream(index_tensor)))
    return out


# ------------------------------------------------------------------ aggregation
def _csc(indptr, indices):
    _chk(indptr, "indptr", (torch.int32, torch.int64))
    _chk(indices, "indices", (torch.int32, torch.int64))
    if indptr.dtype != indices.dtype:
        raise RuntimeError("indptr and indices must have the same dtype")
    if indptr.dim() != 1 or indptr.numel() < 1:
        raise RuntimeError("indptr must be 1-D with at least one element")
    return indptr.numel() - 1


def _block_out(n_dst, width, dtype, device, out_rows):
    """Output of a block kernel: ``[n_dst, width]``, or - with ``out_rows > n_dst`` - ``[out_rows, width]`` whose rows behind
    ``n_dst`` are zero: a caller that pads row counts to a few recurring sizes (for the matrix products that follow) gets
    the padded tensor without a copy."""
    if out_rows is None or out_rows <= n_dst:
        return torch.empty((n_dst, width), dtype=dtype, device=device)
    out = torch.empty((int(out_rows), width), dtype=dtype, device=device)
    out[n_dst:].zero_()
    return out


def spmm_csr(feat, indptr, indices, reduce="mean", out_rows=None):
    """src/fusion_spmm.cu:45-70.  Mean of neighbour rows; output has the dtype of ``feat``."""
    _chk(feat, "feat", (torch.float32, torch.float16, torch.float64))
    n_dst = _csc(indptr, indices)
    if feat.dim() != 2:
        raise RuntimeError("feat must be 2-D")
    out = _block_out(n_dst, feat.shape[1], feat.dtype, feat.device, out_rows)
    with _on(feat):
        check(lib.f2c_spmm_csr(_ptr(feat), _DT[feat.dtype], _ptr(indptr), _ptr(indices), _DT[indptr.dtype], _ptr(out), n_dst,
                               feat.shape[1], _REDUCE[reduce], _stream(feat)))
    return out


def spmm_csr_backward(grad_out, indptr, indices, n_src, reduce="mean"):
    """Gradient of ``spmm_csr(feat, indptr, indices)`` with respect to ``feat`` (float32 [n_src, D]): every edge adds
    ``grad_out[d] / max(deg(d), 1)`` (mean) or ``grad_out[d]`` (sum) to the row of its source."""
    _chk(grad_out, "grad_out", (torch.float32,))
    n_dst = _csc(indptr, indices)
    if grad_out.dim() != 2 or grad_out.shape[0] != n_dst:
        raise RuntimeError("grad_out must be [n_dst, feat_dim]")
    grad = torch.empty((int(n_src), grad_out.shape[1]), dtype=torch.float32, device=grad_out.device)
    with _on(grad_out):
        check(lib.f2c_spmm_csr_backward(_ptr(grad_out), _ptr(indptr), _ptr(indices), _DT[indptr.dtype], _ptr(grad), n_dst, int(n_src),
                                        grad_out.shape[1], _REDUCE[reduce], _stream(grad_out)))
    return grad


def sq_decompress_spmm_csr(compress_feat, codebooks, indptr, indices, target_bit, column_slice, feat_dim, reduce="mean",
                           dropout=None, kernel="auto", check=False, out_rows=None):
    """src/fusion_spmm.cu:240-272.  Fused SQ decode + mean aggregation -> float32 [n_dst, feat_dim]."""
    _chk(compress_feat, "compress_feat", (torch.uint8, torch.int8, torch.int16))
    _chk(codebooks, "codebooks", (torch.float32,))
    n_dst = _csc(indptr, indices)
    if compress_feat.dim() != 2:
        raise RuntimeError("compress_feat must be 2-D")
    _check_block(check, indptr, indices, compress_feat.shape[0])
    out = _block_out(n_dst, feat_dim, torch.float32, compress_feat.device, out_rows)
    ep = _epilogue(dropout, kernel)
    with _on(compress_feat):
        _lib.check(lib.f2c_sq_spmm_csr(_ptr(compress_feat), _DT[compress_feat.dtype], _ptr(codebooks), codebooks.shape[0],
                                  _ptr(indptr), _ptr(indices), _DT[indptr.dtype], _ptr(out), n_dst, compress_feat.shape[0],
                                       compress_feat.shape[1], feat_dim, target_bit, column_slice, _REDUCE[reduce], ep,
                                       _stream(compress_feat)))
    return out


def peer_first_cold_id(n_replicated, rows_per_shard):
    """Id of the first sharded row of a table whose ``n_replicated`` hottest rows are kept on every GPU: the next multiple
    of the shard size (ids between ``n_replicated`` and it are unused)."""
    return int(lib.f2c_peer_hot_first_cold_id(int(n_replicated), int(rows_per_shard)))


def sq_decompress_spmm_csr_peer(peer_table, codebooks, indptr, indices, target_bit, column_slice, feat_dim, reduce="mean",
                                dropout=None, kernel="auto", out_rows=None, replicated=None):
    """``sq_decompress_spmm_csr`` over a row-sharded table (``f2cgt_b200.shard.PeerTable``): indices are global row ids,
    remote rows are read by the kernel itself over NVLink.

    ``replicated``: a local tensor with the most often sampled rows of a table numbered hot rows first - ids below
    ``len(replicated)`` read it, id ``peer_first_cold_id(len(replicated), peer_table.rpr) + r`` reads row r of the sharded
    table (the cold remainder; its ids start at a multiple of the shard size so that one division locates any row)."""
    import ctypes
    _chk(codebooks, "codebooks", (torch.float32,))
    n_dst = _csc(indptr, indices)
    out = _block_out(n_dst, feat_dim, torch.float32, indptr.device, out_rows)
    if len(peer_table.pointers) != peer_table.world:
        raise RuntimeError("the peer table is closed")
    n_rep = 0
    if replicated is not None:
        _chk(replicated, "replicated", (peer_table.dtype,))
        if replicated.dim() != 2 or replicated.shape[1] != peer_table.row_width or replicated.device != indptr.device:
            raise RuntimeError("replicated must hold rows of the sharded table's width on the block's device")
        n_rep = replicated.shape[0]
    ptrs = (ctypes.c_void_p * peer_table.world)(*peer_table.pointers)
    ep = _epilogue(dropout, kernel)
    with _on(indptr):
        check(lib.f2c_sq_spmm_csr_peer_hot(_ptr(replicated) if n_rep else 0, n_rep, ptrs, peer_table.world, peer_table.rpr,
                                           _DT[peer_table.dtype], _ptr(codebooks), codebooks.shape[0], _ptr(indptr), _ptr(indices),
                                           _DT[indptr.dtype], _ptr(out), n_dst, peer_first_cold_id(n_rep, peer_table.rpr) + peer_table.n_rows,
                                           peer_table.row_width,
                                           feat_dim, target_bit, column_slice, _REDUCE[reduce], ep, _stream(indptr)))
    return out


def vq_decompress_spmm_csr(compress_feat, codebooks, indptr, indices, feat_dim, reduce="mean", dropout=None, kernel="auto",
                           check=False, out_rows=None):
    """src/fusion_spmm.cu:107-141.  Fused VQ decode + mean aggregation -> float32 [n_dst, feat_dim]."""
    _chk(compress_feat, "compress_feat", (torch.uint8, torch.int8, torch.int16))
    _chk(codebooks, "codebooks", (torch.float32,))
    n_dst = _csc(indptr, indices)
    if compress_feat.dim() != 2 or codebooks.dim() != 3 or compress_feat.shape[1] != codebooks.shape[0]:
        raise RuntimeError("compress_feat must be [rows, n_codebooks] and codebooks [n_codebooks, length, column_slice]")
    n_cb, K, cs = codebooks.shape
    _check_block(check, indptr, indices, compress_feat.shape[0])
    out = _block_out(n_dst, feat_dim, torch.float32, compress_feat.device, out_rows)
    ep = _epilogue(dropout, kernel)
    with _on(compress_feat):
        _lib.check(lib.f2c_vq_spmm_csr(_ptr(compress_feat), _DT[compress_feat.dtype], _ptr(codebooks), _ptr(indptr), _ptr(indices),
                                  _DT[indptr.dtype], _ptr(out), n_dst, n_cb, K, cs, feat_dim, _REDUCE[reduce], ep,
                                  _stream(compress_feat)))
    return out


def fusion_decompress(sq_data, sq_codebooks, target_bits, column_slice, vq_data, vq_codebooks, feat_dim):
    """cat(sq_decompress(sq_data, ...), vq_decompress(vq_data, ...)) in one launch
    (tests/test_fusion_decompress.py:32-43)."""
    _chk(sq_data, "sq_data", (torch.uint8, torch.int8, torch.int16))
    _chk(sq_codebooks, "sq_codebooks", (torch.float32,))
    _chk(vq_data, "vq_data", (torch.uint8, torch.int8, torch.int16))
    _chk(vq_codebooks, "vq_codebooks", (torch.float32,))
    n_cb, K, cs = vq_codebooks.shape
    out = torch.empty((sq_data.shape[0] + vq_data.shape[0], feat_dim), dtype=torch.float32, device=sq_data.device)
    with _on(sq_data):
        check(lib.f2c_hybrid_decompress(_ptr(sq_data), _DT[sq_data.dtype], _ptr(sq_codebooks), sq_codebooks.shape[0],
                                        target_bits, column_slice, sq_data.shape[0], sq_data.shape[1], _ptr(vq_data),
                                        _DT[vq_data.dtype], _ptr(vq_codebooks), vq_data.shape[0], n_cb, K, cs, _ptr(out),
                                        feat_dim, _stream(sq_data)))
    return out


def two_level_decompress_spmm_csr(sq_data, sq_codebooks, target_bits, column_slice, vq_data, vq_codebooks, slot, indptr,
                                  indices, feat_dim, reduce="mean", dropout=None, kernel="auto", check=False, out_rows=None):
    """Two-level aggregation in one launch.  Source row s is decoded from row ``slot[s]`` of the SQ table
    when ``slot[s] >= 0`` (int32), from row s of the VQ table otherwise; then the reference mean.
    ``slot=None``: hot-first numbering - the hot nodes are ids ``0 .. len(sq_data) - 1`` and node s reads SQ row s."""
    _chk(sq_data, "sq_data", (torch.uint8, torch.int8, torch.int16))
    _chk(sq_codebooks, "sq_codebooks", (torch.float32,))
    _chk(vq_data, "vq_data", (torch.uint8, torch.int8, torch.int16))
    _chk(vq_codebooks, "vq_codebooks", (torch.float32,))
    if slot is not None:
        _chk(slot, "slot", (torch.int32,))
    n_dst = _csc(indptr, indices)
    n_cb, K, cs = vq_codebooks.shape
    _check_block(check, indptr, indices, vq_data.shape[0])
    out = _block_out(n_dst, feat_dim, torch.float32, vq_data.device, out_rows)
    ep = _epilogue(dropout, kernel)
    with _on(vq_data):
        _lib.check(lib.f2c_hybrid_spmm_csr(_ptr(sq_data), _DT[sq_data.dtype], _ptr(sq_codebooks), sq_codebooks.shape[0],
                                      target_bits, column_slice, sq_data.shape[1], _ptr(vq_data), _DT[vq_data.dtype],
                                      _ptr(vq_codebooks), n_cb, K, cs, _ptr(slot), sq_data.shape[0], _ptr(indptr), _ptr(indices),
                                      _DT[indptr.dtype], _ptr(out), n_dst, feat_dim, _REDUCE[reduce], ep, _stream(vq_data)))
    return out


def two_level_decompress_spmm_csr_peer(sq_peers, sq_codebooks, target_bits, column_slice, vq_peers, vq_codebooks, slot_peers, indptr,
                                       indices, feat_dim, reduce="mean", dropout=None, out_rows=None):
    """``two_level_decompress_spmm_csr`` (or, with ``sq_peers=None``, ``vq_decompress_spmm_csr``) over tables row-sharded across
    the GPUs of the box (``f2cgt_b200.shard.PeerTable`` objects: VQ codes and slots sharded by node id, hot SQ rows by slot):
    indices are global node ids, the kernel reads remote rows itself over NVLink.  ``slot_peers=None``: hot-first numbering."""
    import ctypes
    _chk(vq_codebooks, "vq_codebooks", (torch.float32,))
    n_dst = _csc(indptr, indices)
    n_cb, K, cs = vq_codebooks.shape
    world = vq_peers.world

    def ptrs(t):
        if t is None:
            return None
        if len(t.pointers) != world:
            raise RuntimeError("a peer table is closed or spans another number of ranks")
        return (ctypes.c_void_p * world)(*t.pointers)
    two = sq_peers is not None
    if two:
        _chk(sq_codebooks, "sq_codebooks", (torch.float32,))
    out = _block_out(n_dst, feat_dim, torch.float32, indptr.device, out_rows)
    ep = _epilogue(dropout)
    with _on(indptr):
        check(lib.f2c_hybrid_spmm_csr_peer(ptrs(sq_peers), ptrs(vq_peers), ptrs(slot_peers), world, vq_peers.rpr,
                                           sq_peers.rpr if two else 0, vq_peers.n_rows, sq_peers.n_rows if two else 0,
                                           _DT[sq_peers.dtype] if two else _lib.I8, _ptr(sq_codebooks) if two else 0,
                                           sq_codebooks.shape[0] if two else 1, int(target_bits) if two else 8, int(column_slice) if two else 1,
                                           sq_peers.row_width if two else 1, _DT[vq_peers.dtype], _ptr(vq_codebooks), n_cb, K, cs,
                                           _ptr(indptr), _ptr(indices), _DT[indptr.dtype], _ptr(out), n_dst, feat_dim, _REDUCE[reduce], ep,
                                           _stream(indptr)))
    return out


# ------------------------------------------------------------------ dropout
def dropout_inplace(output, p, is_training, seed=None, offset=0, scale=False):
    """src/fusion_dropout.cu:21-29: zero with probability p when training, survivors unchanged
    (``scale=True`` multiplies them by 1/(1-p)); returns its argument.  ``seed=None`` draws a seed from
    torch's generator (the reference seeds from the wall clock)."""
    _chk(output, "output", (torch.float32,))
    if seed is None:
        seed = int(torch.randint(0, 2**62, (1,)).item())
    with _on(output):
        check(lib.f2c_dropout(_ptr(output), output.numel(), float(p), int(bool(is_training)), seed & 0xFFFFFFFFFFFFFFFF,
                              int(offset), int(bool(scale)), _stream(output)))
    return output


# ------------------------------------------------------------------ k-means
def pairwise_distance(x, y, metric):
    """src/kmeans.cu:102-118.  x [n,d], y [k,d] fp32 -> [n,k] squared-L2 or cosine distance."""
    _chk(x, "x", (torch.float32,))
    _chk(y, "y", (torch.float32,))
    if x.dim() != 2 or y.dim() != 2 or x.shape[1] != y.shape[1]:
        raise RuntimeError("x must be [n, d] and y [k, d]")
    dist = torch.empty((x.shape[0], y.shape[0]), dtype=torch.float32, device=x.device)
    with _on(x):
        check(lib.f2c_pairwise_distance(_ptr(x), _ptr(y), _ptr(dist), x.shape[0], y.shape[0], x.shape[1], _metric(metric),
                                        _stream(x)))
    return dist


def kmeans_assign(x, centers, metric, scorer="auto"):
    """labels[i] = first argmin_c dist(x_i, centers_c), int64 (src/kmeans.cu:77-98).  scorer = "auto" | "exact" (fp32 FMA) |
    "tensor" (tcgen05 + exact re-score of undecided points): same labels, pinned per call for tests and timing."""
    _chk(x, "data", (torch.float32,))
    _chk(centers, "centers", (torch.float32,))
    if x.dim() != 2 or centers.dim() != 2 or x.shape[1] != centers.shape[1]:
        raise RuntimeError("data must be [n, d] and centers [k, d]")
    n, d = x.shape
    k = centers.shape[0]
    labels = torch.empty((n,), dtype=torch.int64, device=x.device)
    ws_bytes = lib.f2c_kmeans_assign_workspace(n, k, d)
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=x.device) if ws_bytes > 0 else None
    if ws is not None:
        ws[:256].zero_()  # header: [undecided count, error code]; the library clears it again when it uses the scratch
    with _on(x):
        flags = {"auto": 0, "exact": _lib.SCORER_EXACT, "tensor": _lib.SCORER_TENSOR}[scorer]
        check(lib.f2c_kmeans_assign(_ptr(x), _ptr(centers), _ptr(labels), n, k, d, _metric(metric) | flags, _ptr(ws) if ws is not None else 0,
                                    _stream(x)))
    if ws is not None:
        # word 1 of the scratch header is set when the tensor-core kernel gave up on a bounded wait
        head = ws[:8].view(torch.int32).cpu()
        if int(head[1]) != 0:
            raise RuntimeError("f2cgt_b200: kmeans_assign: tensor-core kernel reported a timed-out wait")
        kmeans_assign.last_undecided = int(head[0])
    return labels


class KMeans:
    """src/pybind.cu:29-47 / src/kmeans.cu:13-100.  ``KMeans(n_cluster, feat_dim, metric, ...)`` or
    ``KMeans(centers, metric, ...)``; the second form aliases ``centers`` (src/kmeans.cu:55) and
    ``get_centers()`` returns that alias (:100)."""

    _DEFAULTS = dict(max_iter=300, tol=1e-4, n_init=1, oversampling_factor=2.0, batch_samples=1 << 15,
                     batch_centroids=0, inertia_check=False)

    def __init__(self, *args, **kw):
        from_centers = (len(args) > 0 and isinstance(args[0], torch.Tensor)) or "centers" in kw
        names = (["centers", "metric"] if from_centers else ["n_cluster", "feat_dim", "metric"]) + list(self._DEFAULTS)
        if len(args) > len(names):
            raise TypeError("KMeans(): too many positional arguments")
        params = dict(self._DEFAULTS)
        params.update(zip(names, args))
        for name, v in kw.items():
            if name not in names or name in names[:len(args)]:
                raise TypeError(f"KMeans(): unexpected or repeated argument '{name}'")
            params[name] = v
        missing = [n for n in names if n not in params]
        if missing:
            raise TypeError(f"KMeans(): missing arguments {missing}")
        self.metric = params["metric"]
        self.max_iter, self.tol, self.n_init = int(params["max_iter"]), float(params["tol"]), int(params["n_init"])
        if from_centers:
            c = params["centers"]
            if not c.is_cuda:
                raise RuntimeError("centers must be a CUDA tensor")
            self.cluster_centers = c
            self.init = "array"
        else:
            self.cluster_centers = torch.zeros((int(params["n_cluster"]), int(params["feat_dim"])), dtype=torch.float32,
                                               device="cuda")
            # src/kmeans.cu:16-22: cosine -> random initial centres, otherwise k-means++
            self.init = "random" if self.metric == "cosine" else "kmeans++"
        self.num_clusters = self.cluster_centers.shape[0]

    def fit(self, data):
        from .kmeans_fit import lloyd_fit
        if not data.is_cuda:
            raise RuntimeError("x must be a CUDA tensor")
        centers = lloyd_fit(data.float().contiguous(), self.num_clusters, self.metric, self.init,
                            self.cluster_centers if self.init == "array" else None, self.max_iter, self.tol, self.n_init)
        self.cluster_centers.copy_(centers)

    def predict(self, data, normalize_weights=True):
        if not data.is_cuda:
            raise RuntimeError("x must be a CUDA tensor")
        return kmeans_assign(data.contiguous(), self.cluster_centers.contiguous(), self.metric)

    def get_centers(self):
        return self.cluster_centers


# ------------------------------------------------------------------ neighbour sampling
def csr_sampling(indptr, indices, seeds, num_pick, replace=False, rng_seed=0, rng_offset=0, exact=True):
    """The reference's ``ShmTensorLib.csr_sampling(indptr, indices, seeds, num_pick, replace)`` (call sites
    examples/dataloader.py:174-175,287-288): uniform sampling of at most ``num_pick`` in-neighbours per seed
    without replacement.  Returns ``(sub_indptr, sub_indices)``, a CSC over the seeds with global ids.

    ``exact=False`` skips the host read of the edge count: ``sub_indices`` then has ``len(seeds) * num_pick`` entries, the
    ones behind ``sub_indptr[-1]`` being copies of ``seeds[0]`` (a block's kernels only read what ``sub_indptr`` spans, and
    relabelling the padded tensor numbers the nodes exactly as relabelling the used part would)."""
    if replace:
        raise RuntimeError("csr_sampling: only replace=False is implemented (the reference never passes True)")
    _chk(indptr, "indptr", (torch.int32, torch.int64))
    _chk(indices, "indices", (indptr.dtype,))
    _chk(seeds, "seeds", (indptr.dtype,))
    n = seeds.numel()
    deg = torch.empty((n,), dtype=indptr.dtype, device=indptr.device)
    st = _stream(indptr)
    with _on(indptr):
        check(lib.f2c_sample_degrees(_ptr(indptr), _ptr(seeds), _ptr(deg), _DT[indptr.dtype], n, int(num_pick), st))
        sub_indptr = torch.zeros((n + 1,), dtype=indptr.dtype, device=indptr.device)
        torch.cumsum(deg, 0, out=sub_indptr[1:])
        if exact or n == 0:
            nnz, capacity = (int(sub_indptr[-1].item()) if n > 0 else 0), 0
        else:
            nnz = capacity = n * int(num_pick)
        sub_indices = torch.empty((nnz,), dtype=indptr.dtype, device=indptr.device)
        check(lib.f2c_sample_neighbors(_ptr(indptr), _ptr(indices), _ptr(seeds), _ptr(sub_indptr), _ptr(sub_indices), capacity,
                                       _DT[indptr.dtype], n, int(num_pick), int(rng_seed) & 0xFFFFFFFFFFFFFFFF,
                                       int(rng_offset), st))
    return sub_indptr, sub_indices


def tensor_relabel(tensors):
    """The reference's ``ShmTensorLib.tensor_relabel([seeds, sub_indices])`` (call sites
    examples/dataloader.py:176-177,289-290): returns ``(unique, relabelled)`` where ``unique`` holds the distinct ids of
    the concatenation in order of first occurrence (distinct seeds keep positions 0..len(seeds)-1, which the model
    relies on: examples/conv.py:48-49) and ``relabelled[j]`` is ``tensors[j]`` rewritten to positions in ``unique``."""
    tensors = list(tensors)
    if not tensors:
        raise RuntimeError("tensor_relabel: needs at least one tensor")
    for t in tensors:
        _chk(t, "ids", (torch.int32, torch.int64))
        if t.dtype != tensors[0].dtype or t.device != tensors[0].device:
            raise RuntimeError("tensor_relabel: all tensors must share dtype and device")
    keys = torch.cat([t.reshape(-1) for t in tensors])
    n = keys.numel()
    dev, dt = keys.device, keys.dtype
    if n == 0:
        return keys, [t.clone() for t in tensors]
    cap = lib.f2c_relabel_capacity(n)
    tab_keys = torch.empty((cap,), dtype=torch.int64, device=dev)
    tab_pos = torch.empty((cap,), dtype=torch.int32, device=dev)
    first = torch.empty((n,), dtype=torch.int32, device=dev)
    err = torch.empty((1,), dtype=torch.int32, device=dev)
    st = _stream(keys)
    with _on(keys):
        check(lib.f2c_relabel_mark(_ptr(keys), _DT[dt], n, _ptr(tab_keys), _ptr(tab_pos), cap, _ptr(first), _ptr(err), st))
        incl = torch.cumsum(first, 0, dtype=dt)
        rank = incl - first.to(dt)
        n_unique, overflow = torch.stack([incl[-1], err[0].to(dt)]).tolist()  # one host read for both
        if overflow == 2:
            raise RuntimeError("tensor_relabel: negative id (ids must be >= 0; strip a sampler's -1 padding first)")
        if overflow != 0:
            raise RuntimeError("tensor_relabel: hash table overflow")
        unique = torch.empty((n_unique,), dtype=dt, device=dev)
        relabelled = torch.empty((n,), dtype=dt, device=dev)
        check(lib.f2c_relabel_assign(_ptr(keys), _DT[dt], n, _ptr(tab_keys), _ptr(tab_pos), cap, _ptr(first), _ptr(rank),
                                     _ptr(unique), _ptr(relabelled), st))
    out, off = [], 0
    for t in tensors:
        out.append(relabelled[off:off + t.numel()].reshape(t.shape))
        off += t.numel()
    return unique, out


class _PendingBlock:
    __slots__ = ("sub_indptr", "keys", "unique", "relabelled", "n", "host", "event", "n_edges")


class BlockBuffers:
    """Device and pinned memory for ``sample_block_launch`` hops of up to ``max_seeds`` seeds, allocated once.  A loader
    that builds minibatches on a stream of its own keeps two sets of these instead of going through the caching
    allocator every hop (no per-hop allocation, no cross-stream bookkeeping; and on a device that has peers mapped a
    fresh device allocation costs milliseconds)."""

    def __init__(self, max_seeds, num_pick, dtype, device):
        self.max_seeds, self.num_pick, self.dtype = int(max_seeds), int(num_pick), dtype
        self.cap = self.max_seeds * (self.num_pick + 1)
        ws_bytes = lib.f2c_sample_block_workspace(self.max_seeds, self.num_pick, _DT[dtype])
        if ws_bytes <= 0:
            raise RuntimeError("sample_block: num_pick must be in [1, 64]")
        self.ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=device)
        self.sub_indptr = torch.empty((self.max_seeds + 1,), dtype=dtype, device=device)
        self.ids = torch.empty((3, self.cap), dtype=dtype, device=device)  # keys, unique, relabelled
        self.header = torch.empty((4,), dtype=torch.int64, device=device)
        self.host = torch.empty((4,), dtype=torch.int64, pin_memory=True)
        self.event = torch.cuda.Event()


def sample_block_launch(indptr, indices, seeds, num_pick, rng_seed=0, rng_offset=0, buffers=None):
    """First half of ``sample_block``: queues the hop on the current stream, starts the copy of its three counters to pinned
    host memory and returns without waiting.  ``sample_block_finish`` of the returned object gives the result; its
    ``event`` tells (``query()``) whether that would block.  A loader uses the pair to build the next minibatch on a
    side stream while the current one trains.  ``buffers``: a ``BlockBuffers`` to work in (the results are then views of
    it, valid until it is used again); default: fresh tensors."""
    _chk(indptr, "indptr", (torch.int32, torch.int64))
    _chk(indices, "indices", (indptr.dtype,))
    _chk(seeds, "seeds", (indptr.dtype,))
    n, dt, dev = seeds.numel(), indptr.dtype, indptr.device
    if n == 0:
        raise RuntimeError("sample_block: needs at least one seed")
    n_keys = n * (int(num_pick) + 1)
    pend = _PendingBlock()
    with _on(indptr):
        if buffers is None:
            ws_bytes = lib.f2c_sample_block_workspace(n, int(num_pick), _DT[dt])
            if ws_bytes <= 0:
                raise RuntimeError("sample_block: num_pick must be in [1, 64]")
            ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
            pend.sub_indptr = torch.empty((n + 1,), dtype=dt, device=dev)
            ids = torch.empty((3, n_keys), dtype=dt, device=dev)
            header = torch.empty((4,), dtype=torch.int64, device=dev)
            pend.host = torch.empty((4,), dtype=torch.int64, pin_memory=True)
            pend.event = torch.cuda.Event()
        else:
            if n > buffers.max_seeds or int(num_pick) != buffers.num_pick or dt != buffers.dtype:
                raise RuntimeError("sample_block: the buffers were sized for another hop")
            ws, ws_bytes, ids, header = buffers.ws, buffers.ws.numel(), buffers.ids, buffers.header
            pend.sub_indptr = buffers.sub_indptr[:n + 1]
            pend.host, pend.event = buffers.host, buffers.event
        pend.keys, pend.unique, pend.relabelled = ids[0, :n_keys], ids[1, :n_keys], ids[2, :n_keys]
        check(lib.f2c_sample_block(_ptr(indptr), _ptr(indices), _ptr(seeds), _DT[dt], n, int(num_pick),
                                   int(rng_seed) & 0xFFFFFFFFFFFFFFFF, int(rng_offset), _ptr(pend.sub_indptr), _ptr(pend.keys),
                                   _ptr(pend.unique), _ptr(pend.relabelled), _ptr(header), _ptr(ws), ws_bytes, _stream(indptr)))
        pend.host.copy_(header, non_blocking=True)
        pend.event.record(torch.cuda.current_stream(dev))
    pend.n = n
    return pend


def sample_block_finish(pend):
    """Second half of ``sample_block``: waits for the hop (host side only) and returns its tensors."""
    pend.event.synchronize()
    pend.n_edges, n_unique, err, _ = pend.host.tolist()  # n_edges: the hop's edge count, for callers that want it on the host
    if err == 2:
        raise RuntimeError("sample_block: negative id in the graph or the seeds")
    if err != 0:
        raise RuntimeError("sample_block: hash table overflow")
    return pend.sub_indptr, pend.keys[pend.n:], pend.unique[:n_unique], pend.relabelled[pend.n:]


def sample_block(indptr, indices, seeds, num_pick, rng_seed=0, rng_offset=0):
    """One hop of a block: ``csr_sampling`` followed by ``tensor_relabel([seeds, sub_indices])`` (the pair at
    examples/dataloader.py:174-177) as ONE library call and one host read.  Returns ``(sub_indptr, sub_indices, unique,
    local_indices)`` with the numbering of the separate operators; ``sub_indices`` / ``local_indices`` have
    ``len(seeds) * num_pick`` entries of which the first ``sub_indptr[-1]`` are the block's edges (the rest repeat
    ``seeds[0]`` and its new number, and no kernel reads them)."""
    return sample_block_finish(sample_block_launch(indptr, indices, seeds, num_pick, rng_seed, rng_offset))
