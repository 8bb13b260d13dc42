"""Generate tests/golden/ref_b200.npz: outputs of the REFERENCE's own CUDA kernels on seeded inputs.

Runs on a machine with a GPU and the extension built by oracle/build_ref.py from the unmodified
reference sources (src/sq_quantization.cu, vq_quantization.cu, packbits.cu, fusion_spmm.cu of
gpzlx1/F2CGT).  Every array a test needs - inputs included - is stored, so the fixtures do not depend
on any random generator being reproducible.  The fixtures pin oracle/f2c_oracle.c (CPU tests) and are
compared with this library's kernels (GPU tests).

    python tests/golden/make_golden.py --out tests/golden/ref_b200.npz
"""
import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import build_ref  # noqa: E402
from oracle import oracle as O  # noqa: E402  (only for the codebook recipe, which is host-side numpy)


def store(cpu_or_cuda_tensor):
    return cpu_or_cuda_tensor.detach().cpu().numpy()


def main(out_path):
    ref = build_ref.load()
    dev = "cuda"
    rng = np.random.default_rng(20241125)
    g = {}

    # ---- random CSC block with empty rows and repeated sources (shared by the aggregation cases)
    n_dst, n_src = 40, 64
    deg = rng.integers(0, 9, n_dst)
    deg[3] = 0
    deg[17] = 0
    deg[5] = 33  # one row longer than a warp
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n_src, indptr[-1]).astype(np.int64)
    g["csc_indptr"], g["csc_indices"] = indptr, indices
    t_indptr, t_indices = torch.from_numpy(indptr).to(dev), torch.from_numpy(indices).to(dev)
    toy_indptr = torch.tensor([0, 1, 3, 6], dtype=torch.int64, device=dev)  # tests/test_fusion_decompress_spmm.py:20-21
    toy_indices = torch.tensor([0, 1, 1, 2, 2, 0], dtype=torch.int64, device=dev)

    # ---- pack / unpack (src/packbits.cu), ragged widths
    for bits in (1, 2, 4):
        for dim in (100, 13, 128):
            u = rng.integers(0, 2 ** bits, (9, dim)).astype(np.uint8)
            p = ref.packbits(torch.from_numpy(u).to(dev), bits)
            g[f"pack_in_b{bits}_d{dim}"] = u
            g[f"pack_out_b{bits}_d{dim}"] = store(p)
            g[f"unpack_out_b{bits}_d{dim}"] = store(ref.unpackbits(p, bits, dim))

    # ---- SQ codec (src/sq_quantization.cu): one codebook row, D=100 (ragged for every packed width)
    x = rng.uniform(-1, 1, (n_src, 100)).astype(np.float32)
    x[0, :4] = [0.0, -0.0, 1e-9, -3.0]  # zero counts as negative; clamps at both ends
    cb = O.sq_codebooks(x, 100)
    g["sq_x"], g["sq_cb"] = x, cb
    tx, tcb = torch.from_numpy(x).to(dev), torch.from_numpy(cb).to(dev)
    for bits in (1, 2, 4, 8, 16):
        codes_f = ref.sq_compress(tx, tcb, bits, 100)
        g[f"sq_codes_f_b{bits}"] = store(codes_f)
        if bits < 8:
            stored = ref.packbits(codes_f.to(torch.uint8), bits)
        elif bits == 8:
            stored = codes_f.to(torch.int8)
        else:
            stored = codes_f.to(torch.int16)
        g[f"sq_stored_b{bits}"] = store(stored)
        dec = ref.sq_decompress(stored, tcb, bits, 100, 100)
        g[f"sq_dec_b{bits}"] = store(dec)
        unfused = ref.spmm_csr(dec, t_indptr, t_indices)
        fused = ref.sq_decompress_spmm_csr(stored, tcb, t_indptr, t_indices, bits, 100, 100)
        assert torch.equal(unfused, fused), f"reference fused != unfused for {bits} bits"
        g[f"sq_spmm_b{bits}"] = store(fused)
        g[f"sq_spmm_toy_b{bits}"] = store(ref.sq_decompress_spmm_csr(stored, tcb, toy_indptr, toy_indices, bits, 100, 100))

    # ---- SQ with two codebook rows, column_slice 64, D=128 (vector-friendly shape)
    x2 = np.concatenate([rng.uniform(-1, 1, (n_src, 64)), rng.uniform(-1, 1, (n_src, 64)) * 4 + 10], axis=1).astype(np.float32)
    cb2 = O.sq_codebooks(x2, 64)
    g["sq2_x"], g["sq2_cb"] = x2, cb2
    tx2, tcb2 = torch.from_numpy(x2).to(dev), torch.from_numpy(cb2).to(dev)
    for bits in (1, 2, 4, 8, 16):
        codes_f = ref.sq_compress(tx2, tcb2, bits, 64)
        if bits < 8:
            stored = ref.packbits(codes_f.to(torch.uint8), bits)
        elif bits == 8:
            stored = codes_f.to(torch.int8)
        else:
            stored = codes_f.to(torch.int16)
        g[f"sq2_stored_b{bits}"] = store(stored)
        g[f"sq2_dec_b{bits}"] = store(ref.sq_decompress(stored, tcb2, bits, 64, 128))
        g[f"sq2_spmm_b{bits}"] = store(ref.sq_decompress_spmm_csr(stored, tcb2, t_indptr, t_indices, bits, 64, 128))

    # ---- VQ (src/vq_quantization.cu): two codebooks of width 60, feat_dim 110 (padded second slice,
    #      as in tests/test_vq.py:70-81), uint8 and int16 codes, fp32 and fp16 codebooks
    cbs = rng.standard_normal((2, 256, 60)).astype(np.float32)
    cbs[1, :, 50:] = 0
    codes_u8 = rng.integers(0, 256, (n_src, 2)).astype(np.uint8)
    g["vq_cbs"], g["vq_codes_u8"] = cbs, codes_u8
    tcbs, tcodes = torch.from_numpy(cbs).to(dev), torch.from_numpy(codes_u8).to(dev)
    g["vq_dec_u8"] = store(ref.vq_decompress(tcodes, tcbs, 110))
    g["vq_dec_u8_f16cb"] = store(ref.vq_decompress(tcodes, tcbs.half(), 110))
    g["vq_dec_i16"] = store(ref.vq_decompress(tcodes.to(torch.int16), tcbs, 110))
    vq_dec = ref.vq_decompress(tcodes, tcbs, 110)
    unfused = ref.spmm_csr(vq_dec, t_indptr, t_indices)
    fused = ref.vq_decompress_spmm_csr(tcodes, tcbs, t_indptr, t_indices, 110)
    assert torch.equal(unfused, fused), "reference fused VQ != unfused"
    g["vq_spmm_u8"] = store(fused)
    # BASELINE-shaped codebooks: 16 x 256 x 8, D=128
    cbs16 = rng.standard_normal((16, 256, 8)).astype(np.float32)
    codes16 = rng.integers(0, 256, (n_src, 16)).astype(np.uint8)
    g["vq16_cbs"], g["vq16_codes"] = cbs16, codes16
    g["vq16_spmm"] = store(ref.vq_decompress_spmm_csr(torch.from_numpy(codes16).to(dev), torch.from_numpy(cbs16).to(dev),
                                                      t_indptr, t_indices, 128))

    # ---- plain mean aggregation (src/fusion_spmm.cu:13-70), fp32 / fp64 / fp16, int64 and int32 indices
    feat = rng.standard_normal((n_src, 100)).astype(np.float32)
    g["spmm_feat"] = feat
    tf = torch.from_numpy(feat).to(dev)
    g["spmm_f32"] = store(ref.spmm_csr(tf, t_indptr, t_indices))
    g["spmm_f32_i32"] = store(ref.spmm_csr(tf, t_indptr.int(), t_indices.int()))
    for name, t in (("spmm_f64", tf.double()), ("spmm_f16", tf.half())):
        try:  # dtypes no caller of the reference uses; keep going if its kernel rejects one
            g[name] = store(ref.spmm_csr(t, t_indptr, t_indices))
        except Exception as e:  # noqa: BLE001
            print(f"reference spmm_csr failed for {name}: {e}")

    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    np.savez_compressed(out_path, **g)
    print(f"wrote {out_path}: {len(g)} arrays, {os.path.getsize(out_path)} bytes")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "ref_b200.npz"))
    main(ap.parse_args().out)
