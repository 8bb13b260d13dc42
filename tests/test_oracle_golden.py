"""CPU: pin the oracle (oracle/f2c_oracle.c) to outputs of the REFERENCE's own CUDA kernels.

tests/golden/ref_b200.npz was produced on a B200 by tests/golden/make_golden.py from the extension
oracle/build_ref.py builds out of the unmodified reference sources.  Integer / gather / summation
order results must agree bit for bit; values that pass through exp2f / log2f may differ in the last
bits between the GPU's libdevice and the host's libm and are held to 2 ulp (codes: to the
neighbouring bucket, only on a quantisation boundary)."""
import numpy as np

from helpers import SQ_MAX_ULP, ulp_diff


def test_pack_unpack(oracle, golden):
    for bits in (1, 2, 4):
        for dim in (100, 13, 128):
            u = golden[f"pack_in_b{bits}_d{dim}"]
            p = oracle.packbits(u, bits)
            assert np.array_equal(p, golden[f"pack_out_b{bits}_d{dim}"])
            assert np.array_equal(oracle.unpackbits(p, bits, dim), golden[f"unpack_out_b{bits}_d{dim}"])


def test_sq_compress_codes(oracle, golden):
    x, cb = golden["sq_x"], golden["sq_cb"]
    for bits in (1, 2, 4, 8, 16):
        got, want = oracle.sq_compress(x, cb, bits, 100), golden[f"sq_codes_f_b{bits}"]
        bad = got != want
        if bad.any():
            pre = oracle.sq_compress_prefloor(x, cb, bits, 100)
            assert np.all(np.abs(pre[bad] - np.round(pre[bad])) < max(1e-3, 2.0 ** (bits - 1) * 2e-6))
            assert np.all(np.abs(got[bad] - want[bad]) == 1) and bad.mean() < 0.015
        # the storage conversion the callers apply is exact
        if not bad.any():
            assert np.array_equal(oracle.sq_codes_to_storage(got, bits), golden[f"sq_stored_b{bits}"])


def test_sq_decode(oracle, golden):
    for tag, cs, D in (("sq", 100, 100), ("sq2", 64, 128)):
        for bits in (1, 2, 4, 8, 16):
            got = oracle.sq_decompress(golden[f"{tag}_stored_b{bits}"], golden[f"{tag}_cb"], bits, cs, D)
            want = golden[f"{tag}_dec_b{bits}"]
            if bits == 1:
                assert np.array_equal(got, want)  # +-mean involves no transcendental
            else:
                assert ulp_diff(got, want).max() <= SQ_MAX_ULP, (tag, bits)


def test_sq_fused_aggregation(oracle, golden):
    ip, ix = golden["csc_indptr"], golden["csc_indices"]
    toy_ip, toy_ix = np.array([0, 1, 3, 6]), np.array([0, 1, 1, 2, 2, 0])
    for bits in (1, 2, 4, 8, 16):
        for key, args in ((f"sq_spmm_b{bits}", ("sq", ip, ix, 100, 100)), (f"sq_spmm_toy_b{bits}", ("sq", toy_ip, toy_ix, 100, 100)),
                          (f"sq2_spmm_b{bits}", ("sq2", ip, ix, 64, 128))):
            tag, a, b, cs, D = args
            got = oracle.sq_decompress_spmm_csr(golden[f"{tag}_stored_b{bits}"], golden[f"{tag}_cb"], a, b, bits, cs, D)
            want = golden[key]
            if bits == 1:
                assert np.array_equal(got, want), key  # same values, same order, same division
            else:
                # decoded values differ by <= 2 ulp, so do their means (relative to the summands)
                dec = np.abs(oracle.sq_decompress(golden[f"{tag}_stored_b{bits}"], golden[f"{tag}_cb"], bits, cs, D))
                mag = oracle.spmm_csr(dec, a, b)
                assert np.all(np.abs(got - want) <= 4e-7 * mag + 1e-30), key
        # feeding the reference's decoded values through the oracle's aggregation is bit exact:
        # this pins the summation order and the division independently of exp2f
        agg = oracle.spmm_csr(golden[f"sq_dec_b{bits}"], ip, ix)
        assert np.array_equal(agg.view(np.uint32), golden[f"sq_spmm_b{bits}"].view(np.uint32)), bits


def test_vq(oracle, golden):
    cbs, codes = golden["vq_cbs"], golden["vq_codes_u8"]
    assert np.array_equal(oracle.vq_decompress(codes, cbs, 110), golden["vq_dec_u8"])
    assert np.array_equal(oracle.vq_decompress(codes, cbs.astype(np.float16), 110), golden["vq_dec_u8_f16cb"])
    assert np.array_equal(oracle.vq_decompress(codes.astype(np.int16), cbs, 110), golden["vq_dec_i16"])
    ip, ix = golden["csc_indptr"], golden["csc_indices"]
    assert np.array_equal(oracle.vq_decompress_spmm_csr(codes, cbs, ip, ix, 110), golden["vq_spmm_u8"])
    assert np.array_equal(oracle.vq_decompress_spmm_csr(golden["vq16_codes"], golden["vq16_cbs"], ip, ix, 128), golden["vq16_spmm"])


def test_plain_aggregation(oracle, golden):
    feat, ip, ix = golden["spmm_feat"], golden["csc_indptr"], golden["csc_indices"]
    assert np.array_equal(oracle.spmm_csr(feat, ip, ix), golden["spmm_f32"])
    assert np.array_equal(oracle.spmm_csr(feat, ip.astype(np.int32), ix.astype(np.int32)), golden["spmm_f32_i32"])
    if "spmm_f64" in golden:
        assert np.array_equal(oracle.spmm_csr(feat.astype(np.float64), ip, ix), golden["spmm_f64"])
    if "spmm_f16" in golden:
        assert np.array_equal(oracle.spmm_csr(feat.astype(np.float16), ip, ix), golden["spmm_f16"])
