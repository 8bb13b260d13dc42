"""GPU parity: codecs (pack/unpack, SQ compress/decode, VQ decode, hybrid decode, dropout) through the
product module against the CPU oracle and the reference-kernel fixtures."""
import numpy as np
import pytest

from helpers import SQ_MAX_ULP, sq_table, ulp_diff

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("shape", [(0, 16), (1, 1), (9, 13), (9, 100), (64, 128), (1000, 128), (257, 7)])
def test_pack_unpack_bit_exact(capi, oracle, bits, shape):
    rng = np.random.default_rng(bits + shape[0] + shape[1])
    u = rng.integers(0, 2 ** bits, shape).astype(np.uint8)
    p = capi.packbits(dev(u), bits)
    assert np.array_equal(host(p), oracle.packbits(u, bits))
    assert np.array_equal(host(capi.unpackbits(p, bits, shape[1])), u)
    # unpack accepts the int8 view the reference stores packed tables in (examples/process_compress.py:109-111)
    assert np.array_equal(host(capi.unpackbits(p.view(torch.int8), bits, shape[1])), u)
    # values above the code range are masked like the reference does (src/packbits.cu:38)
    big = rng.integers(0, 256, shape).astype(np.uint8)
    assert np.array_equal(host(capi.packbits(dev(big), bits)), oracle.packbits(big, bits))


def test_pack_golden(capi, golden):
    for bits in (1, 2, 4):
        for dim in (100, 13, 128):
            u = golden[f"pack_in_b{bits}_d{dim}"]
            p = capi.packbits(dev(u), bits)
            assert np.array_equal(host(p), golden[f"pack_out_b{bits}_d{dim}"])
            assert np.array_equal(host(capi.unpackbits(p, bits, dim)), golden[f"unpack_out_b{bits}_d{dim}"])


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("D,cs", [(100, 100), (128, 128), (128, 32), (110, 60), (7, 7), (128, 1)])
def test_sq_compress_matches_oracle(capi, oracle, bits, D, cs):
    rng = np.random.default_rng(bits * 7 + D)
    x = rng.uniform(-1, 1, (301, D)).astype(np.float32)
    x[0, 0] = 0.0
    cb = oracle.sq_codebooks(x, cs)
    got = host(capi.sq_compress(dev(x), dev(cb), bits, cs))
    want = oracle.sq_compress(x, cb, bits, cs)
    bad = got != want
    if bad.any():
        # log2f differs by an ulp between libdevice and libm; only elements sitting on a quantisation
        # boundary may land in the neighbouring bucket.  The 0.5 % of elements clamped to fmin sit exactly
        # on the lowest boundary (log2f(fmin) - emin is 0 or -1 ulp), so up to ~1 % may differ.
        pre = oracle.sq_compress_prefloor(x, cb, bits, cs)
        assert np.all(np.abs(pre[bad] - np.round(pre[bad])) < max(1e-3, 2.0 ** (bits - 1) * 2e-6))
        assert np.all(np.abs(got[bad] - want[bad]) == 1)
        assert bad.mean() < 0.015


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("D,cs", [(100, 100), (128, 128), (128, 32), (110, 60), (7, 7), (128, 1), (260, 260)])
def test_sq_decompress_matches_oracle(capi, oracle, bits, D, cs):
    rng = np.random.default_rng(bits * 11 + D)
    _, cb, stored = sq_table(oracle, rng, 203, D, bits, cs)
    got = host(capi.sq_decompress(dev(stored), dev(cb), bits, cs, D))
    want = oracle.sq_decompress(stored, cb, bits, cs, D)
    if bits == 1:
        assert np.array_equal(got, want)
    else:
        assert ulp_diff(got, want).max() <= SQ_MAX_ULP
    if bits < 8:  # packed tables are stored as int8 in production; bytes are raw either way
        got8 = host(capi.sq_decompress(dev(stored).view(torch.int8), dev(cb), bits, cs, D))
        assert np.array_equal(got8, got)


def test_sq_decode_all_codes(capi, oracle):
    # every code value of every width <= 8 bits (and a sweep of 16-bit codes), two codebook rows
    cb = np.array([[0.01, 3.0, np.log2(0.01), np.log2(3.0) + 1e-5, 0.8],
                   [1e-5, 2e-5, np.log2(1e-5), np.log2(2e-5) + 1e-5, 0.15]], np.float32)
    for bits in (1, 2, 4, 8):
        per = 8 // bits if bits < 8 else 1
        codes = np.arange(256, dtype=np.uint8).reshape(256, 1).repeat(2, axis=1)  # column 0 -> row 0, column 1 -> row 1
        stored = codes if bits < 8 else codes.view(np.int8)
        got = host(capi.sq_decompress(dev(stored), dev(cb), bits, per, 2 * per))
        want = oracle.sq_decompress(stored, cb, bits, per, 2 * per)
        assert ulp_diff(got, want).max() <= SQ_MAX_ULP
        # uint8 8-bit codes are read as unsigned, like the reference's dtype switch does
        if bits == 8:
            gotu = host(capi.sq_decompress(dev(codes), dev(cb), 8, 1, 2))
            assert ulp_diff(gotu, oracle.sq_decompress(codes, cb, 8, 1, 2)).max() <= SQ_MAX_ULP
    c16 = np.arange(-32768, 32768, 1, dtype=np.int16).reshape(-1, 2)
    got = host(capi.sq_decompress(dev(c16), dev(cb), 16, 1, 2))
    assert ulp_diff(got, oracle.sq_decompress(c16, cb, 16, 1, 2)).max() <= SQ_MAX_ULP


def test_sq_golden_reference_kernels(capi, golden):
    """Against the reference's own CUDA kernels (fixtures made on a B200): codes and decoded values
    must carry the same bits."""
    for tag, cs, D in (("sq", 100, 100), ("sq2", 64, 128)):
        cb = dev(golden[f"{tag}_cb"])
        for bits in (1, 2, 4, 8, 16):
            if tag == "sq":
                codes = host(capi.sq_compress(dev(golden["sq_x"]), cb, bits, cs))
                assert np.array_equal(codes, golden[f"sq_codes_f_b{bits}"])
            stored = golden[f"{tag}_stored_b{bits}"]
            got = host(capi.sq_decompress(dev(stored), cb, bits, cs, D))
            assert np.array_equal(got.view(np.uint32), golden[f"{tag}_dec_b{bits}"].view(np.uint32)), (tag, bits)


@pytest.mark.parametrize("code_dtype", [np.uint8, np.int16, np.int8])
@pytest.mark.parametrize("n_cb,K,cs,D", [(2, 256, 60, 110), (16, 256, 8, 128), (4, 256, 32, 128), (4, 256, 64, 256),
                                         (3, 100, 5, 13), (1, 7, 128, 128)])
def test_vq_decompress_bit_exact(capi, oracle, code_dtype, n_cb, K, cs, D):
    rng = np.random.default_rng(n_cb * K + cs)
    kmax = min(K, 128) if code_dtype == np.int8 else K
    cbs = rng.standard_normal((n_cb, K, cs)).astype(np.float32)
    codes = rng.integers(0, kmax, (333, n_cb)).astype(code_dtype)
    got = host(capi.vq_decompress(dev(codes), dev(cbs), D))
    assert np.array_equal(got, oracle.vq_decompress(codes, cbs, D))
    got16 = host(capi.vq_decompress(dev(codes), dev(cbs.astype(np.float16)), D))
    assert np.array_equal(got16, oracle.vq_decompress(codes, cbs.astype(np.float16), D))


def test_vq_golden(capi, golden):
    cbs, codes = dev(golden["vq_cbs"]), dev(golden["vq_codes_u8"])
    assert np.array_equal(host(capi.vq_decompress(codes, cbs, 110)), golden["vq_dec_u8"])
    assert np.array_equal(host(capi.vq_decompress(codes, cbs.half(), 110)), golden["vq_dec_u8_f16cb"])
    assert np.array_equal(host(capi.vq_decompress(codes.to(torch.int16), cbs, 110)), golden["vq_dec_i16"])


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("D,cs", [(128, 128), (128, 32), (128, 8), (64, 16), (256, 256), (512, 64)])
def test_sq_decompress_streaming_table_kernel(capi, oracle, bits, D, cs):
    """Tables of >= 4096 rows take the persistent table-decode kernel; its rows must have the bits of the
    element-wise kernel (which small calls use) and stay within the exp2f tolerance of the oracle."""
    rng = np.random.default_rng(bits * 100 + D + cs)
    rows = 4096 + 777
    _, cb, stored = sq_table(oracle, rng, rows, D, bits, cs)
    variants = [stored]
    if bits == 8:
        variants.append(stored.view(np.uint8))
    for st in variants:
        big = capi.sq_decompress(dev(st), dev(cb), bits, cs, D)
        for lo in (0, 2000, rows - 300):
            small = capi.sq_decompress(dev(st[lo:lo + 300]), dev(cb), bits, cs, D)
            assert torch.equal(big[lo:lo + 300], small), (lo, st.dtype)
    want = oracle.sq_decompress(stored, cb, bits, cs, D)
    assert ulp_diff(host(capi.sq_decompress(dev(stored), dev(cb), bits, cs, D)), want).max() <= SQ_MAX_ULP


@pytest.mark.parametrize("n_cb,K,cs,D", [(16, 256, 8, 128), (4, 256, 32, 128), (4, 256, 64, 256), (8, 100, 16, 128),
                                         (32, 256, 4, 128), (2, 256, 128, 256), (4, 256, 32, 100)])
def test_vq_decompress_streaming_kernel(capi, oracle, n_cb, K, cs, D):
    """>= 4096 rows with uint8 codes take the shared-memory streaming kernel (where the shape allows): same rows as the
    gather kernel used by small calls and as index_select (tests/test_vq.py:51,86)."""
    rng = np.random.default_rng(n_cb + K + cs)
    rows = 4096 + 1234
    cbs = rng.standard_normal((n_cb, K, cs)).astype(np.float32)
    codes = rng.integers(0, 256, (rows, n_cb)).astype(np.uint8)  # codes >= K are clamped by both kernels
    big = capi.vq_decompress(dev(codes), dev(cbs), D)
    for lo in (0, 3000, rows - 500):
        assert torch.equal(big[lo:lo + 500], capi.vq_decompress(dev(codes[lo:lo + 500]), dev(cbs), D)), lo
    assert np.array_equal(host(big), oracle.vq_decompress(np.minimum(codes, K - 1).astype(np.uint8), cbs, D))


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("D,sq_cs,n_cb,cs", [(128, 128, 4, 32), (128, 32, 16, 8), (256, 256, 4, 64), (110, 110, 2, 60)])
def test_fusion_decompress_is_concatenation(capi, oracle, bits, D, sq_cs, n_cb, cs):
    # tests/test_fusion_decompress.py:32-43 of the reference
    rng = np.random.default_rng(bits + D)
    _, cb, sq = sq_table(oracle, rng, 37, D, bits, sq_cs)
    cbs = rng.standard_normal((n_cb, 256, cs)).astype(np.float32)
    codes = rng.integers(0, 256, (91, n_cb)).astype(np.uint8)
    got = capi.fusion_decompress(dev(sq), dev(cb), bits, sq_cs, dev(codes), dev(cbs), D)
    parts = torch.cat([capi.sq_decompress(dev(sq), dev(cb), bits, sq_cs, D), capi.vq_decompress(dev(codes), dev(cbs), D)])
    assert torch.equal(got, parts)
    want = oracle.fusion_decompress(sq, cb, bits, sq_cs, codes, cbs, D)
    assert ulp_diff(host(got), want).max() <= SQ_MAX_ULP


@pytest.mark.parametrize("n", [0, 1, 3, 4, 1001, 1 << 16])
def test_dropout_matches_oracle_mask(capi, oracle, n):
    x = np.arange(1, n + 1, dtype=np.float32)
    for p, scale in ((0.5, False), (0.1, False), (0.9, True), (0.0, False), (1.0, False)):
        t = dev(x.copy())
        r = capi.dropout_inplace(t, p, True, seed=1234, offset=3, scale=scale)
        assert r.data_ptr() == t.data_ptr()  # returns its argument (src/fusion_dropout.cu:28)
        assert np.array_equal(host(t), oracle.dropout(x, p, True, 1234, 3, scale))
    t = dev(x.copy())
    capi.dropout_inplace(t, 0.5, False, seed=1)
    assert np.array_equal(host(t), x)  # identity when not training (src/fusion_dropout.cu:11)


def test_dropout_reference_statistics(capi):
    # the reference's mask is time-seeded, so parity is statistical: keep rate 1-p within 5 sigma,
    # survivors bit-identical to the input, no rescale
    n = 1 << 20
    x = torch.randn(n, device="cuda")
    for p in (0.25, 0.5):
        y = capi.dropout_inplace(x.clone(), p, True)
        keep = y != 0
        assert torch.equal(y[keep], x[keep])
        assert abs(float(keep.float().mean()) - (1 - p)) < 5 * (p * (1 - p) / n) ** 0.5
    # unaligned view takes the scalar path and still matches the aligned mask
    base = torch.ones(n + 1, device="cuda")
    a = capi.dropout_inplace(base[1:].clone(), 0.5, True, seed=9)
    b = base.clone()
    capi.dropout_inplace(b[1:], 0.5, True, seed=9)
    assert torch.equal(a, b[1:])


def test_errors_raise_not_abort(capi):
    z = torch.zeros(4, 16, dtype=torch.uint8, device="cuda")
    cb = torch.zeros(1, 5, device="cuda")
    with pytest.raises(RuntimeError):
        capi.packbits(z, 3)
    with pytest.raises(RuntimeError):
        capi.sq_decompress(z, cb, 4, 128, 128)  # 16 bytes cannot hold 128 4-bit elements
    with pytest.raises(RuntimeError):
        capi.sq_decompress(z, cb, 5, 32, 32)
    with pytest.raises(RuntimeError):
        capi.sq_decompress(z.t(), cb, 4, 8, 8)  # non-contiguous
    with pytest.raises(RuntimeError):
        capi.vq_decompress(z, torch.zeros(2, 256, 8, device="cuda"), 16)  # 16 code columns vs 2 codebooks
