"""CPU: the oracle against the properties the reference's own tests hold (no GPU, no fixtures)."""
import numpy as np
import pytest

from helpers import random_csc, sq_table


@pytest.mark.parametrize("bits", [1, 2, 4])
@pytest.mark.parametrize("dim", [1, 7, 8, 100, 128])
def test_pack_unpack_identity(oracle, bits, dim):
    rng = np.random.default_rng(bits * 100 + dim)
    u = rng.integers(0, 2 ** bits, (11, dim)).astype(np.uint8)
    p = oracle.packbits(u, bits)
    per = 8 // bits
    assert p.shape == (11, (dim + per - 1) // per)
    assert np.array_equal(oracle.unpackbits(p, bits, dim), u)


def test_pack_bit_order_exhaustive(oracle):
    # element i of a byte sits at bit offset bits*i (src/packbits.cu:37-38): check all 256 bytes
    for bits in (1, 2, 4):
        per = 8 // bits
        allbytes = np.arange(256, dtype=np.uint8).reshape(256, 1)
        u = oracle.unpackbits(allbytes, bits, per)
        expect = np.stack([(np.arange(256) >> (bits * i)) & (2 ** bits - 1) for i in range(per)], axis=1)
        assert np.array_equal(u, expect.astype(np.uint8))
        assert np.array_equal(oracle.packbits(u, bits), allbytes)


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
def test_sq_code_ranges_and_roundtrip(oracle, bits):
    rng = np.random.default_rng(bits)
    x = rng.uniform(-1, 1, (500, 100)).astype(np.float32)
    cb = oracle.sq_codebooks(x, 100)
    c = oracle.sq_compress(x, cb, bits, 100)
    assert np.array_equal(c, np.round(c))
    if bits < 8:
        assert c.min() >= 0 and c.max() <= 2 ** bits - 1
    else:
        assert c.min() >= -2 ** (bits - 1) and c.max() <= 2 ** (bits - 1) - 1
    y = oracle.sq_decompress(oracle.sq_codes_to_storage(c, bits), cb, bits, 100, 100)
    # sign is preserved (zero counts as negative) and the error shrinks with the width
    assert np.array_equal(np.sign(y), np.where(x <= 0, -1, 1))
    if bits >= 8:
        inside = (np.abs(x) > cb[0, 0]) & (np.abs(x) < cb[0, 1])
        rel = np.abs(y - x)[inside] / np.abs(x)[inside]
        assert rel.max() < (0.06 if bits == 8 else 3e-4)
    if bits == 1:
        assert np.array_equal(np.abs(y), np.full_like(y, cb[0, 4]))


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_fused_sq_equals_unfused(oracle, bits, idx_dtype):
    # tests/test_fusion_decompress_spmm.py:93-120 of the reference: torch.equal(fused, unfused)
    rng = np.random.default_rng(10 + bits)
    _, cb, stored = sq_table(oracle, rng, 50, 96, bits, 32)
    indptr, indices = random_csc(rng, 30, 50, dtype=idx_dtype)
    dec = oracle.sq_decompress(stored, cb, bits, 32, 96)
    for reduce in ("mean", "sum"):
        a = oracle.spmm_csr(dec, indptr, indices, reduce)
        b = oracle.sq_decompress_spmm_csr(stored, cb, indptr, indices, bits, 32, 96, reduce)
        assert np.array_equal(a, b)
    # empty destination rows give zeros (deg==0 -> divide by 1, src/fusion_spmm.cu:177)
    deg = np.diff(indptr)
    assert np.all(b[deg == 0] == 0)


def test_fused_vq_equals_unfused_and_index_select(oracle):
    rng = np.random.default_rng(3)
    cbs = rng.standard_normal((2, 256, 60)).astype(np.float32)
    cbs[1, :, 50:] = 0
    codes = rng.integers(0, 256, (64, 2)).astype(np.uint8)
    dec = oracle.vq_decompress(codes, cbs, 110)
    # tests/test_vq.py:63-65,86: decode == cat(index_select per codebook)
    expect = np.concatenate([cbs[0][codes[:, 0]], cbs[1][codes[:, 1]][:, :50]], axis=1)
    assert np.array_equal(dec, expect)
    indptr, indices = random_csc(rng, 33, 64)
    assert np.array_equal(oracle.spmm_csr(dec, indptr, indices), oracle.vq_decompress_spmm_csr(codes, cbs, indptr, indices, 110))
    # int16 codes and fp16 codebooks
    assert np.array_equal(oracle.vq_decompress(codes.astype(np.int16), cbs, 110), dec)
    assert np.array_equal(oracle.vq_decompress(codes, cbs.astype(np.float16), 110), expect.astype(np.float16).astype(np.float32))


def test_hybrid_decode_is_concatenation_and_spmm_is_composition(oracle):
    # tests/test_fusion_decompress.py:32-43 of the reference
    rng = np.random.default_rng(4)
    n, D = 80, 128
    _, cb, sq = sq_table(oracle, rng, 20, D, 4, 128)
    cbs = rng.standard_normal((4, 256, 32)).astype(np.float32)
    codes = rng.integers(0, 256, (n, 4)).astype(np.uint8)
    out = oracle.fusion_decompress(sq, cb, 4, 128, codes[20:], cbs, D)
    assert np.array_equal(out, np.concatenate([oracle.sq_decompress(sq, cb, 4, 128, D), oracle.vq_decompress(codes[20:], cbs, D)]))
    # aggregation: decode every source row with its own codec, then the plain mean
    slot = np.full(n, -1, np.int32)
    hot = rng.choice(n, 20, replace=False)
    slot[hot] = np.arange(20, dtype=np.int32)
    full = oracle.vq_decompress(codes, cbs, D)
    full[hot] = oracle.sq_decompress(sq, cb, 4, 128, D)
    indptr, indices = random_csc(rng, 25, n)
    got = oracle.two_level_decompress_spmm_csr(sq, cb, 4, 128, codes, cbs, slot, indptr, indices, D)
    assert np.array_equal(got, oracle.spmm_csr(full, indptr, indices))


def test_spmm_dtypes_and_sum(oracle):
    rng = np.random.default_rng(5)
    feat = rng.standard_normal((30, 20)).astype(np.float32)
    indptr, indices = random_csc(rng, 12, 30)
    m = oracle.spmm_csr(feat, indptr, indices)
    s = oracle.spmm_csr(feat, indptr, indices, "sum")
    deg = np.maximum(np.diff(indptr), 1).astype(np.float32)[:, None]
    assert np.array_equal(m, s / deg)
    ref64 = np.stack([feat[indices[indptr[d]:indptr[d + 1]]].astype(np.float64).sum(0) for d in range(12)]) / deg
    assert np.allclose(m, ref64, rtol=1e-6, atol=1e-6)
    assert np.allclose(oracle.spmm_csr(feat.astype(np.float64), indptr, indices), ref64, rtol=1e-12)
    h = oracle.spmm_csr(feat.astype(np.float16), indptr, indices)
    assert h.dtype == np.float16 and np.allclose(h.astype(np.float32), ref64, rtol=2e-2, atol=2e-2)


def test_dropout_statistics_and_determinism(oracle):
    x = np.arange(1, 200001, dtype=np.float32)
    for p in (0.0, 0.1, 0.5, 0.9):
        y = oracle.dropout(x, p, seed=7)
        keep = y != 0
        assert np.array_equal(y[keep], x[keep])  # survivors untouched, no rescale (src/fusion_dropout.cu:16)
        n = x.size
        assert abs(keep.mean() - (1 - p)) < 5 * np.sqrt(p * (1 - p) / n) + 1e-12
        assert np.array_equal(y, oracle.dropout(x, p, seed=7))
        if 0 < p < 1:
            assert not np.array_equal(y, oracle.dropout(x, p, seed=8))
            assert not np.array_equal(y, oracle.dropout(x, p, seed=7, offset=1))
    assert np.array_equal(oracle.dropout(x, 0.5, training=False), x)
    assert np.all(oracle.dropout(x, 1.0, seed=1) == 0)
    ys = oracle.dropout(x, 0.5, seed=7, scale=True)
    assert np.array_equal(ys[ys != 0], (x * 2)[ys != 0])


def test_kmeans_oracle_matches_numpy(oracle):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((300, 8)).astype(np.float32)
    c = rng.standard_normal((17, 8)).astype(np.float32)
    d2 = ((x[:, None, :].astype(np.float64) - c[None].astype(np.float64)) ** 2).sum(-1)
    assert np.allclose(oracle.pairwise_distance(x, c, "euclidean"), d2, rtol=1e-6)
    cos = 1 - (x.astype(np.float64) @ c.T.astype(np.float64)) / (np.linalg.norm(x, axis=1)[:, None] * np.linalg.norm(c, axis=1)[None])
    assert np.allclose(oracle.pairwise_distance(x, c, "cosine"), cos, rtol=1e-5, atol=1e-6)
    assert np.array_equal(oracle.kmeans_assign(x, c, "l2"), d2.argmin(1))
    assert np.array_equal(oracle.kmeans_assign(x, c, "cosine"), cos.argmin(1))
    # first minimum wins on exact ties
    c2 = np.concatenate([c, c[:3]])
    assert oracle.kmeans_assign(x, c2, "l2").max() < 17


def test_tensor_relabel_contract(oracle):
    O = oracle
    """Seeds keep their positions, ids are numbered by first occurrence, unique[relabelled] gives the ids back
    (what examples/dataloader.py:176-182 and examples/conv.py:48-49 rely on)."""
    rng = np.random.default_rng(4)
    seeds = rng.choice(1000, 50, replace=False)
    ids = rng.integers(0, 1000, 5000)
    uniq, (rs, ri) = O.tensor_relabel([seeds, ids])
    assert np.array_equal(rs, np.arange(50)) and np.array_equal(uniq[:50], seeds)
    assert np.array_equal(uniq[ri], ids) and len(np.unique(uniq)) == len(uniq)
    first_seen = [np.flatnonzero(np.concatenate([seeds, ids]) == u)[0] for u in uniq]
    assert first_seen == sorted(first_seen)
    u0, (e,) = O.tensor_relabel([np.zeros(0, np.int64)])
    assert u0.size == 0 and e.size == 0
