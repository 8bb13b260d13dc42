"""GPU parity: the aggregation kernels (plain, fused SQ, fused VQ, two-level) against the oracle, the
reference-kernel fixtures and the reference's own property fused == decode-then-aggregate."""
import numpy as np
import pytest

from helpers import AGG_ATOL, AGG_RTOL, SQ_MAX_ULP, random_csc, sq_table, ulp_diff

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def close_to_oracle(got, want64, magnitude=None):
    """The tolerance named for aggregated outputs (1e-5 relative / 1e-6 absolute, fp32, any summation
    order).  `magnitude` = the same aggregation over |decoded values|: where neighbours cancel, no fp32
    summation (the reference's included) can be relative to the tiny result, only to its summands."""
    ref = np.abs(want64) if magnitude is None else np.maximum(np.abs(want64), magnitude)
    return bool(np.all(np.abs(got - want64) <= AGG_ATOL + AGG_RTOL * ref))


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("idx", [np.int64, np.int32])
@pytest.mark.parametrize("D", [1, 100, 128, 260])
def test_spmm_csr_bit_exact(capi, oracle, dtype, idx, D):
    rng = np.random.default_rng(D)
    feat = rng.standard_normal((70, D)).astype(dtype)
    indptr, indices = random_csc(rng, 45, 70, max_deg=40, dtype=idx)
    for reduce in ("mean", "sum"):
        got = host(capi.spmm_csr(dev(feat), dev(indptr), dev(indices), reduce=reduce))
        want = oracle.spmm_csr(feat, indptr, indices, reduce)
        assert got.dtype == dtype and np.array_equal(got, want)


def test_spmm_golden_and_toy(capi, golden):
    feat, indptr, indices = dev(golden["spmm_feat"]), dev(golden["csc_indptr"]), dev(golden["csc_indices"])
    assert np.array_equal(host(capi.spmm_csr(feat, indptr, indices)), golden["spmm_f32"])
    assert np.array_equal(host(capi.spmm_csr(feat, indptr.int(), indices.int())), golden["spmm_f32_i32"])
    if "spmm_f64" in golden:
        assert np.array_equal(host(capi.spmm_csr(feat.double(), indptr, indices)), golden["spmm_f64"])
    if "spmm_f16" in golden:
        assert np.array_equal(host(capi.spmm_csr(feat.half(), indptr, indices)), golden["spmm_f16"])


SQ_SHAPES = [  # (D, column_slice): vector paths, ragged widths, several codebook rows, per-column rows
    (128, 128), (128, 32), (128, 16), (100, 100), (110, 56), (256, 256), (256, 64), (64, 64), (32, 8), (128, 8), (520, 520)]


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("D,cs", SQ_SHAPES)
def test_fused_sq_equals_unfused_and_oracle(capi, oracle, bits, D, cs):
    rng = np.random.default_rng(bits * 1000 + D + cs)
    n_src, n_dst = 300, 157
    _, cb, stored = sq_table(oracle, rng, n_src, D, bits, cs)
    for idx in (np.int64, np.int32):
        indptr, indices = random_csc(rng, n_dst, n_src, max_deg=20, dtype=idx)
        t_codes, t_cb, t_ip, t_ix = dev(stored), dev(cb), dev(indptr), dev(indices)
        for reduce in ("mean", "sum"):
            fused = capi.sq_decompress_spmm_csr(t_codes, t_cb, t_ip, t_ix, bits, cs, D, reduce=reduce)
            unfused = capi.spmm_csr(capi.sq_decompress(t_codes, t_cb, bits, cs, D), t_ip, t_ix, reduce=reduce)
            # the reference's own test: torch.equal (tests/test_fusion_decompress_spmm.py:120)
            assert torch.equal(fused, unfused), (bits, D, cs, idx, reduce)
            want = oracle.sq_decompress_spmm_csr(stored, cb, indptr, indices, bits, cs, D, reduce, acc64=True)
            mag = oracle.spmm_csr(np.abs(oracle.sq_decompress(stored, cb, bits, cs, D)), indptr, indices, reduce)
            assert close_to_oracle(host(fused), want, mag)
    # production tables are int8 views of packed bytes
    if bits < 8:
        again = capi.sq_decompress_spmm_csr(t_codes.view(torch.int8), t_cb, t_ip, t_ix, bits, cs, D, reduce="sum")
        assert torch.equal(again, fused)


def _served(fn):
    """Result of a call that pins a kernel family, or None when that family does not take the shape."""
    try:
        return fn()
    except RuntimeError as e:
        if "not served" in str(e):
            return None
        raise


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("D,cs", [(128, 64), (128, 128), (256, 256), (96, 96), (64, 16), (32, 8)])
def test_fused_sq_every_kernel_family_is_bit_identical(capi, oracle, bits, D, cs):
    """Streamed, register-prefetch (table and exp2f decode) and general kernels: same bits, any degree mix
    (empty rows, rows longer than the streamed kernel's ring groups, ragged last group)."""
    rng = np.random.default_rng(bits + D)
    _, cb, stored = sq_table(oracle, rng, 400, D, bits, cs)
    deg = rng.integers(0, 26, 333)
    deg[::7] = 0
    deg[5::41] = rng.integers(60, 400, len(deg[5::41]))
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, 400, int(indptr[-1])).astype(np.int64)
    for idx in (np.int64, np.int32):
        args = (dev(stored), dev(cb), dev(indptr.astype(idx)), dev(indices.astype(idx)), bits, cs, D)
        base = capi.sq_decompress_spmm_csr(*args, kernel="general")
        ran = []
        for kernel in ("stream", "prefetch", "prefetch_arith", "auto"):
            for kw in (dict(), dict(reduce="sum"), dict(dropout=dict(p=0.3, seed=5, offset=1, training=True))):
                got = _served(lambda: capi.sq_decompress_spmm_csr(*args, kernel=kernel, **kw))
                if got is not None:
                    assert torch.equal(got, capi.sq_decompress_spmm_csr(*args, kernel="general", **kw)), (kernel, kw, idx)
                    ran.append(kernel)
        if D * bits % 128 == 0 and D * bits <= 8 * 256 and cs % (64 // bits if bits > 2 else 32 // bits) == 0:
            assert "stream" in ran, "the streamed kernel must take whole 16-byte rows whose lanes see one codebook row"
        assert torch.equal(capi.sq_decompress_spmm_csr(*args), base)
    from f2cgt_b200 import ops
    assert ops.device_status() == 0


@pytest.mark.parametrize("kind", ["sq1", "sq4", "sq8", "vq", "two_level"])
def test_streamed_kernels_over_several_chunks(capi, oracle, kind):
    """More destination rows than one pass of the grid's indptr slices (148 CTAs x 1024 rows), a table small enough
    that the general kernel is a cheap comparator: chunk boundaries, ring wrap-around, the drain between chunks."""
    rng = np.random.default_rng(11)
    n_src, n_dst, D = 3000, 320_000, 128
    deg = rng.integers(0, 14, n_dst)
    deg[::1000] = 70
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n_src, int(indptr[-1])).astype(np.int64)
    ip, ix = dev(indptr), dev(indices)
    if kind.startswith("sq"):
        bits = int(kind[2:])
        _, cb, stored = sq_table(oracle, rng, n_src, D, bits, 128)
        a = capi.sq_decompress_spmm_csr(dev(stored), dev(cb), ip, ix, bits, 128, D, kernel="stream")
        b = capi.sq_decompress_spmm_csr(dev(stored), dev(cb), ip, ix, bits, 128, D, kernel="prefetch")
    else:
        cbs = dev(rng.standard_normal((4, 256, 32)).astype(np.float32))
        codes = dev(rng.integers(0, 256, (n_src, 4)).astype(np.uint8))
        if kind == "vq":
            a = capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, D, kernel="stream")
            b = capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, D, kernel="prefetch")
        else:
            _, cb, sq = sq_table(oracle, rng, 600, D, 8, 128)
            slot = np.full(n_src, -1, np.int32)
            hot = rng.choice(n_src, 600, replace=False)
            slot[hot] = rng.permutation(600).astype(np.int32)
            t = (dev(sq), dev(cb), 8, 128, codes, cbs, dev(slot), ip, ix, D)
            a = capi.two_level_decompress_spmm_csr(*t, kernel="stream")
            b = capi.two_level_decompress_spmm_csr(*t, kernel="prefetch")
    assert torch.equal(a, b)
    from f2cgt_b200 import ops
    assert ops.device_status() == 0


@pytest.mark.parametrize("bits", [4, 16])
def test_fused_mean_division_is_the_ieee_division(capi, oracle, bits):
    """The fused kernel divides with a hoisted reciprocal and FMA corrections; the plain aggregation
    kernel uses the division operator.  12.8 M quotients, degrees 1..45, must agree bit for bit."""
    rng = np.random.default_rng(bits)
    n_src, n_dst, D = 5000, 100_000, 128
    x = (rng.standard_normal((n_src, D)) * np.exp(rng.uniform(-6, 6, (n_src, 1)))).astype(np.float32)
    cb = oracle.sq_codebooks(x, 128)
    stored = oracle.sq_codes_to_storage(oracle.sq_compress(x, cb, bits, 128), bits)
    indptr, indices = random_csc(rng, n_dst, n_src, max_deg=45, empty_every=0)
    t = (dev(stored), dev(cb), dev(indptr), dev(indices))
    fused = capi.sq_decompress_spmm_csr(*t, bits, 128, D)
    unfused = capi.spmm_csr(capi.sq_decompress(t[0], t[1], bits, 128, D), t[2], t[3])
    assert torch.equal(fused.view(torch.int32), unfused.view(torch.int32))


def test_fused_sq_golden_reference_kernels(capi, golden):
    ip, ix = dev(golden["csc_indptr"]), dev(golden["csc_indices"])
    toy_ip = torch.tensor([0, 1, 3, 6], dtype=torch.int64, device="cuda")
    toy_ix = torch.tensor([0, 1, 1, 2, 2, 0], dtype=torch.int64, device="cuda")
    for bits in (1, 2, 4, 8, 16):
        got = host(capi.sq_decompress_spmm_csr(dev(golden[f"sq_stored_b{bits}"]), dev(golden["sq_cb"]), ip, ix, bits, 100, 100))
        assert np.array_equal(got.view(np.uint32), golden[f"sq_spmm_b{bits}"].view(np.uint32)), bits
        got = host(capi.sq_decompress_spmm_csr(dev(golden[f"sq_stored_b{bits}"]), dev(golden["sq_cb"]), toy_ip, toy_ix, bits, 100, 100))
        assert np.array_equal(got.view(np.uint32), golden[f"sq_spmm_toy_b{bits}"].view(np.uint32)), bits
        got = host(capi.sq_decompress_spmm_csr(dev(golden[f"sq2_stored_b{bits}"]), dev(golden["sq2_cb"]), ip, ix, bits, 64, 128))
        assert np.array_equal(got.view(np.uint32), golden[f"sq2_spmm_b{bits}"].view(np.uint32)), bits


VQ_SHAPES = [  # (n_cb, K, cs, D)
    (16, 256, 8, 128), (4, 256, 32, 128), (4, 256, 64, 256), (2, 256, 60, 110), (3, 100, 5, 13), (1, 16, 128, 128),
    (2, 1000, 64, 128), (8, 256, 64, 512)]


@pytest.mark.parametrize("code_dtype", [np.uint8, np.int16])
@pytest.mark.parametrize("n_cb,K,cs,D", VQ_SHAPES)
def test_fused_vq_equals_unfused_and_oracle(capi, oracle, code_dtype, n_cb, K, cs, D):
    if code_dtype == np.uint8 and K > 256:
        pytest.skip("uint8 codes address at most 256 centroids")
    rng = np.random.default_rng(n_cb * 31 + cs)
    n_src, n_dst = 300, 157
    cbs = rng.standard_normal((n_cb, K, cs)).astype(np.float32)
    codes = rng.integers(0, K, (n_src, n_cb)).astype(code_dtype)
    for idx in (np.int64, np.int32):
        indptr, indices = random_csc(rng, n_dst, n_src, max_deg=40, dtype=idx)
        t = (dev(codes), dev(cbs), dev(indptr), dev(indices))
        for reduce in ("mean", "sum"):
            fused = capi.vq_decompress_spmm_csr(*t, D, reduce=reduce)
            unfused = capi.spmm_csr(capi.vq_decompress(t[0], t[1], D), t[2], t[3], reduce=reduce)
            assert torch.equal(fused, unfused), (n_cb, K, cs, D, idx, reduce)  # tests/test_fusion_decompress_spmm.py:33
            assert np.array_equal(host(fused), oracle.vq_decompress_spmm_csr(codes, cbs, indptr, indices, D, reduce))


def test_fused_vq_golden_reference_kernels(capi, golden):
    ip, ix = dev(golden["csc_indptr"]), dev(golden["csc_indices"])
    got = host(capi.vq_decompress_spmm_csr(dev(golden["vq_codes_u8"]), dev(golden["vq_cbs"]), ip, ix, 110))
    assert np.array_equal(got, golden["vq_spmm_u8"])
    got = host(capi.vq_decompress_spmm_csr(dev(golden["vq16_codes"]), dev(golden["vq16_cbs"]), ip, ix, 128))
    assert np.array_equal(got, golden["vq16_spmm"])


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("D,n_cb,cs", [(128, 4, 32), (256, 4, 64), (128, 16, 8)])
def test_two_level_is_composition(capi, oracle, bits, D, n_cb, cs):
    rng = np.random.default_rng(bits * 17 + D)
    n_src, n_hot, n_dst = 500, 60, 211
    _, cb, sq = sq_table(oracle, rng, n_hot, D, bits, D)
    cbs = rng.standard_normal((n_cb, 256, cs)).astype(np.float32)
    codes = rng.integers(0, 256, (n_src, n_cb)).astype(np.uint8)
    slot = np.full(n_src, -1, np.int32)
    hot = rng.choice(n_src, n_hot, replace=False)
    slot[hot] = rng.permutation(n_hot).astype(np.int32)
    for idx in (np.int64, np.int32):
        indptr, indices = random_csc(rng, n_dst, n_src, max_deg=40, dtype=idx)
        got = capi.two_level_decompress_spmm_csr(dev(sq), dev(cb), bits, D, dev(codes), dev(cbs), dev(slot), dev(indptr),
                                                 dev(indices), D)
        # composition on the GPU: decode all rows by their own codec, then the plain mean - must be bit-equal
        full = capi.vq_decompress(dev(codes), dev(cbs), D)
        full[dev(hot)] = capi.sq_decompress(dev(sq), dev(cb), bits, D, D)[dev(slot[hot].astype(np.int64))]
        assert torch.equal(got, capi.spmm_csr(full, dev(indptr), dev(indices)))
        want = oracle.two_level_decompress_spmm_csr(sq, cb, bits, D, codes, cbs, slot, indptr, indices, D, acc64=True)
        assert close_to_oracle(host(got), want, host(capi.spmm_csr(full.abs(), dev(indptr), dev(indices))))
    # hot-first numbering: no slot array, node s < n_hot reads SQ row s
    prefix = np.where(np.arange(n_src) < n_hot, np.arange(n_src), -1).astype(np.int32)
    for kernel in ("auto", "stream", "prefetch", "general"):
        fn = lambda sl: capi.two_level_decompress_spmm_csr(dev(sq), dev(cb), bits, D, dev(codes), dev(cbs), sl, dev(indptr),  # noqa: E731
                                                           dev(indices), D, kernel=kernel)
        a = _served(lambda: fn(None))
        if a is not None:
            assert torch.equal(a, fn(dev(prefix))), kernel
    # all-cold and all-hot degenerate to the single-codec kernels
    cold = capi.two_level_decompress_spmm_csr(dev(sq), dev(cb), bits, D, dev(codes), dev(cbs), dev(np.full(n_src, -1, np.int32)),
                                              dev(indptr), dev(indices), D)
    assert torch.equal(cold, capi.vq_decompress_spmm_csr(dev(codes), dev(cbs), dev(indptr), dev(indices), D))


@pytest.mark.parametrize("n_cb,K,cs,D", [(4, 256, 32, 128), (4, 100, 32, 100), (8, 200, 16, 128), (16, 256, 8, 128),
                                         (16, 256, 4, 64), (4, 256, 64, 256), (8, 256, 32, 256), (4, 37, 128, 512)])
@pytest.mark.parametrize("hot_bits,hot_cs", [(0, 0), (8, 0), (8, 32), (4, 0), (4, 64)])
def test_pipelined_vq_kernel_equals_general_kernel(capi, oracle, n_cb, K, cs, D, hot_bits, hot_cs):
    """The streamed and register-prefetch kernels (shared-memory codebooks, table decode of hot rows) against the
    general one and the oracle: rows with 0, 1..16, 17..32 and more than 32 neighbours, codes >= K, ragged feat_dim,
    several column parts."""
    rng = np.random.default_rng(n_cb * 7 + cs + hot_bits)
    n_src, n_hot, n_dst = 700, 90, 333
    cbs = rng.standard_normal((n_cb, K, cs)).astype(np.float32)
    codes = rng.integers(0, 256, (n_src, n_cb)).astype(np.uint8)  # some codes >= K when K < 256
    if D % 4:
        pytest.skip("two-level needs feat_dim % 4 == 0")
    deg = rng.integers(0, 14, n_dst)
    deg[::5] = rng.integers(17, 33, len(deg[::5]))
    deg[::11] = rng.integers(33, 100, len(deg[::11]))
    deg[::7] = 0
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n_src, int(indptr[-1])).astype(np.int64)
    drop = dict(p=0.3, seed=5, offset=1, training=True)

    def both(fn):
        """(kernel-family results that took the shape, general-kernel result)"""
        fast = [r for r in (_served(lambda k=k: fn(k)) for k in ("stream", "prefetch", "auto")) if r is not None]
        assert len(fast) >= 2  # "auto" always runs; the prefetch kernel takes every shape of this test
        if K == 256:
            assert len(fast) == 3, "the streamed kernel must take 256-centroid codebooks"
        return fast, fn("general")

    for idx in (np.int64, np.int32):
        ip, ix = dev(indptr.astype(idx)), dev(indices.astype(idx))
        if hot_bits == 0:
            for kw in (dict(), dict(reduce="sum"), dict(dropout=drop)):
                fast, b = both(lambda k: capi.vq_decompress_spmm_csr(dev(codes), dev(cbs), ip, ix, D, kernel=k, **kw))
                assert all(torch.equal(a, b) for a in fast), kw
            want = oracle.vq_decompress_spmm_csr(np.minimum(codes, K - 1).astype(np.uint8), cbs, indptr, indices, D, "mean")
            assert np.array_equal(host(capi.vq_decompress_spmm_csr(dev(codes), dev(cbs), ip, ix, D)), want)
        else:
            hcs = hot_cs or D
            for signed in (True, False):
                _, cb, sq = sq_table(oracle, rng, n_hot, D, hot_bits, hcs)
                if hot_bits == 8 and not signed:
                    sq = sq.view(np.uint8)
                slot = np.full(n_src, -1, np.int32)
                hot = rng.choice(n_src, n_hot, replace=False)
                slot[hot] = rng.permutation(n_hot).astype(np.int32)
                for kw in (dict(), dict(reduce="sum"), dict(dropout=drop)):
                    fast, b = both(lambda k: capi.two_level_decompress_spmm_csr(dev(sq), dev(cb), hot_bits, hcs, dev(codes), dev(cbs),
                                                                                dev(slot), ip, ix, D, kernel=k, **kw))
                    assert all(torch.equal(a, b) for a in fast), (kw, signed)


def test_config5_shape_at_scale(capi, oracle):
    """Configuration 5's codecs on a block of realistic size: D = 256, hot 2 % SQ 4 bits + VQ 4 x 64 (256 KB of
    codebooks: two column parts), 150,000 source rows, 12,000 destination rows of up to 15 neighbours.  Every kernel
    family against the composition decode-each-row-by-its-codec, then the plain mean (bit-equal), and the oracle."""
    rng = np.random.default_rng(5)
    n_src, n_hot, n_dst, D = 150_000, 3000, 12_000, 256
    _, cb, sq = sq_table(oracle, rng, n_hot, D, 4, D)
    cbs = rng.standard_normal((4, 256, 64)).astype(np.float32)
    codes = rng.integers(0, 256, (n_src, 4)).astype(np.uint8)
    slot = np.full(n_src, -1, np.int32)
    hot = rng.choice(n_src, n_hot, replace=False)
    slot[hot] = rng.permutation(n_hot).astype(np.int32)
    deg = rng.integers(0, 16, n_dst)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    # half of the edges point at hot rows, as degree-proportional sampling does
    indices = np.where(rng.random(int(indptr[-1])) < 0.5, rng.choice(hot, int(indptr[-1])), rng.integers(0, n_src, int(indptr[-1]))).astype(np.int64)
    t = (dev(sq), dev(cb), 4, D, dev(codes), dev(cbs), dev(slot), dev(indptr), dev(indices), D)
    full = capi.vq_decompress(dev(codes), dev(cbs), D)
    full[dev(hot)] = capi.sq_decompress(dev(sq), dev(cb), 4, D, D)[dev(slot[hot].astype(np.int64))]
    want = capi.spmm_csr(full, dev(indptr), dev(indices))
    for kernel in ("auto", "stream", "prefetch", "general"):
        assert torch.equal(capi.two_level_decompress_spmm_csr(*t, kernel=kernel), want), kernel
    ref = oracle.two_level_decompress_spmm_csr(sq, cb, 4, D, codes, cbs, slot, indptr, indices, D, acc64=True)
    assert close_to_oracle(host(want), ref, host(capi.spmm_csr(full.abs(), dev(indptr), dev(indices))))
    cold = capi.vq_decompress_spmm_csr(dev(codes), dev(cbs), dev(indptr), dev(indices), D)
    assert np.array_equal(host(cold), oracle.vq_decompress_spmm_csr(codes, cbs, indptr, indices, D))


@pytest.mark.parametrize("kind", ["sq", "vq", "two_level"])
def test_fused_dropout_equals_dropout_after(capi, oracle, kind):
    rng = np.random.default_rng(99)
    D, n_src, n_dst = 128, 300, 200
    indptr, indices = random_csc(rng, n_dst, n_src)
    ip, ix = dev(indptr), dev(indices)
    drop = dict(p=0.5, seed=77, offset=5, training=True)
    cbs = dev(rng.standard_normal((4, 256, 32)).astype(np.float32))
    codes = dev(rng.integers(0, 256, (n_src, 4)).astype(np.uint8))
    _, cb, sq = sq_table(oracle, rng, n_src, D, 4, 128)
    if kind == "sq":
        plain = capi.sq_decompress_spmm_csr(dev(sq), dev(cb), ip, ix, 4, 128, D)
        fused = capi.sq_decompress_spmm_csr(dev(sq), dev(cb), ip, ix, 4, 128, D, dropout=drop)
    elif kind == "vq":
        plain = capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, D)
        fused = capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, D, dropout=drop)
    else:
        slot = dev(np.where(rng.random(n_src) < 0.3, np.arange(n_src), -1).astype(np.int32))
        plain = capi.two_level_decompress_spmm_csr(dev(sq), dev(cb), 4, 128, codes, cbs, slot, ip, ix, D)
        fused = capi.two_level_decompress_spmm_csr(dev(sq), dev(cb), 4, 128, codes, cbs, slot, ip, ix, D, dropout=drop)
    after = capi.dropout_inplace(plain.clone(), 0.5, True, seed=77, offset=5)
    assert torch.equal(fused, after)
    assert 0.4 < float((fused == 0).float().mean()) < 0.62
    assert np.array_equal(host(after), oracle.dropout(host(plain), 0.5, True, 77, 5))


def test_config1_sq8_block(capi, oracle):
    """The CPU-runnable configuration: 100,000 x 128 N(0,1) features, 8-bit codes, 10,000 destination
    rows with exactly 12 uniform neighbours, int64 CSC, seed 0."""
    rng = np.random.default_rng(0)
    x, cb, stored = sq_table(oracle, rng, 100_000, 128, 8, 128)
    indptr = np.arange(0, 120_001, 12, dtype=np.int64)
    indices = rng.integers(0, 100_000, 120_000).astype(np.int64)
    got = host(capi.sq_decompress_spmm_csr(dev(stored), dev(cb), dev(indptr), dev(indices), 8, 128, 128))
    want = oracle.sq_decompress_spmm_csr(stored, cb, indptr, indices, 8, 128, 128, acc64=True)
    assert got.shape == (10_000, 128) and close_to_oracle(got, want)
    # per-column codebooks (column_slice = 1)
    cb1 = oracle.sq_codebooks(x[:20000], 1)
    st1 = oracle.sq_codes_to_storage(oracle.sq_compress(x[:20000], cb1, 8, 1), 8)
    ix1 = indices[:24000] % 20000
    got1 = host(capi.sq_decompress_spmm_csr(dev(st1), dev(cb1), dev(indptr[:2001]), dev(ix1), 8, 1, 128))
    assert close_to_oracle(got1, oracle.sq_decompress_spmm_csr(st1, cb1, indptr[:2001], ix1, 8, 1, 128, acc64=True))


def test_empty_and_degenerate_blocks(capi):
    cb = torch.tensor([[0.01, 3.0, -6.6, 1.6, 0.8]], device="cuda")
    codes = torch.zeros((5, 64), dtype=torch.uint8, device="cuda")
    # no destination rows
    out = capi.sq_decompress_spmm_csr(codes, cb, torch.zeros(1, dtype=torch.int64, device="cuda"),
                                      torch.zeros(0, dtype=torch.int64, device="cuda"), 4, 128, 128)
    assert out.shape == (0, 128)
    # destination rows without any edge -> zeros
    out = capi.sq_decompress_spmm_csr(codes, cb, torch.zeros(8, dtype=torch.int64, device="cuda"),
                                      torch.zeros(0, dtype=torch.int64, device="cuda"), 4, 128, 128)
    assert out.shape == (7, 128) and float(out.abs().max()) == 0.0
    cbs = torch.randn(4, 256, 32, device="cuda")
    out = capi.vq_decompress_spmm_csr(torch.zeros((5, 4), dtype=torch.uint8, device="cuda"), cbs,
                                      torch.zeros(8, dtype=torch.int32, device="cuda"),
                                      torch.zeros(0, dtype=torch.int32, device="cuda"), 128)
    assert out.shape == (7, 128) and float(out.abs().max()) == 0.0
    with pytest.raises(RuntimeError):  # mixed index dtypes
        capi.vq_decompress_spmm_csr(torch.zeros((5, 4), dtype=torch.uint8, device="cuda"), cbs,
                                    torch.zeros(8, dtype=torch.int32, device="cuda"),
                                    torch.zeros(0, dtype=torch.int64, device="cuda"), 128)


def test_runs_on_the_callers_stream(capi):
    # the reference launches on the legacy stream; this library must honour torch's current stream
    s = torch.cuda.Stream()
    cbs = torch.randn(4, 256, 32, device="cuda")
    codes = torch.randint(0, 256, (1000, 4), dtype=torch.uint8, device="cuda")
    ip = torch.arange(0, 1201, 12, dtype=torch.int64, device="cuda")
    ix = torch.randint(0, 1000, (1200,), dtype=torch.int64, device="cuda")
    want = capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, 128)
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        got = capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, 128)
    s.synchronize()
    assert torch.equal(got, want)


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("world", [2, 3, 8])
def test_peer_sharded_table_equals_whole_table(capi, oracle, bits, world):
    """The row-sharded entry point with every shard on this GPU (the pointers could as well be peer mappings)."""
    from f2cgt_b200 import ops, shard
    rng = np.random.default_rng(bits + world)
    n_src, n_dst, D = 1003, 400, 128
    _, cb, stored = sq_table(oracle, rng, n_src, D, bits, 128)
    indptr, indices = random_csc(rng, n_dst, n_src, max_deg=20)
    table = dev(stored)
    rpr = shard.rows_per_rank(n_src, world)

    class FakePeers:  # what shard.PeerTable exposes
        pass
    pt = FakePeers()
    pt.world, pt.rpr, pt.n_rows = world, rpr, n_src
    tensors = [table[r * rpr:(r + 1) * rpr].clone() if r * rpr < n_src else table[:1].clone() for r in range(world)]
    pt.pointers = [t.data_ptr() for t in tensors]
    pt.dtype, pt.row_width = table.dtype, table.shape[1]
    got = ops.sq_decompress_spmm_csr_peer(pt, dev(cb), dev(indptr), dev(indices), bits, 128, D)
    want = capi.sq_decompress_spmm_csr(table, dev(cb), dev(indptr), dev(indices), bits, 128, D)
    assert torch.equal(got, want)


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("world,n_rep", [(2, 1), (3, 100), (8, 400), (4, 700), (2, 850)])
def test_peer_sharded_table_with_replicated_leading_rows(capi, oracle, bits, world, n_rep):
    """Hot-first numbering: rows [0, n_rep) from the local copy, row n_rep + r from the sharded remainder (every shard on
    this GPU here); up to most of the table replicated; more replicated rows than the 16 slots of the pointer table hold are refused."""
    from f2cgt_b200 import ops, shard
    rng = np.random.default_rng(bits * 10 + world)
    n_src, n_dst, D = 1003, 400, 128
    _, cb, stored = sq_table(oracle, rng, n_src, D, bits, 128)
    indptr, indices = random_csc(rng, n_dst, n_src, max_deg=20)
    table = dev(stored)
    cold = n_src - n_rep
    rpr = shard.rows_per_rank(cold, world)

    class FakePeers:
        pass
    pt = FakePeers()
    pt.world, pt.rpr, pt.n_rows = world, rpr, cold
    tail = table[n_rep:]
    tensors = [tail[r * rpr:(r + 1) * rpr].clone() if r * rpr < cold else table[:1].clone() for r in range(world)]
    pt.pointers = [t.data_ptr() for t in tensors]
    pt.dtype, pt.row_width = table.dtype, table.shape[1]
    head = table[:n_rep].clone()
    # ids of the sharded rows start at the next multiple of the shard size
    first_cold = ops.peer_first_cold_id(n_rep, rpr)
    assert first_cold >= n_rep and first_cold % rpr == 0 and first_cold - n_rep < rpr
    ids = np.where(indices < n_rep, indices, indices - n_rep + first_cold)
    got = ops.sq_decompress_spmm_csr_peer(pt, dev(cb), dev(indptr), dev(ids), bits, 128, D, replicated=head)
    want = capi.sq_decompress_spmm_csr(table, dev(cb), dev(indptr), dev(indices), bits, 128, D)
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError):  # the streamed family does not serve this layout and says so
        ops.sq_decompress_spmm_csr_peer(pt, dev(cb), dev(indptr), dev(ids), bits, 128, D, replicated=head, kernel="stream")
    if world == 8:
        with pytest.raises(RuntimeError):  # 900 replicated rows = 69 slots of 13 rows beside 8 shards
            big = FakePeers()
            big.world, big.rpr, big.n_rows, big.pointers, big.dtype, big.row_width = 8, 13, 103, pt.pointers, table.dtype, table.shape[1]
            ops.sq_decompress_spmm_csr_peer(big, dev(cb), dev(indptr), dev(ids), bits, 128, D, replicated=table[:900].clone())


@pytest.mark.parametrize("hot_bits,D,n_cb,cs", [(8, 128, 4, 32), (4, 256, 4, 64), (8, 128, 16, 8), (0, 128, 4, 32)])
@pytest.mark.parametrize("world,hot_first", [(2, False), (3, True), (8, False)])
def test_two_level_over_sharded_tables_equals_whole_tables(capi, oracle, hot_bits, D, n_cb, cs, world, hot_first):
    """The sharded two-level / VQ entry point with every shard on this GPU (the pointers could as well be peer mappings)."""
    from f2cgt_b200 import ops, shard
    rng = np.random.default_rng(hot_bits + world + D)
    n_src, n_hot, n_dst = 1003, 101, 400
    cbs = dev(rng.standard_normal((n_cb, 256, cs)).astype(np.float32))
    codes = dev(rng.integers(0, 256, (n_src, n_cb)).astype(np.uint8))
    indptr, indices = random_csc(rng, n_dst, n_src, max_deg=40)
    ip, ix = dev(indptr), dev(indices)

    class Peers:  # what shard.PeerTable exposes
        def __init__(self, table, n_rows):
            self.world, self.n_rows = world, n_rows
            self.rpr = shard.rows_per_rank(n_rows, world)
            self.keep = [table[r * self.rpr:(r + 1) * self.rpr].clone() if r * self.rpr < n_rows else table[:1].clone() for r in range(world)]
            self.pointers = [t.data_ptr() for t in self.keep]
            self.dtype, self.row_width = table.dtype, table.shape[1]
    vq_peers = Peers(codes, n_src)
    if hot_bits == 0:
        got = ops.two_level_decompress_spmm_csr_peer(None, None, 0, 0, vq_peers, cbs, None, ip, ix, D)
        assert torch.equal(got, capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, D))
        return
    _, cb, sq = sq_table(oracle, rng, n_hot, D, hot_bits, D)
    sq_t = dev(sq)
    if hot_first:
        slot = torch.where(torch.arange(n_src, device="cuda") < n_hot, torch.arange(n_src, device="cuda"), -1).to(torch.int32)
        slot_peers = None
    else:
        slot_np = np.full(n_src, -1, np.int32)
        slot_np[rng.choice(n_src, n_hot, replace=False)] = rng.permutation(n_hot).astype(np.int32)
        slot = dev(slot_np)
        slot_peers = Peers(slot.reshape(-1, 1), n_src)
    got = ops.two_level_decompress_spmm_csr_peer(Peers(sq_t, n_hot), dev(cb), hot_bits, D, vq_peers, cbs, slot_peers, ip, ix, D)
    want = capi.two_level_decompress_spmm_csr(sq_t, dev(cb), hot_bits, D, codes, cbs, slot, ip, ix, D)
    assert torch.equal(got, want)
