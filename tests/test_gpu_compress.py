"""GPU: the offline compressor and its artefact format (flow of examples/process_compress.py of the reference)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def corr(a, b):
    a, b = a.flatten().double(), b.flatten().double()
    return float(((a - a.mean()) * (b - b.mean())).mean() / (a.std(unbiased=False) * b.std(unbiased=False)))


def test_sq_codebook_recipe_matches_oracle(capi, oracle):
    from f2cgt_b200 import compress
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(20000, 24, generator=g, device="cuda") * 3
    _, cb = compress.sq_compress_features(x, 4, 8, sample_size=1 << 30)  # sample = every row, as the oracle takes it
    want = oracle.sq_codebooks(x.cpu().numpy(), 8)
    assert cb.shape == (3, 5)
    assert np.allclose(cb.cpu().numpy(), want, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("ratio,bits,min_corr", [(4, 8, 0.999), (8, 4, 0.95), (16, 2, 0.8), (32, 1, 0.55)])
def test_sq_artefact(capi, oracle, ratio, bits, min_corr, tmp_path):
    from f2cgt_b200 import compress
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(30000, 64, generator=g, device="cuda")
    meta = compress.compress(x, target_compression_ratio=ratio)
    assert meta["methods"] == ["sq"] and meta["configs"] == [(64, bits)] and meta["feat_dim"] == 64
    table = meta["compression_data"]
    assert table.dtype == torch.int8 and tuple(table.shape) == (30000, 64 * bits // 8)
    assert meta["data"]["compression_data"] == (torch.int8, (30000, 64 * bits // 8))
    # the stored codes are the oracle's codes for these codebooks (modulo elements on a quantisation boundary)
    cb_np, x_np = meta["codebooks"][0].cpu().numpy(), x.cpu().numpy()
    want = oracle.sq_compress(x_np, cb_np, bits, 64)
    # compare element by element (unpacked): a stored code may differ from the oracle's only where the pre-floor value
    # sits on a quantisation boundary (log2f differs by an ulp between libdevice and libm), and then by one bucket
    stored = table.view(torch.uint8) if bits < 8 else table
    got = capi.unpackbits(stored.contiguous(), bits, 64).cpu().numpy().astype(np.int64) if bits < 8 else table.cpu().numpy().astype(np.int64)
    want_store = np.asarray(want).astype(np.int64) & ((1 << bits) - 1) if bits < 8 else np.asarray(want).astype(np.int64)
    bad = got != want_store
    if bad.any():
        pre = oracle.sq_compress_prefloor(x_np, cb_np, bits, 64)
        assert np.all(np.abs(pre[bad] - np.round(pre[bad])) < max(1e-3, 2.0 ** (bits - 1) * 2e-6))
        assert bad.mean() < 0.015
    dec = compress.decompress(meta)
    assert corr(dec, x) > min_corr
    compress.save(meta, str(tmp_path))
    back = compress.load(str(tmp_path))
    assert back["methods"] == meta["methods"] and back["configs"] == meta["configs"]
    assert torch.equal(back["compression_data"], table) and torch.equal(back["codebooks"][0], meta["codebooks"][0])


def test_vq_and_two_level_artefact(capi, tmp_path):
    from f2cgt_b200 import compress, ops, sage
    g = torch.Generator(device="cuda").manual_seed(2)
    n, D = 40000, 128
    # clustered features: every 32-column slice is one of 64 prototypes plus noise, so 256 centres can represent them
    protos = torch.randn(4, 64, 32, generator=g, device="cuda") * 2
    which = torch.randint(0, 64, (n, 4), generator=g, device="cuda")
    x = torch.cat([protos[s][which[:, s]] for s in range(4)], dim=1) + 0.05 * torch.randn(n, D, generator=g, device="cuda")
    seeds = torch.randperm(n, generator=g, device="cuda")[:1000]
    meta = compress.compress(x, seeds=seeds, target_compression_ratio=128, n_clusters=256, max_iter=30)
    assert meta["methods"] == ["sq", "vq"] and meta["configs"] == [(128, 4), (32, -1)]
    assert meta["compression_data"].dtype == torch.uint8 and tuple(meta["compression_data"].shape) == (n, 4)
    assert tuple(meta["seeds_compression_data"].shape) == (1000, 64) and tuple(meta["codebooks"][1].shape) == (4, 256, 32)
    dec = compress.decompress(meta)
    assert corr(dec, x) > 0.98
    compress.save(meta, str(tmp_path))
    back = compress.load(str(tmp_path))
    assert torch.equal(back["compression_data"], meta["compression_data"]) and torch.equal(back["seeds"], seeds)
    cm = compress.to_manager(back)
    assert isinstance(cm, sage.CompressionManager) and cm.is_two_level
    # seeds decode from their SQ rows, everybody else from the VQ table
    hot_dec = ops.sq_decompress(meta["seeds_compression_data"], meta["codebooks"][0], 4, 128, D)
    assert torch.equal(cm.decode_rows(seeds), hot_dec)
    others = torch.tensor([i for i in range(200) if i not in set(seeds.tolist())], device="cuda")
    assert torch.equal(cm.decode_rows(others), dec[others])
    assert corr(hot_dec, x[seeds]) > 0.97


def test_rank_split_equals_single_process(capi):
    """The compressor split over a process group (column slices for the codebooks, row ranges for the codes) gives the
    artefact a single process computes for the same world size.  One rank here; two ranks in tests/test_gpu_multi.py."""
    import os
    import torch.distributed as dist
    from f2cgt_b200 import compress
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(20000, 64, generator=g, device="cuda")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        for ratio in (8, 64):
            a = compress.compress(x, target_compression_ratio=ratio, max_iter=10)
            b = compress.compress(x, target_compression_ratio=ratio, max_iter=10, group=dist.group.WORLD)
            assert torch.equal(a["compression_data"], b["compression_data"]) and torch.equal(a["codebooks"][0], b["codebooks"][0])
            c = compress.compress(x, target_compression_ratio=ratio, max_iter=10, group=dist.group.WORLD, gather=False)
            assert c["row_range"] == (0, 20000) and torch.equal(c["compression_data"], a["compression_data"])
    finally:
        dist.destroy_process_group()
