"""GPU parity of the minibatch builders: neighbour sampling and relabelling (stand-ins for the reference's absent
ShmTensor operators, contracts read from examples/dataloader.py:167-182) against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def small_graph(rng, n, max_deg, dtype=np.int64):
    deg = rng.integers(0, max_deg + 1, n)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(dtype)
    indices = rng.integers(0, n, int(indptr[-1])).astype(dtype)
    return indptr, indices


@pytest.mark.parametrize("idx", [np.int64, np.int32])
@pytest.mark.parametrize("num_pick", [1, 5, 12, 64])
def test_csr_sampling_equals_oracle(capi, oracle, idx, num_pick):
    from f2cgt_b200 import ops
    rng = np.random.default_rng(num_pick)
    indptr, indices = small_graph(rng, 3000, 40, idx)
    seeds = rng.choice(3000, 700, replace=False).astype(idx)
    ip, ix = ops.csr_sampling(dev(indptr), dev(indices), dev(seeds), num_pick, False, rng_seed=11, rng_offset=3)
    want_ip, want_ix = oracle.sample_neighbors(indptr, indices, seeds, num_pick, 11, 3)
    assert np.array_equal(host(ip), want_ip) and np.array_equal(host(ix), want_ix)
    # contract: min(deg, num_pick) distinct positions of the seed's own adjacency list
    ip, ix = host(ip), host(ix)
    for j, v in enumerate(seeds[:200]):
        mine = ix[ip[j]:ip[j + 1]]
        adj = indices[indptr[v]:indptr[v + 1]]
        assert len(mine) == min(len(adj), num_pick)
        assert np.all(np.isin(mine, adj))
        if len(adj) <= num_pick:
            assert np.array_equal(mine, adj)


def test_csr_sampling_is_uniform():
    """Every neighbour of a high-degree seed is picked with probability num_pick / degree (chi-square over seeds)."""
    from f2cgt_b200 import ops
    deg, num_pick, copies = 40, 10, 20000
    indptr = np.arange(0, (copies + 1) * deg, deg, dtype=np.int64)
    indices = np.tile(np.arange(deg, dtype=np.int64), copies)  # every node has neighbours 0..39
    seeds = np.arange(copies, dtype=np.int64)
    _, ix = ops.csr_sampling(dev(indptr), dev(indices), dev(seeds), num_pick, False, rng_seed=5)
    counts = np.bincount(host(ix), minlength=deg).astype(np.float64)
    expect = copies * num_pick / deg
    chi2 = ((counts - expect) ** 2 / expect).sum()
    assert chi2 < 90.0  # 39 degrees of freedom: P(chi2 > 90) ~ 1e-5


@pytest.mark.parametrize("idx", [np.int64, np.int32])
@pytest.mark.parametrize("n_seeds,n_ids,space", [(0, 0, 10), (5, 0, 100), (1024, 12000, 5000), (300, 50000, 1 << 30), (1, 100000, 7)])
def test_tensor_relabel_equals_oracle(capi, oracle, idx, n_seeds, n_ids, space):
    from f2cgt_b200 import ops
    rng = np.random.default_rng(n_seeds + n_ids)
    seeds = rng.choice(space, n_seeds, replace=False).astype(idx) if n_seeds else np.zeros(0, idx)
    ids = rng.integers(0, space, n_ids).astype(idx)
    uniq, (rs, ri) = ops.tensor_relabel([dev(seeds), dev(ids)])
    want_u, (want_s, want_i) = oracle.tensor_relabel([seeds, ids])
    assert np.array_equal(host(uniq), want_u)
    assert np.array_equal(host(rs), want_s) and np.array_equal(host(ri), want_i)
    # the contract itself: seeds keep their positions, unique[relabelled] reproduces the ids
    assert np.array_equal(host(rs), np.arange(n_seeds))
    if n_ids:
        assert np.array_equal(host(uniq)[host(ri)], ids)


def test_blocks_feed_the_fused_kernel(capi, oracle):
    """sample -> relabel -> block: destination nodes are a prefix of the source nodes in every hop, and aggregating the
    block-local rows gives the rows obtained by global ids."""
    from f2cgt_b200 import synth
    indptr, indices = synth.power_law_graph(20000, 20, 2.1, seed=3, device="cuda")
    seeds = torch.randperm(20000, device="cuda")[:256]
    blocks = synth.sample_blocks(indptr, indices, seeds, (5, 4, 3), rng_seed=2)
    assert len(blocks) == 3 and torch.equal(blocks[-1]["dst_nodes"], seeds)
    codes, cb = synth.sq_table_from_normal(20000, 128, 4, 128, seed=0, device="cuda")
    for b in blocks:
        n_dst = b["dst_nodes"].numel()
        assert torch.equal(b["src_nodes"][:n_dst], b["dst_nodes"])
        assert b["src_nodes"].unique().numel() == b["src_nodes"].numel()
        assert torch.equal(b["src_nodes"][b["indices_local"]], b["indices_global"])
        by_global = capi.sq_decompress_spmm_csr(codes, cb, b["indptr"], b["indices_global"], 4, 128, 128)
        gathered = codes[b["src_nodes"]]
        by_local = capi.sq_decompress_spmm_csr(gathered, cb, b["indptr"], b["indices_local"], 4, 128, 128)
        assert torch.equal(by_global, by_local)
    for outer, inner in zip(blocks[:-1], blocks[1:]):
        assert torch.equal(outer["dst_nodes"], inner["src_nodes"])


def test_relabel_rejects_negative_ids_and_padded_sampling_numbers_alike(capi):
    from f2cgt_b200 import ops
    ids = torch.tensor([5, 3, -1, 5], dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="negative id"):
        ops.tensor_relabel([ids])
    # csr_sampling(exact=False) pads its index tensor with copies of seeds[0]: same CSC, same numbering
    from f2cgt_b200 import synth
    indptr, indices = synth.power_law_graph(5000, 20, 2.1, seed=2, device="cuda")
    seeds = torch.randperm(5000, device="cuda")[:300]
    ip_a, ix_a = ops.csr_sampling(indptr, indices, seeds, 7, False, rng_seed=5, rng_offset=2)
    ip_b, ix_b = ops.csr_sampling(indptr, indices, seeds, 7, False, rng_seed=5, rng_offset=2, exact=False)
    nnz = int(ip_a[-1])
    assert torch.equal(ip_a, ip_b) and ix_b.numel() == 300 * 7 and torch.equal(ix_a, ix_b[:nnz])
    assert bool((ix_b[nnz:] == seeds[0]).all())
    ua, (_, la) = ops.tensor_relabel([seeds, ix_a])
    ub, (_, lb) = ops.tensor_relabel([seeds, ix_b])
    assert torch.equal(ua, ub) and torch.equal(la, lb[:nnz])


@pytest.mark.parametrize("idx", [np.int64, np.int32])
@pytest.mark.parametrize("num_pick,n_seeds", [(1, 1), (5, 700), (12, 1000), (64, 33)])
def test_sample_block_equals_the_separate_operators_and_the_oracle(capi, oracle, idx, num_pick, n_seeds):
    """The one-call hop gives the sampler's CSC and the relabelling's numbering, bit for bit."""
    from f2cgt_b200 import ops
    rng = np.random.default_rng(num_pick * 31 + n_seeds)
    indptr, indices = small_graph(rng, 3000, 40, idx)
    seeds = rng.choice(3000, n_seeds, replace=False).astype(idx)
    ip, ix, uniq, local = ops.sample_block(dev(indptr), dev(indices), dev(seeds), num_pick, rng_seed=11, rng_offset=3)
    want_ip, want_ix = oracle.sample_neighbors(indptr, indices, seeds, num_pick, 11, 3)
    want_uniq, (_, want_local) = oracle.tensor_relabel([seeds, want_ix])
    nnz = int(want_ip[-1])
    assert ix.numel() == n_seeds * num_pick and local.numel() == n_seeds * num_pick
    assert np.array_equal(host(ip), want_ip)
    assert np.array_equal(host(ix)[:nnz], want_ix) and np.all(host(ix)[nnz:] == seeds[0])
    assert np.array_equal(host(uniq), want_uniq)
    assert np.array_equal(host(local)[:nnz], want_local) and np.all(host(local)[nnz:] == 0)
    # and the separate entry points agree with it
    ip2, ix2 = ops.csr_sampling(dev(indptr), dev(indices), dev(seeds), num_pick, False, rng_seed=11, rng_offset=3)
    uniq2, (_, local2) = ops.tensor_relabel([dev(seeds), ix2])
    assert torch.equal(ip, ip2) and torch.equal(ix[:nnz], ix2) and torch.equal(uniq, uniq2) and torch.equal(local[:nnz], local2)


def test_sample_block_of_isolated_seeds(capi):
    """Seeds without neighbours: an empty block whose only nodes are the seeds."""
    from f2cgt_b200 import ops
    indptr = torch.zeros(11, dtype=torch.int64, device="cuda")
    indices = torch.zeros(0, dtype=torch.int64, device="cuda")
    seeds = torch.tensor([4, 2, 9], device="cuda")
    ip, ix, uniq, local = ops.sample_block(indptr, indices, seeds, 5)
    assert ip.tolist() == [0, 0, 0, 0] and uniq.tolist() == [4, 2, 9]
    assert ix.tolist() == [4] * 15 and local.tolist() == [0] * 15
