"""Two GPUs, one process each (NCCL): the row-sharded table read through CUDA-IPC peer mappings and through the
all-to-all row exchange gives the same aggregated rows as the whole table on one GPU.  Skipped on a one-GPU box."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import F2CGTLib as capi
        from f2cgt_b200 import ops, shard
        n_rows, D = 20011, 128
        for bits in (1, 4, 8):
            g = torch.Generator().manual_seed(bits)  # the same table, codebook and block on every rank
            width = D * bits // 8
            table = torch.randint(0, 256, (n_rows, width), generator=g, dtype=torch.uint8).to(device)
            cb = torch.tensor([[1e-3, 4.0, -9.97, 2.0, 0.7]], dtype=torch.float32, device=device)
            g2 = torch.Generator().manual_seed(1000 + rank)  # a different block per rank
            deg = torch.randint(0, 30, (700,), generator=g2)
            indptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(deg, 0)]).to(device)
            indices = torch.randint(0, n_rows, (int(deg.sum()),), generator=g2).to(device)
            want = capi.sq_decompress_spmm_csr(table, cb, indptr, indices, bits, D, D)
            lo, hi = shard.shard_bounds(n_rows, world, rank)
            local = table[lo:hi].clone()
            # 1. all-to-all row exchange (NCCL), kernel on block-local rows
            st = shard.ShardedTable(local, n_rows)
            src, inverse = torch.unique(indices, return_inverse=True)
            rows = st.fetch(src)
            got2 = capi.sq_decompress_spmm_csr(rows, cb, indptr, inverse, bits, D, D)
            assert torch.equal(got2, want), f"all-to-all fetch differs at {bits} bits"
            print(f"rank {rank} bits {bits}: all-to-all ok", file=sys.stderr, flush=True)
            # 2. the peer mappings, through the copy engine: head and tail of every shard
            peers = shard.PeerTable(local, n_rows)
            for r in range(world):
                rlo, rhi = shard.shard_bounds(n_rows, world, r)
                whole = table[rlo:rhi].reshape(-1)
                n = min(4096, whole.numel())
                assert torch.equal(peers.read(r, 0, n), whole[:n]), f"mapping of shard {r}: head differs"
                assert torch.equal(peers.read(r, whole.numel() - n, n), whole[-n:]), f"mapping of shard {r}: tail differs"
            print(f"rank {rank} bits {bits}: mappings ok", file=sys.stderr, flush=True)
            # 3. the kernel reads remote rows itself
            for kernel in ("auto", "stream", "prefetch"):
                got = ops.sq_decompress_spmm_csr_peer(peers, cb, indptr, indices, bits, D, D, kernel=kernel)
                torch.cuda.synchronize()
                assert torch.equal(got, want), f"peer loads ({kernel} kernel) differ at {bits} bits"
            print(f"rank {rank} bits {bits}: peer loads ok", file=sys.stderr, flush=True)
            peers.close()  # collective: nobody frees its shard while a peer may still read it
            # 4. the first 1,500 rows on every GPU, the rest sharded (its ids start at the next multiple of the shard size)
            n_rep = 1500
            cold = n_rows - n_rep
            clo, chi = shard.shard_bounds(cold, world, rank)
            tail = shard.PeerTable(table[n_rep + clo:n_rep + chi].clone(), cold)
            first_cold = ops.peer_first_cold_id(n_rep, tail.rpr)
            ids = torch.where(indices < n_rep, indices, indices + (first_cold - n_rep))
            got = ops.sq_decompress_spmm_csr_peer(tail, cb, indptr, ids, bits, D, D, replicated=table[:n_rep].clone())
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"peer loads with replicated leading rows differ at {bits} bits"
            tail.close()
        # a table too small to give every rank rows: the last shard is short or empty
        for tiny in (3, 2):
            g = torch.Generator().manual_seed(tiny)
            table = torch.randint(0, 256, (tiny, 64), generator=g, dtype=torch.uint8).to(device)
            cb = torch.tensor([[1e-3, 4.0, -9.97, 2.0, 0.7]], dtype=torch.float32, device=device)
            indptr = torch.tensor([0, 2, 2, 5], dtype=torch.int64, device=device)
            indices = torch.tensor([0, tiny - 1, 1, 0, tiny - 1], dtype=torch.int64, device=device)
            lo, hi = shard.shard_bounds(tiny, world, rank)
            peers = shard.PeerTable(table[lo:hi].clone(), tiny)
            got = ops.sq_decompress_spmm_csr_peer(peers, cb, indptr, indices, 4, D, D)
            assert torch.equal(got, capi.sq_decompress_spmm_csr(table, cb, indptr, indices, 4, D, D)), f"{tiny}-row table"
            peers.close()
        assert ops.device_status() == 0
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def _run(target, world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results == {r: "ok" for r in range(world)}, results


def test_sharded_table_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(_worker, 2)


def _manager_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from f2cgt_b200 import sage, shard, synth
        n, D, n_hot = 30011, 128, 1777
        g = torch.Generator(device=device).manual_seed(7)  # the same tables on every rank
        indptr, indices = synth.power_law_graph(n, 15, 2.1, seed=1, device=device)
        vq_codes = torch.randint(0, 256, (n, 4), generator=g, dtype=torch.uint8, device=device)
        vq_cbs = torch.randn(4, 256, 32, generator=g, device=device)
        hot = torch.randperm(n, generator=g, device=device)[:n_hot]
        slot = torch.full((n,), -1, dtype=torch.int32, device=device)
        slot[hot] = torch.arange(n_hot, dtype=torch.int32, device=device)
        sq_codes = torch.randint(-128, 128, (n_hot, D), generator=g, dtype=torch.int8, device=device)
        sq_cb = synth.sq_codebook_from_sample(torch.randn(5000, D, generator=g, device=device), D)
        methods, configs, cbs = ["sq", "vq"], [(D, 8), (32, 8)], [sq_cb, vq_cbs]
        whole = sage.CompressionManager(D, methods, configs, cbs, [sq_codes, vq_codes], slot)
        lo, hi = shard.shard_bounds(n, world, rank)
        hlo, hhi = shard.shard_bounds(n_hot, world, rank)
        parts = sage.ShardedCompressionManager(D, methods, configs, cbs, [sq_codes[hlo:hhi].clone(), vq_codes[lo:hi].clone()],
                                               [n_hot, n], slot[lo:hi].clone())
        g2 = torch.Generator(device=device).manual_seed(100 + rank)  # a different minibatch per rank
        seeds = torch.randperm(n, generator=g2, device=device)[:200]
        loader = sage.GPUSamplingDataloader(indptr, indices, seeds, 200, (5, 4), shuffle=False, rng_seed=rank)
        for _ in range(2):
            _, _, blocks = next(iter(loader))
            b = blocks[0]
            sm, neigh, dst = parts.for_block(b)
            assert torch.equal(sm.aggregate(b["indptr"], neigh), whole.aggregate(b["indptr"], b["indices_global"]))
            assert torch.equal(sm.decode_rows(dst), whole.decode_rows(b["dst_nodes"]))
        # the same shards mapped into every rank: the kernel reads remote code rows, slots and hot rows itself (no exchange)
        peers = sage.PeerCompressionManager(D, methods, configs, cbs, [sq_codes[hlo:hhi].clone(), vq_codes[lo:hi].clone()],
                                            [n_hot, n], slot[lo:hi].clone())
        sm, neigh, dst = peers.for_block(b)
        assert torch.equal(sm.aggregate(b["indptr"], neigh), whole.aggregate(b["indptr"], b["indices_global"]))
        assert torch.equal(sm.decode_rows(dst), whole.decode_rows(b["dst_nodes"]))
        torch.cuda.synchronize()
        peers.close()
        vq_peers = sage.PeerCompressionManager(D, ["vq"], [(32, 8)], [vq_cbs], [vq_codes[lo:hi].clone()], [n])
        ref_vq = sage.CompressionManager(D, ["vq"], [(32, 8)], [vq_cbs], [vq_codes])
        assert torch.equal(vq_peers.aggregate(b["indptr"], b["indices_global"]), ref_vq.aggregate(b["indptr"], b["indices_global"]))
        torch.cuda.synchronize()
        vq_peers.close()
        # single-level table through the same path
        one = sage.ShardedCompressionManager(D, ["vq"], [(32, 8)], [vq_cbs], [vq_codes[lo:hi].clone()], [n])
        sm, neigh, dst = one.for_block(b)
        ref = sage.CompressionManager(D, ["vq"], [(32, 8)], [vq_cbs], [vq_codes])
        assert torch.equal(sm.aggregate(b["indptr"], neigh), ref.aggregate(b["indptr"], b["indices_global"]))
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, repr(e) + traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_sharded_compression_manager_equals_resident_tables(world):
    """Row-sharded tables + all-to-all row fetch feed the fused two-level kernel the same rows as the resident tables."""
    if torch.cuda.device_count() < world:
        pytest.skip("needs more GPUs")
    _run(_manager_worker, world)


def _compress_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from f2cgt_b200 import compress
        g = torch.Generator(device=device).manual_seed(9)  # the same features on every rank
        n, D = 30001, 128
        protos = torch.randn(4, 64, 32, generator=g, device=device) * 2
        which = torch.randint(0, 64, (n, 4), generator=g, device=device)
        x = torch.cat([protos[s][which[:, s]] for s in range(4)], dim=1) + 0.05 * torch.randn(n, D, generator=g, device=device)
        seeds = torch.randperm(n, generator=g, device=device)[:700]
        for kw in (dict(target_compression_ratio=8), dict(target_compression_ratio=128, seeds=seeds, max_iter=10)):
            split = compress.compress(x, group=dist.group.WORLD, **kw)               # column slices / row ranges per rank
            single = compress.compress(x, world_size=world, **kw)                     # the same artefact in one process
            assert split["methods"] == single["methods"] and split["configs"] == single["configs"]
            for a, b in zip(split["codebooks"], single["codebooks"]):
                assert torch.equal(a, b), "codebooks differ"
            assert torch.equal(split["compression_data"], single["compression_data"])
            if "seeds" in kw:
                assert torch.equal(split["seeds_compression_data"], single["seeds_compression_data"])
            shard_only = compress.compress(x, group=dist.group.WORLD, gather=False, **kw)
            lo, hi = shard_only["row_range"]
            assert torch.equal(shard_only["compression_data"], single["compression_data"][lo:hi])
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, repr(e) + traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


def test_compressor_rank_split_two_gpus():
    """The offline compressor split over two ranks (examples/process_compress.py:82-107,192-196,225,236-238) writes the
    artefact one process writes."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(_compress_worker, 2)
