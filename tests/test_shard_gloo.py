"""CPU, two gloo ranks: the row-sharded table fetch (bucketing, count / id / row exchange, un-sorting)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from f2cgt_b200 import shard


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n_rows, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        table = torch.randint(0, 256, (n_rows, 16), generator=g, dtype=torch.uint8)  # same on every rank
        lo, hi = shard.shard_bounds(n_rows, world, rank)
        st = shard.ShardedTable(table[lo:hi].clone(), n_rows)
        g2 = torch.Generator().manual_seed(100 + rank)
        for n_ids in (0, 1, 257, 5000):
            ids = torch.randint(0, n_rows, (n_ids,), generator=g2)  # duplicates and any order
            rows = st.fetch(ids)
            assert rows.shape == (n_ids, 16) and torch.equal(rows, table[ids])
            # the same rows as they arrive (grouped by owner), found through the plan's positions
            plan = st.plan(ids)
            arrived = st.fetch_rows(plan, ordered=False)
            assert arrived.shape == (n_ids, 16) and torch.equal(arrived[plan["position"]], table[ids])
        # every id on one remote rank, and an id outside the table
        other = (rank + 1) % world
        olo, ohi = shard.shard_bounds(n_rows, world, other)
        ids = torch.arange(olo, ohi)
        assert torch.equal(st.fetch(ids), table[ids])
        try:
            st.plan(torch.tensor([n_rows]))
            ok = False
        except IndexError:
            ok = True
        assert ok
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [1001, 64])
def test_sharded_fetch_two_ranks(n_rows):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_rows, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_bucketing_is_stable_and_complete():
    ids = torch.tensor([5, 900, 3, 450, 901, 4, 0])
    order, sorted_ids, counts = shard.bucket_by_owner(ids, 300, 4)
    assert counts.tolist() == [4, 1, 0, 2]
    assert sorted_ids.tolist() == [5, 3, 4, 0, 450, 900, 901]  # grouped by owner, original order kept inside a group
    assert torch.equal(ids[order], sorted_ids)
    assert shard.shard_bounds(1001, 2, 0) == (0, 501) and shard.shard_bounds(1001, 2, 1) == (501, 1001)
    assert shard.shard_bounds(10, 4, 3) == (9, 10)


def _manager_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from f2cgt_b200 import sage
        n, n_hot = 5003, 611
        g = torch.Generator().manual_seed(3)  # the same tables on every rank
        vq = torch.randint(0, 256, (n, 4), generator=g, dtype=torch.uint8)
        hot_rows = torch.randint(-128, 128, (n_hot, 128), generator=g, dtype=torch.int8)
        slot = torch.full((n,), -1, dtype=torch.int32)
        slot[torch.randperm(n, generator=g)[:n_hot]] = torch.arange(n_hot, dtype=torch.int32)
        lo, hi = shard.shard_bounds(n, world, rank)
        hlo, hhi = shard.shard_bounds(n_hot, world, rank)
        cb = [torch.zeros(1, 5), torch.zeros(4, 256, 32)]
        parts = sage.ShardedCompressionManager(128, ["sq", "vq"], [(128, 8), (32, 8)], cb, [hot_rows[hlo:hhi].clone(), vq[lo:hi].clone()],
                                               [n_hot, n], slot[lo:hi].clone())
        g2 = torch.Generator().manual_seed(50 + rank)  # a different block per rank
        for n_src in (700, 1):
            src = torch.randperm(n, generator=g2)[:n_src]
            n_dst = min(50, n_src)
            ix = torch.randint(0, n_src, (40,), generator=g2)
            block = dict(src_nodes=src, dst_nodes=src[:n_dst], indices_local=ix)
            local, neigh, dst = parts.for_block(block)
            # fetched rows stay where the exchange put them; the block's indices and its destination ids are renumbered
            # to that order, so looking a node up through them finds the node's own rows
            assert torch.equal(local.tables[1][neigh], vq[src[ix]]) and torch.equal(local.tables[1][dst], vq[src[:n_dst]])
            assert sorted(dst.tolist() + [-1])[1:] == sorted(set(dst.tolist()))  # distinct positions
            order = torch.empty(n_src, dtype=torch.int64)   # arrival position -> block-local id
            for probe in (neigh, dst):
                assert int(probe.min()) >= 0 and int(probe.max()) < n_src
            full_pos = parts.level2.plan(src)["position"]   # (collective: every rank calls it)
            order[full_pos] = torch.arange(n_src)
            arrived = src[order]
            assert torch.equal(local.tables[1], vq[arrived])
            want_hot = slot[arrived] >= 0
            assert torch.equal(local.slot >= 0, want_hot)
            assert torch.equal(local.tables[0][local.slot[want_hot].long()], hot_rows[slot[arrived][want_hot].long()])
            assert local.tables[0].shape[0] == int(want_hot.sum())
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, repr(e) + traceback.format_exc()[-500:]))
    finally:
        dist.destroy_process_group()


def test_sharded_compression_manager_assembles_block_tables():
    """Two ranks: the block-local tables handed to the fused two-level kernel hold exactly the rows of the block's source
    nodes (VQ codes, slots re-numbered to the fetched hot rows)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_manager_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results == {0: "ok", 1: "ok"}, results


class _FakeShards:
    """Stand-in for the library's shard calls on CPU ranks: handles are made-up bytes, `fail` names the call that raises."""

    def __init__(self, fail=None):
        self.fail, self.log = fail, []

    def create(self, rows):
        if self.fail == "create":
            raise RuntimeError("out of memory (injected)")
        self.log.append("create")
        return 1000 + rows.shape[0], b"handle-%d" % rows.shape[0]

    def open(self, handle):
        if self.fail == "open":
            raise RuntimeError("cannot map (injected)")
        self.log.append("open")
        return 5000 + len(handle)

    def close(self, ptr):
        self.log.append("close")

    def free(self, ptr):
        self.log.append("free")


def _peer_error_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # an uneven table whose last shard is empty: 2 rows over 2 ranks of at least 2 rows each
        n_rows = 2
        lo, hi = shard.shard_bounds(n_rows, world, rank)
        assert (lo, hi) == ((0, 2) if rank == 0 else (2, 2))
        rows = torch.zeros((hi - lo, 16), dtype=torch.uint8)
        ok = shard.PeerTable(rows, n_rows, backend=_FakeShards())
        assert len(ok.pointers) == world and ok.shard_bytes == [32, 0]
        ok.close()
        assert ok.backend.log == ["create", "open", "close", "free"]
        # a failure on ONE rank is raised on EVERY rank, after the collectives (nobody hangs)
        for call in ("create", "open"):
            backend = _FakeShards(fail=call if rank == 1 else None)
            try:
                shard.PeerTable(rows, n_rows, backend=backend)
                raise AssertionError("no error raised")
            except RuntimeError as e:
                assert "rank 1" in str(e) and "injected" in str(e), str(e)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, repr(e) + traceback.format_exc()[-500:]))
    finally:
        dist.destroy_process_group()


def test_peer_table_raises_collectively_and_takes_empty_shards():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_peer_error_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results == {0: "ok", 1: "ok"}, results


def _split_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from f2cgt_b200 import compress
        # 5 column slices over 2 ranks: 3 + 2; 11 rows: 6 + 5 (examples/process_compress.py:192-196,236-238)
        (s_lo, s_hi), (r_lo, r_hi) = compress.split_plan(11, 5, world, rank)
        assert (s_lo, s_hi, r_lo, r_hi) == ((0, 3, 0, 6) if rank == 0 else (3, 5, 6, 11))
        # more ranks than slices: the last ranks own nothing
        assert compress.split_plan(11, 1, world, 1)[0] == (1, 1)
        part = torch.arange(s_lo, s_hi, dtype=torch.float32).reshape(-1, 1, 1).expand(-1, 2, 3).contiguous()
        whole = compress.gather_parts(part, dist.group.WORLD)
        assert whole.shape == (5, 2, 3) and torch.equal(whole[:, 0, 0], torch.arange(5, dtype=torch.float32))
        rows = torch.arange(r_lo, r_hi, dtype=torch.int8).reshape(-1, 1)
        assert torch.equal(compress.gather_parts(rows, dist.group.WORLD).reshape(-1), torch.arange(11, dtype=torch.int8))
        # a rank with nothing to contribute
        nothing = torch.zeros((0, 4)) if rank == 1 else torch.ones((2, 4))
        assert torch.equal(compress.gather_parts(nothing, dist.group.WORLD), torch.ones((2, 4)))
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, repr(e) + traceback.format_exc()[-500:]))
    finally:
        dist.destroy_process_group()


def test_compressor_split_plan_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_split_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results == {0: "ok", 1: "ok"}, results
