"""Benchmark of the fused decompress + mean-aggregation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (both arms, identical inputs): the packed low-bit SQ configuration - a 2,449,029 x 128 feature table stored
as 1-, 2- and 4-bit log-domain SQ codes of N(0,1) features, a synthetic power-law graph (Zipf 2.1 degrees, mean 50),
six minibatches of 1024 seeds with fan-out 12,12,12.  Graph, tables and the six outermost blocks (the ones the fused
first GraphSAGE layer sees: ~7 * 10^4 destination rows, ~8 * 10^5 edges) come from ONE seeded CPU generator
(`cpu_workload`, cached on disk between the two arms); the GPU arm uploads them.  One STEP aggregates one block with
the fused kernel once per code width (three launches), gathering rows straight from the HBM-resident table by
global id.  Successive steps rotate through the six blocks and L2 is flushed between steps (outside the event pair).

Prints ONE JSON line (rank 0).  `value` = sampled edges aggregated per second by the whole job with all inputs
resident in HBM; at N > 1 the table is ROW-SHARDED over the GPUs (1/N of the rows each, plus the 5 % most often sampled
rows on every GPU) and the kernel reads remote rows over NVLink; the purely sharded, the replicated and the NCCL
all-to-all placements are timed beside it.  `e2e` = the same work called
through the public module with the block's CSC in pinned host memory and the aggregated rows read back to the host
inside the timed region.  `epoch` = GraphSAGE training (3 layers, two-level table) seconds per epoch, replicated and
sharded table.  `--impl reference` times the reference's PyTorch CPU path (oracle/torch_cpu_path.py) on the same
blocks and tables on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NUM_NODES = 2_449_029
FEAT_DIM = 128
AVG_DEGREE = 50
ZIPF = 2.1
BATCH = 1024
FAN_OUT = (12, 12, 12)
BITS = (1, 2, 4)
COLUMN_SLICE = 128
N_MINIBATCHES = 6
HOT_REPLICATED = 0.05  # share of the rows (the most often sampled ones) every GPU keeps beside its shard of the rest
METRIC = "fused_sq_decompress_spmm_sampled_edges_per_s"
WORKLOAD = ("SQ 1/2/4-bit packed table 2449029x128 (N(0,1) features), power-law graph (Zipf 2.1, mean degree 50), "
            "6 minibatches of 1024 seeds x fan-out 12,12,12, outermost block, all three widths per step; graph, tables and "
            "blocks from one seeded CPU generator")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the 4-bit kernel on a block of this generator, from an ncu
# capture (not measured in this run); below the algorithmic bytes because the output is still dirty in L2 at kernel end
NCU_DRAM_TRAFFIC_BYTES_SQ4 = 49.8e6


def algorithmic_bytes(n_edges, n_dst, row_bytes, idx_bytes, feat_dim, codebook_bytes):
    """E*(row_bytes + idx_bytes) + (n_dst+1)*ptr_bytes + n_dst*D*4 + codebook bytes."""
    return n_edges * (row_bytes + idx_bytes) + (n_dst + 1) * idx_bytes + n_dst * feat_dim * 4 + codebook_bytes


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------- shared workload
def cpu_workload(need_graph=False):
    """Graph, SQ tables (1/2/4 bits) and the six outermost blocks, generated on the CPU from seed 0 with torch's CPU
    generator, the oracle's compressor and the oracle's neighbour sampler.  Both arms call this; the result is cached
    on disk (plain .npy files) so that the second arm on a box only reads it back.  Returns numpy arrays."""
    import numpy as np
    cache = os.environ.get("F2CGT_BENCH_CACHE", "/tmp/f2cgt_b200_bench_workload_v3")
    done = os.path.join(cache, "done")
    names = [f"codes{b}" for b in BITS] + ["codebook"] + [f"blk{i}_{k}" for i in range(N_MINIBATCHES) for k in ("indptr", "indices")]

    def load(with_graph):
        w = {n: np.load(os.path.join(cache, n + ".npy"), mmap_mode="r") for n in names}
        if with_graph:
            w["graph_indptr"] = np.load(os.path.join(cache, "graph_indptr.npy"), mmap_mode="r")
            w["graph_indices"] = np.load(os.path.join(cache, "graph_indices.npy"), mmap_mode="r")
        return w

    if os.path.exists(done):
        try:
            return load(need_graph)
        except Exception:  # noqa: BLE001
            pass
    import torch
    from oracle import oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator(); g.manual_seed(0)
    u = torch.rand(NUM_NODES, generator=g, dtype=torch.float64).clamp_min(1e-12)
    raw = u.pow(-1.0 / (ZIPF - 1.0)).clamp_max(NUM_NODES // 20)
    deg = torch.floor(raw * (AVG_DEGREE / float(raw.mean()))).to(torch.int64)
    indptr = torch.zeros(NUM_NODES + 1, dtype=torch.int64)
    torch.cumsum(deg, 0, out=indptr[1:])
    nnz = int(indptr[-1])
    indices = torch.empty(nnz, dtype=torch.int64)
    for s in range(0, nnz, 1 << 25):
        e = min(s + (1 << 25), nnz)
        indices[s:e] = torch.searchsorted(indptr, torch.randint(0, nnz, (e - s,), generator=g), right=True) - 1
    ip_np, ix_np = indptr.numpy(), indices.numpy()
    # tables: codes of N(0,1) features, encoded chunk-wise with the oracle's compressor
    sample = torch.randn((250_000, FEAT_DIM), generator=g).numpy()
    cb = O.sq_codebooks(sample, COLUMN_SLICE)
    tables = {b: [] for b in BITS}
    for s in range(0, NUM_NODES, 1 << 18):
        x = torch.randn((min(1 << 18, NUM_NODES - s), FEAT_DIM), generator=g).numpy()
        for b in BITS:
            tables[b].append(O.sq_codes_to_storage(O.sq_compress(x, cb, b, COLUMN_SLICE), b))
    w = {f"codes{b}": np.concatenate(v).view(np.uint8) for b, v in tables.items()}
    w["codebook"] = cb
    # minibatch blocks with the oracle's sampler: hops in reversed(fan_out) order, frontier = [frontier, new nodes]
    for mb in range(N_MINIBATCHES):
        frontier = torch.randperm(NUM_NODES, generator=g)[:BATCH].numpy()
        for hop, pick in enumerate(reversed(FAN_OUT)):
            sip, six = O.sample_neighbors(ip_np, ix_np, frontier, pick, mb, hop)
            if hop == len(FAN_OUT) - 1:
                w[f"blk{mb}_indptr"], w[f"blk{mb}_indices"] = sip, six
            else:
                fresh = np.setdiff1d(np.unique(six), frontier)
                frontier = np.concatenate([frontier, fresh])
    try:
        os.makedirs(cache, exist_ok=True)
        for n in names:
            np.save(os.path.join(cache, n + ".npy"), np.ascontiguousarray(w[n]))
        np.save(os.path.join(cache, "graph_indptr.npy"), ip_np)
        np.save(os.path.join(cache, "graph_indices.npy"), ix_np)
        open(done, "w").write("ok")
    except OSError:
        pass  # no cache: the next arm generates again
    if need_graph:
        w["graph_indptr"], w["graph_indices"] = ip_np, ix_np
    return w


def shared_config(w):
    n_edges = statistics.mean(int(w[f"blk{i}_indices"].shape[0]) for i in range(N_MINIBATCHES))
    n_dst = statistics.mean(int(w[f"blk{i}_indptr"].shape[0]) - 1 for i in range(N_MINIBATCHES))
    return {"workload": WORKLOAD, "edges_per_block": int(n_edges), "dst_rows_per_block": int(n_dst), "index_dtype": "int64",
            "minibatches_rotated": N_MINIBATCHES}


# --------------------------------------------------------------------------------------------- ours
def build_workload(device, rank, world, dist):
    """Tables and blocks on the device.  Rank 0 holds the CPU generator's six blocks; at N > 1 every other rank draws
    its own six minibatches from the same (uploaded) graph with the GPU sampler (data parallel: own seeds per rank)."""
    import numpy as np
    import torch
    from f2cgt_b200 import synth
    if world > 1:
        if rank == 0:
            cpu_workload(need_graph=True)  # fill the cache once; the other ranks read it after the barrier
        dist.barrier()
    w = cpu_workload(need_graph=world > 1 and rank != 0)
    cb = torch.from_numpy(np.array(w["codebook"])).to(device)
    tables = {b: (torch.from_numpy(np.array(w[f"codes{b}"])).to(device).view(torch.int8), cb) for b in BITS}
    blocks, extra = [], []
    if rank == 0:
        for i in range(N_MINIBATCHES):
            blocks.append((torch.from_numpy(np.array(w[f"blk{i}_indptr"])).to(device), torch.from_numpy(np.array(w[f"blk{i}_indices"])).to(device)))
    else:
        indptr = torch.from_numpy(np.array(w["graph_indptr"])).to(device)
        indices = torch.from_numpy(np.array(w["graph_indices"])).to(device)
        g = torch.Generator(device=device)
        g.manual_seed(1000 + rank)
        for b in range(N_MINIBATCHES):
            seeds = torch.randperm(NUM_NODES, generator=g, device=device)[:BATCH]
            blk = synth.sample_blocks(indptr, indices, seeds, FAN_OUT, rng_seed=rank * 1000 + b)[0]
            blocks.append((blk["indptr"].contiguous(), blk["indices_global"].contiguous()))
        del indptr, indices
        torch.cuda.empty_cache()
    if world > 1:  # what the all-to-all placement needs: the block's distinct source rows and block-local ids
        from f2cgt_b200 import ops
        for ip, ix in blocks:
            src, (local,) = ops.tensor_relabel([ix])
            extra.append((src.contiguous(), local.contiguous()))
    return w, tables, blocks, extra


def time_steps(step_fn, blocks, steps, warmup, flush, torch):
    """Per-step CUDA events on the current stream; returns (sum of step ms, edges done)."""
    for w in range(warmup):
        step_fn(w % len(blocks))
        flush.sum()
    torch.cuda.synchronize()
    ms, edges = [], 0
    for s in range(steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(250_000)
        a.record()
        step_fn(s % len(blocks))
        b.record()
        flush.sum()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
        edges += blocks[s % len(blocks)][1].numel() * len(BITS)
    return sum(ms), edges


def sharded_placements(args, capi, tables, blocks, extra, flush, device, rank, world, torch, dist):
    """Row-sharded table at N > 1: the fused kernel reading remote rows over NVLink (peer mappings), and the NCCL
    all-to-all fetch followed by the kernel on block-local rows.  Each is checked once against the replicated table."""
    from f2cgt_b200 import ops, shard
    out = {}
    lo, hi = shard.shard_bounds(NUM_NODES, world, rank)
    shards = {b: tables[b][0][lo:hi].contiguous() for b in BITS}
    try:
        peers = {b: shard.PeerTable(shards[b], NUM_NODES) for b in BITS}

        def step_peer(i):
            ip, ix = blocks[i]
            for b in BITS:
                ops.sq_decompress_spmm_csr_peer(peers[b], tables[b][1], ip, ix, b, COLUMN_SLICE, FEAT_DIM)
        out["sharded_peer_loads"] = time_steps(step_peer, blocks, args.steps, args.warmup, flush, torch)
        ip, ix = blocks[0]
        for b in BITS:
            a = ops.sq_decompress_spmm_csr_peer(peers[b], tables[b][1], ip, ix, b, COLUMN_SLICE, FEAT_DIM)
            ref = capi.sq_decompress_spmm_csr(tables[b][0], tables[b][1], ip, ix, b, COLUMN_SLICE, FEAT_DIM)
            assert torch.equal(a, ref), f"peer-load result differs from the replicated table at {b} bits"
    except Exception as e:  # noqa: BLE001
        out["sharded_peer_loads_error"] = repr(e)[:300]
    # The same partitioning with the HOT_REPLICATED most often sampled rows on every GPU (the reference's loader ranks
    # nodes by a presampling pass and caches the hottest per GPU: examples/dataloader.py:234-260,273-304; here the rank is
    # the in-degree, which is what the synthetic graph's sampling probability follows).  The table is numbered hot rows
    # first - a one-off relabelling of graph, table and block indices outside the timed region.
    try:
        import numpy as np
        deg = torch.from_numpy(np.diff(np.asarray(cpu_workload(need_graph=True)["graph_indptr"]))).to(device)
        order = torch.argsort(deg, descending=True, stable=True)          # new id -> old id
        new_id = torch.empty_like(order)
        new_id[order] = torch.arange(NUM_NODES, device=device)            # old id -> new id
        n_rep = int(NUM_NODES * args.hot_replicated)
        n_rep += (NUM_NODES - n_rep) % world                               # equal shards of the remainder
        cold = NUM_NODES - n_rep
        rps = shard.rows_per_rank(cold, world)
        # ids of the sharded rows start at the next multiple of the shard size (one division locates any row), and
        # the remainder is dealt round-robin over the shards (by blocks it would leave the warmest rows to shard 0)
        first_cold = ops.peer_first_cold_id(n_rep, rps)
        c = new_id - n_rep
        new_id = torch.where(new_id < n_rep, new_id, first_cold + (c % world) * rps + torch.div(c, world, rounding_mode="floor"))
        heads, tails = {}, {}
        for b in BITS:
            renumbered = tables[b][0][order]
            heads[b] = renumbered[:n_rep].contiguous()
            tails[b] = shard.PeerTable(renumbered[n_rep + rank::world].contiguous(), cold)
            del renumbered
        blocks_hot_first = [(ip, new_id[ix]) for ip, ix in blocks]
        mine_lo = first_cold + rank * rps
        remote = sum(int(((ix >= first_cold) & ((ix < mine_lo) | (ix >= mine_lo + rps))).sum()) for _, ix in blocks_hot_first)
        out["hot_replicated_remote_edge_share"] = remote / max(sum(ix.numel() for _, ix in blocks), 1)

        def step_hot(i):
            ip, ix = blocks_hot_first[i]
            for b in BITS:
                ops.sq_decompress_spmm_csr_peer(tails[b], tables[b][1], ip, ix, b, COLUMN_SLICE, FEAT_DIM, replicated=heads[b])
        out["sharded_peer_loads_hot_replicated"] = time_steps(step_hot, blocks, args.steps, args.warmup, flush, torch)
        ip, ix = blocks_hot_first[0]
        for b in BITS:
            a = ops.sq_decompress_spmm_csr_peer(tails[b], tables[b][1], ip, ix, b, COLUMN_SLICE, FEAT_DIM, replicated=heads[b])
            ref = capi.sq_decompress_spmm_csr(tables[b][0], tables[b][1], blocks[0][0], blocks[0][1], b, COLUMN_SLICE, FEAT_DIM)
            assert torch.equal(a, ref), f"hot-replicated peer-load result differs from the replicated table at {b} bits"
    except Exception as e:  # noqa: BLE001
        out["sharded_peer_loads_hot_replicated_error"] = repr(e)[:300]
    try:
        st = {b: shard.ShardedTable(shards[b], NUM_NODES) for b in BITS}
        # the id exchange happens when the block is sampled, and so does the renumbering of the block's indices to the
        # order in which the fetched rows arrive (rows are then used where the exchange puts them, no un-sorting pass)
        plans = [st[BITS[0]].plan(src) for src, _ in extra]
        ix_arrival = [plans[i]["position"][extra[i][1]] for i in range(len(extra))]

        def step_a2a(i):
            ip, _ = blocks[i]
            for b in BITS:
                rows = st[b].fetch_rows(plans[i], ordered=False)
                capi.sq_decompress_spmm_csr(rows, tables[b][1], ip, ix_arrival[i], b, COLUMN_SLICE, FEAT_DIM)
        out["sharded_nccl_all_to_all"] = time_steps(step_a2a, blocks, args.steps, args.warmup, flush, torch)
        rows = st[4].fetch_rows(plans[0], ordered=False)
        a = capi.sq_decompress_spmm_csr(rows, tables[4][1], blocks[0][0], ix_arrival[0], 4, COLUMN_SLICE, FEAT_DIM)
        ref = capi.sq_decompress_spmm_csr(tables[4][0], tables[4][1], blocks[0][0], blocks[0][1], 4, COLUMN_SLICE, FEAT_DIM)
        assert torch.equal(a, ref), "all-to-all result differs from the replicated table"
    except Exception as e:  # noqa: BLE001
        out["sharded_nccl_all_to_all_error"] = repr(e)[:300]
    return out


def parity_check(capi, tables, blocks, torch):
    """Block 0 of the timed workload (global-id gathers into the 2.45 M-row table, ~0.8 M power-law edges): every width
    against the reference's own CUDA kernel when its build is present, else against decode-then-aggregate of the block's
    distinct source rows with this library's unfused operators (the reference's own test property)."""
    from f2cgt_b200 import ops
    out = {}
    ip, ix = blocks[0]
    try:
        from oracle import build_ref
        ref = build_ref.load()
    except Exception:  # noqa: BLE001
        ref = None
    src, (local,) = ops.tensor_relabel([ix])
    for bits in BITS:
        codes, cb = tables[bits]
        got = capi.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
        unfused = capi.spmm_csr(capi.sq_decompress(codes[src].contiguous(), cb, bits, COLUMN_SLICE, FEAT_DIM), ip, local)
        ok = torch.equal(got, unfused)
        how = "bit-exact vs decode-then-aggregate"
        if ref is not None:
            want = ref.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
            torch.cuda.synchronize()
            ok = ok and torch.equal(got, want)
            how = "bit-exact vs the reference's CUDA kernel and vs decode-then-aggregate"
        out[f"sq{bits}"] = how if ok else "MISMATCH"
    return out


def two_level_parity(torch):
    """The two-level single launch on a block of the same shape against its composition (decode every source row by its
    own codec with the unfused operators, then the plain mean): bit-equal."""
    from f2cgt_b200 import ops, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    n = 200_000
    indptr, indices = synth.power_law_graph(n, 50, 2.1, seed=3, device=dev)
    g = torch.Generator(device=dev); g.manual_seed(7)
    seeds = torch.randperm(n, generator=g, device=dev)[:1024]
    blk = synth.sample_blocks(indptr, indices, seeds, FAN_OUT, rng_seed=3)[0]
    ip, ix = blk["indptr"].contiguous(), blk["indices_global"].contiguous()
    vq = torch.randint(0, 256, (n, 4), generator=g, dtype=torch.uint8, device=dev)
    cbs = torch.randn(4, 256, 32, generator=g, device=dev)
    deg = indptr[1:] - indptr[:-1]
    hot = torch.topk(deg, n // 20).indices
    slot = torch.full((n,), -1, dtype=torch.int32, device=dev)
    slot[hot] = torch.arange(hot.numel(), dtype=torch.int32, device=dev)
    sq_hot, sq_cb = synth.sq_table_from_normal(hot.numel(), FEAT_DIM, 8, FEAT_DIM, seed=1, device=dev)
    got = ops.two_level_decompress_spmm_csr(sq_hot, sq_cb, 8, FEAT_DIM, vq, cbs, slot, ip, ix, FEAT_DIM)
    full = ops.vq_decompress(vq, cbs, FEAT_DIM)
    full[hot] = ops.sq_decompress(sq_hot, sq_cb, 8, FEAT_DIM, FEAT_DIM)
    return "bit-exact vs composition of the unfused decoders + spmm_csr" if torch.equal(got, ops.spmm_csr(full, ip, ix)) else "MISMATCH"


def run_ours(args):
    import torch
    import torch.distributed as dist
    import F2CGTLib as capi

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    w, tables, blocks, extra = build_workload(device, rank, world, dist)
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=device)  # 256 MiB, read (not written) to evict L2

    def step_device(i):
        ip, ix = blocks[i]
        for bits in BITS:
            codes, cb = tables[bits]
            capi.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)

    # ---- replicated table, device-resident: per-step and per-kernel CUDA events on the launching (current) stream
    for wu in range(args.warmup):
        step_device(wu % len(blocks))
        flush.sum()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    step_ms, kern_ms = [], {b: [] for b in BITS}
    edges_done = 0
    wall0 = time.perf_counter()
    for s in range(args.steps):
        ip, ix = blocks[s % len(blocks)]
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(BITS) + 1)]
        # park the GPU for ~0.1 ms so that the host has queued the step's launches before the first event
        # fires: the events then bracket device time only, not the Python launch path
        torch.cuda._sleep(250_000)
        evs[0].record()
        for j, bits in enumerate(BITS):
            codes, cb = tables[bits]
            capi.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
            evs[j + 1].record()
        flush.sum()  # evict the table and the block from L2 before the next step (clean lines: no write-backs later)
        torch.cuda.synchronize()
        step_ms.append(evs[0].elapsed_time(evs[-1]))
        for j, bits in enumerate(BITS):
            kern_ms[bits].append(evs[j].elapsed_time(evs[j + 1]))
        edges_done += ix.numel() * len(BITS)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - wall0
    total_ms = sum(step_ms)

    # ---- end to end through the public module with HOST buffers: pinned CSC in, aggregated rows out
    host_blocks = [(ip.cpu().pin_memory(), ix.cpu().pin_memory()) for ip, ix in blocks]
    max_dst = max(ip.numel() - 1 for ip, _ in blocks)
    # Two result sets in pinned memory: the results of step i travel to the host (copy stream, D2H engine) while step
    # i + 1 uploads its block and aggregates (compute stream, H2D engine); the host waits for step i's results before it
    # queues step i + 2.  Every step still uploads its own inputs and delivers all of its own results to the host.
    host_out = [[torch.empty((max_dst, FEAT_DIM), dtype=torch.float32).pin_memory() for _ in BITS] for _ in range(2)]
    e2e_steps = max(3, min(args.steps, 10))
    copy_stream = torch.cuda.Stream(device=device)
    delivered = [torch.cuda.Event(), torch.cuda.Event()]

    def step_e2e(hb, slot):
        hip, hix = hb
        ip = hip.to(device, non_blocking=True)
        ix = hix.to(device, non_blocking=True)
        n_dst = hip.numel() - 1
        for j, bits in enumerate(BITS):
            codes, cb = tables[bits]
            out = capi.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
            ready = torch.cuda.Event()
            ready.record()
            copy_stream.wait_event(ready)
            with torch.cuda.stream(copy_stream):
                host_out[slot][j][:n_dst].copy_(out, non_blocking=True)
            out.record_stream(copy_stream)
        delivered[slot].record(copy_stream)
        return (hip.numel() + hix.numel()) * 8, n_dst * FEAT_DIM * 4 * len(BITS), hix.numel() * len(BITS)

    for wu in range(2):
        step_e2e(host_blocks[wu % len(host_blocks)], wu % 2)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h2d = d2h = e2e_edges = 0
    for s in range(e2e_steps):
        a, b, c = step_e2e(host_blocks[s % len(host_blocks)], s % 2)
        h2d += a; d2h += b; e2e_edges += c
        if s >= 1:
            delivered[(s - 1) % 2].synchronize()  # the previous step's rows are on the host
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    # ---- aggregate over ranks: max time, summed edges
    def reduce_rate(ms, edges):
        if world == 1:
            return edges / (ms * 1e-3)
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        e = torch.tensor([float(edges)], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX); dist.all_reduce(e, op=dist.ReduceOp.SUM)
        return float(e[0]) / (float(t[0]) * 1e-3)

    placements = {"replicated": reduce_rate(total_ms, edges_done)}
    e2e_rate = reduce_rate(e2e_s * 1e3, e2e_edges)
    value, value_ms, placement_of_value = placements["replicated"], total_ms, "replicated (one GPU holds the whole table)"
    if world > 1:
        raw = sharded_placements(args, capi, tables, blocks, extra, flush, device, rank, world, torch, dist)
        names = ("sharded_peer_loads_hot_replicated", "sharded_peer_loads", "sharded_nccl_all_to_all")
        for name in names:
            ok = torch.tensor([1.0 if name in raw else 0.0], dtype=torch.float64, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok[0]) == 1.0:
                placements[name] = reduce_rate(*raw[name])
            elif rank == 0 and name + "_error" in raw:
                placements[name + "_error"] = raw[name + "_error"]
        if "hot_replicated_remote_edge_share" in raw:
            share = torch.tensor([raw["hot_replicated_remote_edge_share"]], dtype=torch.float64, device=device)
            dist.all_reduce(share, op=dist.ReduceOp.MAX)
            placements["hot_replicated_remote_edge_share"] = float(share[0])
        # The headline at N > 1 is a placement in which the table is really partitioned: every GPU holds 1/N of the rows
        # and, in the first choice, the HOT_REPLICATED hottest rows besides.
        what = {
            "sharded_peer_loads_hot_replicated": f"row-sharded over the GPUs with the {args.hot_replicated:.0%} most often sampled rows on every GPU "
                                                 f"({args.hot_replicated:.0%} + {1 - args.hot_replicated:.0%} / N of the table per GPU); the fused kernel reads "
                                                 "the remaining remote rows over NVLink (peer mappings, no collective)",
            "sharded_peer_loads": "row-sharded over the GPUs (1/N of the table per GPU), the fused kernel reads remote rows over NVLink "
                                  "(peer mappings, no collective)",
            "sharded_nccl_all_to_all": "row-sharded over the GPUs, rows fetched with an NCCL all-to-all before the fused kernel",
        }
        for name in names:
            if name in placements:
                value = placements[name]
                tmax = torch.tensor([raw[name][0]], dtype=torch.float64, device=device)
                dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
                value_ms = float(tmax[0])
                placement_of_value = what[name]
                break

    # ---- GraphSAGE epoch (second half of the metric): replicated and sharded table, same process group
    epoch = []
    if not args.no_epoch:
        from f2cgt_b200 import train_graphsage
        del flush
        torch.cuda.empty_cache()
        # every rank on its own share of the node's CPUs from here on (the training threads start below and inherit it)
        pinned = train_graphsage.pin_rank_cpus(local_rank, int(os.environ.get("LOCAL_WORLD_SIZE", world)))
        what = {
            "small": ("2,449,029 nodes, mean degree 50", "two-level: hot 5 % SQ 8 bits + VQ 4 x 32 (ratio 128), D = 128, 172 classes, 122,880 "
                      "training ids split over the ranks, batch 1024, fan-out 12,12,12, dropout 0.5"),
            "config4": ("111,059,956 nodes, mean degree 14.4 (1.6 G edges, int64 CSC replicated per GPU)", "two-level: hot 5 % SQ 8 bits + VQ 4 x 32, "
                        "D = 128, 172 classes, 1.2 M training ids split over the ranks, batch 1024, fan-out 12,12,12, dropout 0.5"),
            "config5": ("65,608,366 nodes, mean degree 54.9 (3.6 G edges, int64 CSC replicated per GPU)", "two-level: hot 2 % SQ 4 bits + VQ 4 x 64, "
                        "D = 256, 64 classes, 1.2 M training ids split over the ranks, batch 1024 per GPU, fan-out 15,10,5, dropout 0.5"),
        }
        # the 2.45 M-node graph with every table placement, then the two large configurations of the metric with the
        # placement a deployment would use (replicated on one GPU, row-sharded with peer loads on several)
        runs = [("small", t, dict(epochs=2, min_timed_steps=100)) for t in ("replicated", "sharded_peer", "sharded") if t == "replicated" or world > 1]
        runs += [(ps, "replicated" if world == 1 else "sharded_peer", dict(epochs=2)) for ps in ("config4", "config5")]
        for preset, table, kw in runs:
            try:
                rec = train_graphsage.train(preset, table, rank, world, local_rank, **kw)
                epoch.append({"preset": preset, "table": table, "ms_per_step": rec["ms_per_step"], "s_per_epoch": rec["value"],
                              "steps": rec["steps_per_epoch_per_gpu"], "timed_steps": rec["timed_steps_per_gpu"],
                              "breakdown_ms": rec["breakdown_ms"], "precision": rec["precision"],
                              "blocks_built_ahead": rec["blocks_built_ahead"], "cpus_per_rank": len(pinned) if pinned else os.cpu_count(),
                              "graph": what[preset][0], "codecs": what[preset][1]})
            except Exception as e:  # noqa: BLE001
                epoch.append({"preset": preset, "table": table, "error": repr(e)[:300]})
            torch.cuda.empty_cache()
        flush = torch.zeros(64 << 20, dtype=torch.float32, device=device)

    if rank == 0:
        peak, peak_kind = measured_peak()
        cfg = shared_config(w)
        n_edges = statistics.mean(ix.numel() for _, ix in blocks)
        n_dst = statistics.mean(ip.numel() - 1 for ip, _ in blocks)
        variants = {}
        for bits in BITS:
            row_bytes = FEAT_DIM * bits // 8
            byts = algorithmic_bytes(n_edges, n_dst, row_bytes, 8, FEAT_DIM, 20)
            ms = statistics.mean(kern_ms[bits])
            variants[f"sq{bits}"] = {"ms": round(ms, 5), "edges_per_s": n_edges / (ms * 1e-3), "algorithmic_bytes": int(byts),
                                     "gbs": byts / (ms * 1e-3) / 1e9, "frac_of_peak": byts / (ms * 1e-3) / 1e9 / peak}
        dom = variants["sq4"]
        parity = parity_check(capi, tables, blocks, torch)
        try:
            parity["two_level_sq8_vq4x32"] = two_level_parity(torch)
        except Exception as e:  # noqa: BLE001
            parity["two_level_sq8_vq4x32"] = "not run: " + repr(e)[:120]
        from f2cgt_b200 import ops
        parity["device_status"] = ops.device_status()
        line = {
            "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": value_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8 codes -> f32", "data": "synthetic", "config": cfg,
            "arm_details": {
                "gather": "global ids into the HBM-resident table", "table_placement_of_value": placement_of_value,
                "l2": "256 MiB read sweep between steps (outside the step's event pair) evicts L2; tables 39/78/157 MB",
                "timing": "CUDA events on the launching stream, max over ranks; one fused launch per width per step",
                "kernels": "sq_spmm_kernel<1>, sq_stream_kernel<2>, sq_spmm_kernel<4> (library's choice per width)"},
            "roofline": {"bound": "hbm", "kernel": "sq_spmm_kernel<4-bit> (replicated table, one GPU)", "achieved": dom["gbs"], "peak": peak,
                         "unit": "GB/s", "frac": dom["frac_of_peak"], "traffic": NCU_DRAM_TRAFFIC_BYTES_SQ4,
                         "traffic_unit": "bytes/launch: ncu dram read+write of one 4-bit launch on a block of this generator, from an "
                                         "earlier capture, not measured in this run", "algorithmic_bytes": dom["algorithmic_bytes"],
                         "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})"},
            "variants": variants,
            "e2e": {"value": e2e_rate, "unit": "edges/s", "h2d_bytes_per_step": h2d // e2e_steps,
                    "d2h_bytes_per_step": d2h // e2e_steps, "steps": e2e_steps,
                    "what": "pinned-host CSC -> device, 3 fused launches via F2CGTLib (replicated table), aggregated rows -> pinned host; "
                            "a step's result copy overlaps the next step's upload and launches (two result sets)"},
            "gpu_launches": args.steps * len(BITS), "table_placements_edges_per_s": placements, "parity_check": parity,
            "epoch": epoch, "clocks": clocks, "wall_s_timed_region": wall,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_leg(w, steps=1, warmup=1)
        if world == 1:
            line["reference_cuda_kernels"] = reference_cuda_leg(tables, blocks, flush)
            line["other_fused_kernels"] = other_kernels_leg()
        emit(line)
        if any(v == "MISMATCH" for v in parity.values()):
            sys.stderr.write("bench.py: parity check failed\n")
            sys.exit(1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def other_kernels_leg():
    """The VQ and two-level fused kernels on the same kind of block (f2cgt_b200.kernel_bench cases, CUDA events, cold L2),
    reported beside the headline: they are not part of `value`."""
    try:
        import argparse as _ap
        from f2cgt_b200 import kernel_bench
        b = kernel_bench.Bench(_ap.Namespace(only="vq_spmm,two_level", reps=10, small=False, launches=0, json="", kernel="auto"))
        kernel_bench.cases(b)
        return [{k: r[k] for k in ("kernel", "ms", "algorithmic_bytes", "gbs", "frac_of_hbm_peak", "edges_per_s", "note") if k in r}
                for r in b.rows]
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:200]}


def reference_cuda_leg(tables, blocks, flush):
    """The reference's own CUDA kernel for the same op on the same GPU and block (extension built from its sources by
    oracle/build_ref.py), timed like ours: CUDA events on the stream it launches on (the legacy default stream, which
    is torch's current stream here), cold L2, launch path hidden behind a parked GPU; its output allocation
    (torch::zeros, a memset on the same stream) is part of its operator and inside the events."""
    import torch
    try:
        from oracle import build_ref
        ref = build_ref.load()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": str(e)[:200]}
    out = {}
    ip, ix = blocks[0]
    for bits in BITS:
        codes, cb = tables[bits]
        for _ in range(2):  # also pre-touches the caching allocator for the output shape
            ref.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
            flush.sum()
        torch.cuda.synchronize()
        ms = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(250_000)
            a.record()
            ref.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
            b.record()
            flush.sum()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        out[f"sq{bits}_ms"] = statistics.median(ms)
    out["note"] = "CUDA events on its (legacy default) stream, cold L2, block 0, includes its zero-fill of the output"
    return out


# --------------------------------------------------------------------------------------------- CPU
def cpu_tables(w):
    import numpy as np
    import torch
    cb = torch.from_numpy(np.array(w["codebook"]))
    return {b: (torch.from_numpy(np.array(w[f"codes{b}"])), cb) for b in BITS}


def cpu_blocks(w):
    import numpy as np
    import torch
    return [(torch.from_numpy(np.array(w[f"blk{i}_indptr"])), torch.from_numpy(np.array(w[f"blk{i}_indices"]))) for i in range(N_MINIBATCHES)]


def cpu_leg(w, steps, warmup):
    """Reference PyTorch CPU path on block 0, all three widths per step."""
    import torch
    from oracle import torch_cpu_path as T
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tables_host = cpu_tables(w)
    ip, ix = cpu_blocks(w)[0]
    times = []
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        for bits in BITS:
            codes, cb = tables_host[bits]
            T.sq_spmm(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
        if s >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.mean(times)
    return {"value": ix.numel() * len(BITS) / sec, "unit": "edges/s", "cores": cores, "kind": "port",
            "sample": f"one full step (block 0, {ix.numel()} edges, widths 1/2/4), {steps} timed after {warmup} warm-up",
            "seconds_per_step": sec, "impl": "torch CPU: gather rows, shift/mask unpack, exp2 decode, sparse CSR mean matmul"}


def run_reference(args):
    """Reference arm: the reference's PyTorch-level CPU path (oracle/torch_cpu_path.py) on the same tables and the same
    six blocks as the GPU arm, all host threads; nothing of the CUDA library is loaded."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    import torch
    from oracle import torch_cpu_path as T
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = cpu_workload()
    tables_host = cpu_tables(w)
    blocks = cpu_blocks(w)
    times, edges = [], 0
    for s in range(args.warmup + args.steps):
        ip, ix = blocks[s % len(blocks)]
        t0 = time.perf_counter()
        for bits in BITS:
            codes, cbt = tables_host[bits]
            T.sq_spmm(codes, cbt, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
        if s >= args.warmup:
            times.append(time.perf_counter() - t0)
            edges += ix.numel() * len(BITS)
    total = sum(times)
    value = edges / total
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": int(os.environ.get("WORLD_SIZE", 1)),
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u8 codes -> f32", "data": "synthetic", "config": shared_config(w),
            "arm_details": {"what": "torch CPU: gather the block's distinct source rows, shift/mask unpack, exp2 decode, sparse CSR mean matmul"},
            "cpu_baseline": {"value": value, "unit": "edges/s", "cores": cores, "kind": "port",
                             "sample": "every step is one full block at all three widths (no sub-sampling)"},
            "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


_RESULT_FD = None


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode()); sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-epoch", action="store_true", help="skip the GraphSAGE epoch records")
    ap.add_argument("--hot-replicated", type=float, default=HOT_REPLICATED,
                    help="N > 1: share of the rows (the most often sampled ones) kept on every GPU beside its shard of the rest")
    args = ap.parse_args()
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the JSON line must be the only thing
    # on stdout, so everything else is sent to stderr and the line is written to the saved descriptor.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
