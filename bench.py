"""Benchmark of the fused decompress + mean-aggregation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the packed low-bit SQ configuration - a 2,449,029 x 128 feature table stored as 1-,
2- and 4-bit log-domain SQ codes of N(0,1) features, a synthetic power-law graph (Zipf 2.1 degrees,
mean 50), minibatches of 1024 seeds with fan-out 12,12,12.  One STEP aggregates the outermost block
(the one the fused first GraphSAGE layer sees: ~10^5 destination rows, ~10^6 edges) of one minibatch
with the fused kernel once per code width (three launches), gathering rows straight from the HBM-
resident table by global id.  Successive steps use different pre-sampled minibatches and L2 is
flushed between steps (outside the step's event pair).

Prints ONE JSON line (rank 0).  `value` = sampled edges aggregated per second by the whole job with
all inputs resident in HBM; `e2e` = the same work called through the public module with the block's
CSC in pinned host memory and the aggregated rows read back to the host inside the timed region.
`--impl reference` times the reference's PyTorch CPU path (oracle/torch_cpu_path.py) on the same
configuration on the host cores.
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
METRIC = "fused_sq_decompress_spmm_sampled_edges_per_s"
# dram__bytes_read.sum + dram__bytes_write.sum per launch on this block, from one ncu capture per width
# (profiles/sq_spmm_bench_block.md); below the algorithmic bytes because the output is still dirty in L2 at kernel end
NCU_DRAM_TRAFFIC_BYTES = {1: 34.9e6, 2: 43.1e6, 4: 48.5e6}


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


# --------------------------------------------------------------------------------------------- ours
def build_workload(device, rank, world):
    import torch
    from f2cgt_b200 import synth
    indptr, indices = synth.power_law_graph(NUM_NODES, AVG_DEGREE, ZIPF, seed=0, device=device)
    tables = {}
    for bits in BITS:
        tables[bits] = synth.sq_table_from_normal(NUM_NODES, FEAT_DIM, bits, COLUMN_SLICE, seed=0, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(1000 + rank)  # every rank draws its own seed minibatches (data parallel)
    blocks = []
    for b in range(N_MINIBATCHES):
        seeds = torch.randperm(NUM_NODES, generator=g, device=device)[:BATCH]
        blk = synth.sample_blocks(indptr, indices, seeds, FAN_OUT, rng_seed=rank * 1000 + b)[0]
        blocks.append((blk["indptr"].contiguous(), blk["indices_global"].contiguous()))
        if world > 1:  # what the sharded modes need: the block's distinct source rows and block-local ids
            BLOCK_EXTRA.append((blk["src_nodes"].contiguous(), blk["indices_local"].contiguous()))
    del indptr, indices
    torch.cuda.empty_cache()
    return tables, blocks


BLOCK_EXTRA = []


def time_steps(step_fn, blocks, steps, warmup, flush, torch):
    """Per-step CUDA events on the current stream; returns (list of step ms, edges done)."""
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
    return ms, edges


def multi_gpu_modes(args, capi, tables, blocks, flush, device, rank, world, torch, dist):
    """Row-sharded table at N > 1: NCCL all-to-all fetch (what the task statement describes) and direct peer loads."""
    from f2cgt_b200 import ops, shard
    out = {}
    lo, hi = shard.shard_bounds(NUM_NODES, world, rank)
    shards = {b: tables[b][0][lo:hi].contiguous() for b in BITS}
    # --- peer loads: every rank maps the other shards (CUDA IPC) and the kernel reads remote rows itself
    try:
        peers = {b: shard.PeerTable(shards[b], NUM_NODES) for b in BITS}

        def step_peer(i):
            ip, ix = blocks[i]
            for b in BITS:
                ops.sq_decompress_spmm_csr_peer(peers[b], tables[b][1], ip, ix, b, COLUMN_SLICE, FEAT_DIM)
        ms, edges = time_steps(step_peer, blocks, args.steps, args.warmup, flush, torch)
        out["sharded_peer_loads"] = (sum(ms), edges)
        # one-off check against the replicated table
        ip, ix = blocks[0]
        a = ops.sq_decompress_spmm_csr_peer(peers[4], tables[4][1], ip, ix, 4, COLUMN_SLICE, FEAT_DIM)
        bref = capi.sq_decompress_spmm_csr(tables[4][0], tables[4][1], ip, ix, 4, COLUMN_SLICE, FEAT_DIM)
        assert torch.equal(a, bref), "peer-load result differs from the replicated table"
    except Exception as e:  # noqa: BLE001
        out["sharded_peer_loads_error"] = repr(e)[:300]
    # --- NCCL all-to-all: owners gather rows, rows are exchanged, the kernel runs on block-local rows
    try:
        st = {b: shard.ShardedTable(shards[b], NUM_NODES) for b in BITS}
        plans = [st[BITS[0]].plan(src) for src, _ in BLOCK_EXTRA]  # id exchange happens when the block is sampled

        def step_a2a(i):
            ip, _ = blocks[i]
            _, ix_local = BLOCK_EXTRA[i]
            for b in BITS:
                rows = st[b].fetch_rows(plans[i])
                capi.sq_decompress_spmm_csr(rows, tables[b][1], ip, ix_local, b, COLUMN_SLICE, FEAT_DIM)
        ms, edges = time_steps(step_a2a, blocks, args.steps, args.warmup, flush, torch)
        out["sharded_nccl_all_to_all"] = (sum(ms), edges)
        rows = st[4].fetch_rows(plans[0])
        a = capi.sq_decompress_spmm_csr(rows, tables[4][1], blocks[0][0], BLOCK_EXTRA[0][1], 4, COLUMN_SLICE, FEAT_DIM)
        bref = capi.sq_decompress_spmm_csr(tables[4][0], tables[4][1], blocks[0][0], blocks[0][1], 4, COLUMN_SLICE, FEAT_DIM)
        assert torch.equal(a, bref), "all-to-all result differs from the replicated table"
    except Exception as e:  # noqa: BLE001
        out["sharded_nccl_all_to_all_error"] = repr(e)[:300]
    return out


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
    tables, blocks = build_workload(device, rank, world)
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=device)  # 256 MiB, read (not written) to evict L2

    def step_device(blk, out_sink=None):
        ip, ix = blk
        outs = []
        for bits in BITS:
            codes, cb = tables[bits]
            outs.append(capi.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM))
        return outs

    # ---- device-resident timing: per-step and per-kernel CUDA events on the launching (current) stream
    for w in range(args.warmup):
        step_device(blocks[w % len(blocks)])
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
    clocks = sampler.stop() if rank == 0 else None
    total_ms = sum(step_ms)

    # ---- end to end through the public module with HOST buffers: pinned CSC in, aggregated rows out
    host_blocks = [(ip.cpu().pin_memory(), ix.cpu().pin_memory()) for ip, ix in blocks]
    max_dst = max(ip.numel() - 1 for ip, _ in blocks)
    host_out = [torch.empty((max_dst, FEAT_DIM), dtype=torch.float32).pin_memory() for _ in BITS]
    e2e_steps = max(3, min(args.steps, 10))

    def step_e2e(hb):
        hip, hix = hb
        ip = hip.to(device, non_blocking=True)
        ix = hix.to(device, non_blocking=True)
        n_dst = hip.numel() - 1
        for j, bits in enumerate(BITS):
            codes, cb = tables[bits]
            out = capi.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
            host_out[j][:n_dst].copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        return (hip.numel() + hix.numel()) * 8, n_dst * FEAT_DIM * 4 * len(BITS), hix.numel() * len(BITS)

    for w in range(2):
        step_e2e(host_blocks[w % len(host_blocks)])
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h2d = d2h = e2e_edges = 0
    for s in range(e2e_steps):
        a, b, c = step_e2e(host_blocks[s % len(host_blocks)])
        h2d += a; d2h += b; e2e_edges += c
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    # ---- aggregate over ranks: max time, summed edges
    stats = torch.tensor([total_ms, e2e_s, float(edges_done), float(e2e_edges)], dtype=torch.float64, device=device)
    modes = {}
    if world > 1:
        mx = stats.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_s = float(mx[0]), float(mx[1])
        edges_all, e2e_edges_all = float(sm[2]), float(sm[3])
        modes["replicated"] = edges_all / (total_ms * 1e-3)
        raw = multi_gpu_modes(args, capi, tables, blocks, flush, device, rank, world, torch, dist)
        for name in ("sharded_peer_loads", "sharded_nccl_all_to_all"):
            ok = torch.tensor([1.0 if name in raw else 0.0], dtype=torch.float64, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok[0]) == 1.0:
                t = torch.tensor([raw[name][0]], dtype=torch.float64, device=device)
                e = torch.tensor([float(raw[name][1])], dtype=torch.float64, device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX); dist.all_reduce(e, op=dist.ReduceOp.SUM)
                modes[name] = float(e[0]) / (float(t[0]) * 1e-3)
            elif rank == 0 and name + "_error" in raw:
                modes[name + "_error"] = raw[name + "_error"]
    else:
        edges_all, e2e_edges_all = float(edges_done), float(e2e_edges)

    if rank == 0:
        peak, peak_kind = measured_peak()
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
        line = {
            "metric": METRIC, "value": edges_all / (total_ms * 1e-3), "unit": "edges/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8 codes -> f32", "data": "synthetic",
            "config": {"workload": "SQ 1/2/4-bit packed table 2449029x128 (N(0,1) features), power-law graph (Zipf 2.1, mean degree 50), "
                                   "1024 seeds x fan-out 12,12,12, outermost block, one fused launch per width per step",
                       "edges_per_block": int(n_edges), "dst_rows_per_block": int(n_dst), "index_dtype": "int64",
                       "gather": "global ids into the HBM-resident table", "minibatches_rotated": len(blocks),
                       "l2": "256 MiB read sweep between steps (outside the step's event pair) evicts L2; tables 39/78/157 MB",
                       "table": "replicated per GPU (157 MB at 4 bits); the row-sharded placements are timed beside it at N>1 "
                                "and reported in table_placements_edges_per_s", "timing": "CUDA events on the launching stream, max over ranks"},
            "roofline": {"bound": "hbm", "kernel": "sq_spmm_kernel<4-bit>", "achieved": dom["gbs"], "peak": peak, "unit": "GB/s",
                         "frac": dom["frac_of_peak"], "traffic": NCU_DRAM_TRAFFIC_BYTES[4], "traffic_unit": "bytes/launch (ncu dram read+write, profiles/sq_spmm_bench_block.md)", "algorithmic_bytes": dom["algorithmic_bytes"], "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})"},
            "variants": variants,
            "e2e": {"value": e2e_edges_all / e2e_s, "unit": "edges/s", "h2d_bytes_per_step": h2d // e2e_steps,
                    "d2h_bytes_per_step": d2h // e2e_steps, "steps": e2e_steps,
                    "what": "pinned-host CSC -> device, 3 fused launches via F2CGTLib, aggregated rows -> pinned host"},
            "gpu_launches": args.steps * len(BITS), "table_placements_edges_per_s": modes,
            "clocks": clocks, "wall_s_timed_region": wall,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_leg(blocks[0], steps=1, warmup=1, tables_dev=tables)
        if world == 1:
            line["reference_cuda_kernels"] = reference_cuda_leg(tables, blocks)
            line["other_fused_kernels"] = other_kernels_leg()
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def other_kernels_leg():
    """The VQ and two-level fused kernels on the same kind of block (f2cgt_b200.kernel_bench cases, CUDA events, cold L2),
    reported beside the headline: they are not part of `value`."""
    try:
        import argparse as _ap
        from f2cgt_b200 import kernel_bench
        b = kernel_bench.Bench(_ap.Namespace(only="vq_spmm,two_level", reps=10, small=False, launches=0, json=""))
        kernel_bench.cases(b)
        return [{k: r[k] for k in ("kernel", "ms", "algorithmic_bytes", "gbs", "frac_of_hbm_peak", "edges_per_s", "note") if k in r}
                for r in b.rows]
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:200]}


def reference_cuda_leg(tables, blocks):
    """The reference's own CUDA kernel for the same op on the same GPU (extension built from its sources
    by oracle/build_ref.py), for context; absent when that extension was not built."""
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
        for _ in range(2):
            ref.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(5):
            ref.sq_decompress_spmm_csr(codes, cb, ip, ix, bits, COLUMN_SLICE, FEAT_DIM)
        torch.cuda.synchronize()
        out[f"sq{bits}_ms"] = (time.perf_counter() - t0) / 5 * 1e3
    out["note"] = "warm L2, includes its torch::zeros output allocation, legacy default stream"
    return out


# --------------------------------------------------------------------------------------------- CPU
def cpu_leg(block, steps, warmup, tables_dev=None, tables_host=None):
    """Reference PyTorch CPU path on blocks[0] of one minibatch, all three widths per step."""
    import torch
    from oracle import torch_cpu_path as T
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ip, ix = block[0].cpu(), block[1].cpu()
    if tables_host is None:
        tables_host = {b: (t[0].cpu().view(torch.uint8), t[1].cpu()) for b, t in tables_dev.items()}
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
            "sample": f"one full step (blocks[0] of one minibatch, {ix.numel()} edges, widths 1/2/4), {steps} timed after {warmup} warm-up",
            "seconds_per_step": sec, "impl": "torch CPU: gather rows, shift/mask unpack, exp2 decode, sparse CSR mean matmul"}


def run_reference(args):
    """Reference arm: the whole configuration on the host - graph, table, sampler and the timed path all
    on CPU (torch + the oracle's sampler); nothing of the CUDA library is loaded."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    import numpy as np
    import torch
    from oracle import oracle as O
    from oracle import torch_cpu_path as T
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    # graph: same generator as the GPU arm, on the CPU device
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
    tables_host = {b: (torch.from_numpy(np.concatenate(v)), torch.from_numpy(cb)) for b, v in tables.items()}
    # minibatch blocks with the oracle's sampler
    blocks = []
    for mb in range(2):
        frontier = torch.randperm(NUM_NODES, generator=g)[:BATCH].numpy()
        for hop, pick in enumerate(reversed(FAN_OUT)):
            sip, six = O.sample_neighbors(ip_np, ix_np, frontier, pick, mb, hop)
            if hop == len(FAN_OUT) - 1:
                blocks.append((torch.from_numpy(sip), torch.from_numpy(six)))
            else:
                fresh = np.setdiff1d(np.unique(six), frontier)
                frontier = np.concatenate([frontier, fresh])
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
    n_edges = statistics.mean(ix.numel() for _, ix in blocks)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": int(os.environ.get("WORLD_SIZE", 1)),
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u8 codes -> f32", "data": "synthetic",
            "config": {"workload": "SQ 1/2/4-bit packed table 2449029x128 (N(0,1) features), power-law graph (Zipf 2.1, mean degree 50), "
                                   "1024 seeds x fan-out 12,12,12, outermost block, all three widths per step",
                       "edges_per_block": int(n_edges), "index_dtype": "int64"},
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
