"""Per-kernel micro-benchmark: every operator of the library on the shapes of the five benchmark
configurations, timed with CUDA events and compared with the roofline that bounds it.

    python -m f2cgt_b200.kernel_bench [--only SUBSTR] [--reps 20] [--small] [--json PATH] [--launches N] [--kernel FAMILY]

* fused aggregation kernels and decoders: algorithmic bytes / time against the measured HBM copy bandwidth;
* k-means assignment: 2*n*k*d flops / time (reported beside the bytes figure).

Between launches a 256 MiB read sweep evicts L2.  ``--small`` shrinks the tables so that one launch under a
profiler stays short; ``--launches N`` runs each selected case exactly N times without timing (for a profiler);
``--kernel stream|prefetch|general`` pins the kernel family of the fused aggregation cases (default: the library's choice).
Synthetic, seeded inputs; graph and sampler are the ones of ``f2cgt_b200.synth``.
"""
import argparse
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from f2cgt_b200 import ops, synth  # noqa: E402

FEAT = 128


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


class Bench:
    def __init__(self, args):
        self.args = args
        self.dev = torch.device("cuda", 0)
        self.flush = torch.zeros(64 << 20, dtype=torch.float32, device=self.dev)
        self.rows = []
        self.peak, self.peak_kind = hbm_peak()
        self._graph = None
        self._blocks = {}
        self.kernel = getattr(args, "kernel", "auto") or "auto"

    # ---- workload pieces
    def n_nodes(self):
        return 300_000 if self.args.small else 2_449_029

    def graph(self):
        if self._graph is None:
            self._graph = synth.power_law_graph(self.n_nodes(), 50, 2.1, seed=0, device=self.dev)
        return self._graph

    def block(self, fan_out=(12, 12, 12), which=0):
        """CSC of one sampled block: `which` = 0 outermost (the one the fused first layer sees), 1 = middle."""
        key = (fan_out, which)
        if key not in self._blocks:
            indptr, indices = self.graph()
            g = torch.Generator(device=self.dev)
            g.manual_seed(1000)
            seeds = torch.randperm(self.n_nodes(), generator=g, device=self.dev)[:1024]
            blk = synth.sample_blocks(indptr, indices, seeds, fan_out, rng_seed=0)[which]
            self._blocks[key] = (blk["indptr"].contiguous(), blk["indices_global"].contiguous())
        return self._blocks[key]

    def wanted(self, *names):
        """False when --only excludes every one of these case names (their inputs need not be built)."""
        if not self.args.only:
            return True
        return any(f in n for f in self.args.only.split(",") for n in names)

    # ---- timing
    def run(self, name, fn, nbytes=None, flops=None, units=None, unit_name="edges", note=""):
        if self.args.only and not any(s in name for s in self.args.only.split(",")):
            return
        if self.args.launches:
            for _ in range(self.args.launches):
                self.flush.sum()
                fn()
            torch.cuda.synchronize()
            print(f"{name}: {self.args.launches} launches done", flush=True)
            return
        for _ in range(3):
            fn()
            self.flush.sum()
        torch.cuda.synchronize()
        ms = []
        for _ in range(self.args.reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(200_000)  # the host queues the launch while the GPU is parked
            a.record()
            fn()
            b.record()
            self.flush.sum()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        t = statistics.median(ms)
        row = {"kernel": name, "ms": round(t, 5), "note": note}
        if nbytes is not None:
            row["algorithmic_bytes"] = int(nbytes)
            row["gbs"] = nbytes / (t * 1e-3) / 1e9
            row["frac_of_hbm_peak"] = row["gbs"] / self.peak
        if flops is not None:
            row["tflops"] = flops / (t * 1e-3) / 1e12
        if units is not None:
            row[f"{unit_name}_per_s"] = units / (t * 1e-3)
        self.rows.append(row)
        print(json.dumps(row), flush=True)


def fused_bytes(E, n_dst, row_bytes, idx_bytes, D, extra=0):
    return E * (row_bytes + idx_bytes) + (n_dst + 1) * idx_bytes + n_dst * D * 4 + extra


def cases(b):
    dev = b.dev
    N = b.n_nodes()
    g = torch.Generator(device=dev)
    g.manual_seed(0)

    # ------------------------------------------------ fused SQ (row widths of configurations 1 and 2)
    ip, ix = b.block()
    E, n_dst = ix.numel(), ip.numel() - 1
    for bits in (1, 2, 4, 8):
        if not b.wanted(f"sq_spmm_{bits}bit", f"sq_decompress_{bits}bit"):
            continue
        codes, cb = synth.sq_table_from_normal(N, FEAT, bits, FEAT, seed=0, device=dev)
        rb = codes.shape[1]
        b.run(f"sq_spmm_{bits}bit", lambda c=codes, k=cb, w=bits: ops.sq_decompress_spmm_csr(c, k, ip, ix, w, FEAT, FEAT, kernel=b.kernel),
              nbytes=fused_bytes(E, n_dst, rb, 8, FEAT, 20), units=E, note=f"E={E} n_dst={n_dst} table {N}x{rb}B")
        if bits == 8:
            rows = min(N, 1_000_000)
            sub = codes[:rows]
            b.run("sq_decompress_8bit", lambda c=sub, k=cb: ops.sq_decompress(c, k, 8, FEAT, FEAT),
                  nbytes=rows * (rb + FEAT * 4), units=rows, unit_name="rows")
        if bits == 4:
            rows = min(N, 1_000_000)
            sub = codes[:rows]
            b.run("sq_decompress_4bit", lambda c=sub, k=cb: ops.sq_decompress(c, k, 4, FEAT, FEAT),
                  nbytes=rows * (rb + FEAT * 4), units=rows, unit_name="rows")
        del codes
    # configuration 1: 100k x 128 int8, 10k destinations x exactly 12 uniform neighbours
    codes1, cb1 = synth.sq_table_from_normal(100_000, FEAT, 8, FEAT, seed=0, device=dev)
    ip1 = torch.arange(0, 120_001, 12, dtype=torch.int64, device=dev)
    ix1 = torch.randint(0, 100_000, (120_000,), generator=g, device=dev)
    b.run("sq_spmm_8bit_config1", lambda: ops.sq_decompress_spmm_csr(codes1, cb1, ip1, ix1, 8, FEAT, FEAT),
          nbytes=fused_bytes(120_000, 10_000, 128, 8, FEAT, 20), units=120_000, note="12.8 MB table: L2-resident after the first touch")

    # ------------------------------------------------ fused VQ (configurations 3 and 4) and the two-level kernel
    for n_cb, cs, tag in ((16, 8, "config3_16x8"), (4, 32, "config4_4x32")):
        if not b.wanted(f"vq_spmm_{tag}", "vq_decompress_4x32", "two_level_spmm_sq8_vq4x32", "two_level_spmm_sq8_vq4x32_hot_first"):
            continue
        vq = torch.randint(0, 256, (N, n_cb), generator=g, dtype=torch.uint8, device=dev)
        cbs = torch.randn(n_cb, 256, cs, generator=g, device=dev)
        b.run(f"vq_spmm_{tag}", lambda c=vq, k=cbs: ops.vq_decompress_spmm_csr(c, k, ip, ix, FEAT, kernel=b.kernel),
              nbytes=fused_bytes(E, n_dst, n_cb, 8, FEAT, cbs.numel() * 4), units=E, note=f"E={E} n_dst={n_dst}")
        if n_cb == 4:
            rows = min(N, 1_000_000)
            b.run("vq_decompress_4x32", lambda c=vq[:rows], k=cbs: ops.vq_decompress(c, k, FEAT),
                  nbytes=rows * (n_cb + FEAT * 4), units=rows, unit_name="rows")
            # two-level: the 5 % highest-degree nodes are hot (SQ 8 bits), everything else VQ 4x32
            indptr, _ = b.graph()
            deg = (indptr[1:] - indptr[:-1])
            n_hot = N // 20
            hot = torch.topk(deg, n_hot).indices
            slot = torch.full((N,), -1, dtype=torch.int32, device=dev)
            slot[hot] = torch.arange(n_hot, dtype=torch.int32, device=dev)
            sq_hot, sq_cb = synth.sq_table_from_normal(n_hot, FEAT, 8, FEAT, seed=1, device=dev)
            hot_edges = int((slot[ix] >= 0).sum())
            nb = (E - hot_edges) * (4 + 8 + 4) + hot_edges * (128 + 8 + 4) + (n_dst + 1) * 8 + n_dst * FEAT * 4 + cbs.numel() * 4 + 20
            b.run("two_level_spmm_sq8_vq4x32",
                  lambda: ops.two_level_decompress_spmm_csr(sq_hot, sq_cb, 8, FEAT, vq, cbs, slot, ip, ix, FEAT, kernel=b.kernel),
                  nbytes=nb, units=E, note=f"E={E} hot edges={hot_edges} n_dst={n_dst}; 4 B/edge slot lookup counted")
            b.run("two_level_spmm_sq8_vq4x32_dropout",
                  lambda: ops.two_level_decompress_spmm_csr(sq_hot, sq_cb, 8, FEAT, vq, cbs, slot, ip, ix, FEAT,
                                                            dropout=dict(p=0.5, seed=1, offset=0, training=True, scale=False)),
                  nbytes=nb, units=E, note="dropout fused in the epilogue")
            # the same block with HOT-FIRST NUMBERING: nodes renumbered by descending degree, so the hot 5 % are ids
            # 0 .. n_hot-1 and the kernel needs no slot array (same edges, same hot set; one random 4-byte read less per edge)
            rank_of = torch.empty(N, dtype=torch.int64, device=dev)
            rank_of[torch.argsort(deg, descending=True, stable=True)] = torch.arange(N, dtype=torch.int64, device=dev)
            ix_hf = rank_of[ix].contiguous()
            hot_hf = int((ix_hf < n_hot).sum())
            nb_hf = (E - hot_hf) * (4 + 8) + hot_hf * (128 + 8) + (n_dst + 1) * 8 + n_dst * FEAT * 4 + cbs.numel() * 4 + 20
            b.run("two_level_spmm_sq8_vq4x32_hot_first",
                  lambda: ops.two_level_decompress_spmm_csr(sq_hot, sq_cb, 8, FEAT, vq, cbs, None, ip, ix_hf, FEAT),
                  nbytes=nb_hf, units=E, note=f"E={E} hot edges={hot_hf} n_dst={n_dst}; hot nodes numbered first, no slot array")
            del slot, sq_hot, rank_of, ix_hf
        del vq

    # ------------------------------------------------ two-level, configuration-5 codecs: D = 256, hot 2 % SQ 4 bits + VQ 4 x 64
    # (256 KB of codebooks: two column parts), fan-out 15,10,5 (outermost hop takes 15).  The table has the rows of this
    # benchmark's 2.45 M-node graph; the configuration's own graph (65.6 M nodes, 3.6 B edges) is too large to build here.
    if b.wanted("two_level_spmm_sq4_vq4x64_config5", "vq_spmm_config5_4x64"):
        D5 = 256
        ip5, ix5 = b.block(fan_out=(15, 10, 5))
        E5, n5 = ix5.numel(), ip5.numel() - 1
        vq5 = torch.randint(0, 256, (N, 4), generator=g, dtype=torch.uint8, device=dev)
        cbs5 = torch.randn(4, 256, 64, generator=g, device=dev)
        b.run("vq_spmm_config5_4x64", lambda: ops.vq_decompress_spmm_csr(vq5, cbs5, ip5, ix5, D5),
              nbytes=fused_bytes(E5, n5, 4, 8, D5, cbs5.numel() * 4), units=E5, note=f"E={E5} n_dst={n5} D=256, two column parts")
        indptr, _ = b.graph()
        deg = (indptr[1:] - indptr[:-1])
        n_hot = N // 50
        hot = torch.topk(deg, n_hot).indices
        slot5 = torch.full((N,), -1, dtype=torch.int32, device=dev)
        slot5[hot] = torch.arange(n_hot, dtype=torch.int32, device=dev)
        sq5, sq5_cb = synth.sq_table_from_normal(n_hot, D5, 4, D5, seed=2, device=dev)
        hot_edges = int((slot5[ix5] >= 0).sum())
        nb5 = (E5 - hot_edges) * (4 + 8 + 4) + hot_edges * (128 + 8 + 4) + (n5 + 1) * 8 + n5 * D5 * 4 + cbs5.numel() * 4 + 20
        b.run("two_level_spmm_sq4_vq4x64_config5",
              lambda: ops.two_level_decompress_spmm_csr(sq5, sq5_cb, 4, D5, vq5, cbs5, slot5, ip5, ix5, D5),
              nbytes=nb5, units=E5, note=f"E={E5} hot edges={hot_edges} n_dst={n5} D=256; 4 B/edge slot lookup counted")
        del vq5, slot5, sq5

    # ------------------------------------------------ plain aggregation, dropout, packing, compress
    if not b.wanted("spmm_csr_f32", "dropout_inplace", "sq_compress_4bit", "packbits_4bit", "unpackbits_4bit") and \
            not b.wanted(*[f"kmeans_assign_d{d}_{m}" for d in (8, 32, 64) for m in ("l2", "cosine")]) and \
            not b.wanted(*[f"sample_block_hop{h}" for h in range(3)]):
        return
    rows = n_dst
    feat = torch.randn(min(N, 1_000_000), FEAT, generator=g, device=dev)
    ixs = ix % feat.shape[0]
    b.run("spmm_csr_f32", lambda: ops.spmm_csr(feat, ip, ixs), nbytes=fused_bytes(E, n_dst, FEAT * 4, 8, FEAT), units=E)
    big = torch.randn(1_000_000 if not b.args.small else 200_000, FEAT, generator=g, device=dev)
    b.run("dropout_inplace", lambda: ops.dropout_inplace(big, 0.5, True, seed=3), nbytes=2 * big.numel() * 4, units=big.numel(),
          unit_name="elements")
    cbq = torch.tensor([[1e-3, 4.0, -9.97, 2.0, 0.8]], device=dev)
    b.run("sq_compress_4bit", lambda: ops.sq_compress(big, cbq, 4, FEAT), nbytes=2 * big.numel() * 4, units=big.shape[0], unit_name="rows")
    un = torch.randint(0, 16, (big.shape[0], FEAT), generator=g, dtype=torch.uint8, device=dev)
    b.run("packbits_4bit", lambda: ops.packbits(un, 4), nbytes=un.numel() * 1.5, units=un.shape[0], unit_name="rows")
    pk = ops.packbits(un, 4)
    b.run("unpackbits_4bit", lambda: ops.unpackbits(pk, 4, FEAT), nbytes=un.numel() * 1.5, units=un.shape[0], unit_name="rows")
    del big, un, pk, feat

    # ------------------------------------------------ a block hop (sampler + relabel): one cooperative kernel against the
    #                                                  separate entry points, for the three hops of a fan-out 12,12,12 minibatch
    if b.wanted(*[f"sample_block_hop{h}" for h in range(3)]):
        gi, gx = b.graph()
        gs = torch.Generator(device=dev)
        gs.manual_seed(1000)
        seeds = torch.randperm(N, generator=gs, device=dev)[:1024]
        for hop in range(3):
            n = seeds.numel()
            keys = n * 13

            def separate(sd=seeds):
                ptr, idx = ops.csr_sampling(gi, gx, sd, 12, False, rng_seed=0, rng_offset=hop, exact=False)
                return ops.tensor_relabel([sd, idx])

            b.run(f"sample_block_hop{hop}", lambda sd=seeds: ops.sample_block_launch(gi, gx, sd, 12, rng_seed=0, rng_offset=hop),
                  units=n, unit_name="seeds", note=f"{n} seeds x 12 picks = {keys} keys, one cooperative kernel, no host read")
            b.run(f"sample_block_hop{hop}_separate_entry_points", separate, units=n, unit_name="seeds",
                  note="csr_sampling(exact=False) + tensor_relabel: 12 kernels, 3 memsets, one host read inside the timed pair")
            seeds = ops.sample_block(gi, gx, seeds, 12, rng_seed=0, rng_offset=hop)[2]

    # ------------------------------------------------ k-means assignment (configurations 3, 4, 5 sub-vector widths)
    for d in (8, 32, 64):
        x = torch.randn(N, d, generator=g, device=dev)
        c = torch.randn(256, d, generator=g, device=dev)
        for metric in ("l2", "cosine"):
            b.run(f"kmeans_assign_d{d}_{metric}", lambda x=x, c=c, m=metric: ops.kmeans_assign(x, c, m),
                  nbytes=N * d * 4 + N * 8 + 256 * d * 4, flops=2.0 * N * 256 * d, units=N, unit_name="points",
                  note="tensor-core scorer + exact re-score of undecided points")
        del x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--launches", type=int, default=0)
    ap.add_argument("--json", default="")
    ap.add_argument("--kernel", default="auto", choices=["auto", "stream", "prefetch", "general"])
    args = ap.parse_args()
    b = Bench(args)
    cases(b)
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"hbm_peak_gbs": b.peak, "peak_source": b.peak_kind, "rows": b.rows}, f, indent=1)


if __name__ == "__main__":
    main()
