"""GraphSAGE node classification over two-level compressed features: the training loop of the reference's
examples/train_graphsage_nodeclass.py (3-layer SAGE, fused first layer, Adam lr 0.003, ExponentialLR 0.978, one
process per GPU, DistributedDataParallel gradient all-reduce over NCCL) on seeded synthetic data with the shapes of
the benchmark configurations, reporting seconds per epoch.

    python -m f2cgt_b200.train_graphsage [--preset small|config4|config5] [--epochs 3]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m f2cgt_b200.train_graphsage --preset small

Data (no dataset can be downloaded here): power-law graph, uint8 VQ codes drawn uniformly with N(0,1) codebooks, hot
rows = the top fraction by a log-normal hotness, stored as SQ codes drawn uniformly with a codebook made by the
reference recipe from an N(0,1) sample, uniform random labels.  The whole compressed table and the graph are resident
in HBM on every rank; the training ids are split contiguously over the ranks (strong scaling of the epoch).
Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from f2cgt_b200 import sage, synth  # noqa: E402

PRESETS = {
    # nodes, avg degree, feat dim, classes, train ids, hot fraction, hot bits, VQ (n_cb, cs), hidden, fan-out
    "small": dict(nodes=2_449_029, degree=50, feat=128, classes=172, train=122_880, hot=0.05, hot_bits=8, vq=(4, 32), hidden=128,
                  fan_out=(12, 12, 12)),
    "config4": dict(nodes=111_059_956, degree=14.4, feat=128, classes=172, train=1_200_000, hot=0.05, hot_bits=8, vq=(4, 32), hidden=128,
                    fan_out=(12, 12, 12)),
    "config5": dict(nodes=65_608_366, degree=54.9, feat=256, classes=64, train=1_200_000, hot=0.02, hot_bits=4, vq=(4, 64), hidden=256,
                    fan_out=(15, 10, 5)),
}


def build_data(cfg, device, index_dtype, table="replicated"):
    n = cfg["nodes"]
    indptr, indices = synth.power_law_graph(n, cfg["degree"], 2.1, seed=0, device=device, index_dtype=index_dtype)
    g = torch.Generator(device=device)
    g.manual_seed(1)
    n_cb, cs = cfg["vq"]
    vq_codes = torch.randint(0, 256, (n, n_cb), generator=g, dtype=torch.uint8, device=device)
    vq_cbs = torch.randn(n_cb, 256, cs, generator=g, device=device)
    hotness = torch.empty(n, device=device).log_normal_(0.0, 1.0, generator=g)
    n_hot = max(1, int(n * cfg["hot"]))
    hot_nodes = torch.argsort(hotness, descending=True)[:n_hot]
    del hotness
    slot = torch.full((n,), -1, dtype=torch.int32, device=device)
    slot[hot_nodes] = torch.arange(n_hot, dtype=torch.int32, device=device)
    bits = cfg["hot_bits"]
    sample = torch.randn(100_000, cfg["feat"], generator=g, device=device)
    sq_cb = synth.sq_codebook_from_sample(sample, cfg["feat"])
    row_bytes = cfg["feat"] * bits // 8
    sq_codes = torch.randint(-128, 128, (n_hot, row_bytes), generator=g, dtype=torch.int8, device=device)
    labels = torch.randint(0, cfg["classes"], (n,), generator=g, device=device)
    train_ids = torch.randperm(n, generator=g, device=device)[:cfg["train"]].to(index_dtype)
    methods, configs, cbs = ["sq", "vq"], [(cfg["feat"], bits), (cs, 8)], [sq_cb, vq_cbs]
    if table == "sharded":  # every rank keeps only its row shard of the three tables
        from f2cgt_b200 import shard
        rank, world = dist.get_rank(), dist.get_world_size()
        lo, hi = shard.shard_bounds(n, world, rank)
        hlo, hhi = shard.shard_bounds(n_hot, world, rank)
        cm = sage.ShardedCompressionManager(cfg["feat"], methods, configs, cbs, [sq_codes[hlo:hhi].clone(), vq_codes[lo:hi].clone()],
                                            [n_hot, n], slot[lo:hi].clone())
        del sq_codes, vq_codes, slot
        torch.cuda.empty_cache()
    else:
        cm = sage.CompressionManager(cfg["feat"], methods, configs, cbs, [sq_codes, vq_codes], slot)
    return indptr, indices, labels, train_ids, cm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="small", choices=sorted(PRESETS))
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--batch-size", type=int, default=1024)
    ap.add_argument("--lr", type=float, default=0.003)
    ap.add_argument("--dropout", type=float, default=0.5)
    ap.add_argument("--index-dtype", default="int64", choices=["int32", "int64"])
    ap.add_argument("--max-steps", type=int, default=0, help="cut every epoch after this many steps (0 = whole epoch)")
    ap.add_argument("--no-autocast", action="store_true")
    ap.add_argument("--table", default="replicated", choices=["replicated", "sharded"],
                    help="sharded: every table row-sharded over the ranks, rows fetched per minibatch with an all-to-all exchange")
    args = ap.parse_args()
    cfg = PRESETS[args.preset]

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 or args.table == "sharded":
        if world == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("nccl", device_id=device, rank=rank, world_size=world)
    idt = torch.int32 if args.index_dtype == "int32" else torch.int64
    indptr, indices, labels, train_ids, cm = build_data(cfg, device, idt, args.table)

    torch.manual_seed(0)
    model = sage.SAGE(cfg["feat"], cfg["hidden"], cfg["classes"], len(cfg["fan_out"]), args.dropout, cm).to(device)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank]) if world > 1 else model
    optimizer = torch.optim.Adam(net.parameters(), lr=args.lr)
    scheduler = torch.optim.lr_scheduler.ExponentialLR(optimizer, gamma=0.978)
    loader = sage.GPUSamplingDataloader(indptr, indices, train_ids, args.batch_size, cfg["fan_out"], rank, world, shuffle=True)
    steps = torch.tensor([len(loader)], device=device)
    if world > 1:
        dist.all_reduce(steps, op=dist.ReduceOp.MIN)  # every rank takes the same number of steps (gradient all-reduce)
    steps = int(steps.item())
    if args.max_steps:
        steps = min(steps, args.max_steps)

    epoch_s, losses, edges = [], [], 0
    for epoch in range(args.epochs):
        net.train()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        it = iter(loader)
        for step in range(steps):
            input_nodes, output_nodes, blocks = next(it)
            y = labels[output_nodes]
            with torch.autocast("cuda", dtype=torch.bfloat16, enabled=not args.no_autocast):
                pred = net(blocks)
            loss = F.cross_entropy(pred.float(), y)
            optimizer.zero_grad(set_to_none=True)
            loss.backward()
            optimizer.step()
            if epoch == args.epochs - 1:
                edges += blocks[0]["indices_global"].numel()
        scheduler.step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        epoch_s.append(time.perf_counter() - t0)
        losses.append(float(loss.detach()))
    timed = epoch_s[1:] if len(epoch_s) > 1 else epoch_s
    tmax = torch.tensor([sum(timed) / len(timed)], device=device, dtype=torch.float64)
    etot = torch.tensor([float(edges)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(etot, op=dist.ReduceOp.SUM)
    if rank == 0:
        print(json.dumps({
            "metric": "graphsage_epoch_seconds", "value": float(tmax[0]), "unit": "s/epoch", "n_gpus": world, "preset": args.preset,
            "steps_per_epoch_per_gpu": steps, "batch_size": args.batch_size, "epochs_run": args.epochs,
            "epoch_seconds_all": [round(t, 4) for t in epoch_s], "ms_per_step": float(tmax[0]) / steps * 1e3,
            "first_layer_edges_per_s": float(etot[0]) / float(tmax[0]), "loss_last_step_per_epoch": [round(v, 4) for v in losses],
            "config": {k: (list(v) if isinstance(v, tuple) else v) for k, v in cfg.items()}, "index_dtype": args.index_dtype,
            "autocast_bf16": not args.no_autocast, "table": args.table, "data": "synthetic", "scaling": "strong (train ids split over ranks)",
            "timing": "wall clock around barrier + synchronize delimited epochs, first epoch discarded, max over ranks"}), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
