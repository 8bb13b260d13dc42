"""GraphSAGE node classification over two-level compressed features: the training loop of the reference's
examples/train_graphsage_nodeclass.py (3-layer SAGE, fused first layer, Adam lr 0.003, ExponentialLR 0.978, one
process per GPU, gradients all-reduced over NCCL every step) on seeded synthetic data with the shapes of
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
    if table in ("sharded", "sharded_peer"):  # every rank keeps only its row shard of the three tables
        from f2cgt_b200 import shard
        rank, world = dist.get_rank(), dist.get_world_size()
        lo, hi = shard.shard_bounds(n, world, rank)
        hlo, hhi = shard.shard_bounds(n_hot, world, rank)
        kind = sage.ShardedCompressionManager if table == "sharded" else sage.PeerCompressionManager
        cm = kind(cfg["feat"], methods, configs, cbs, [sq_codes[hlo:hhi].clone(), vq_codes[lo:hi].clone()], [n_hot, n], slot[lo:hi].clone())
        del sq_codes, vq_codes, slot
        torch.cuda.empty_cache()
    else:
        cm = sage.CompressionManager(cfg["feat"], methods, configs, cbs, [sq_codes, vq_codes], slot)
    return indptr, indices, labels, train_ids, cm


class DirectFusedAdam:
    """Adam through the same fused multi-tensor kernel ``torch.optim.Adam(fused=True)`` launches, without the optimizer
    class around it: ``step()`` is two launches and a dozen Python operations where the class spends ~0.15 ms per step on
    parameter groups, state dictionaries and device / dtype grouping - a tenth of a host-bound training step.  Same update,
    bit for bit (``tests/test_gpu_sage.py``).  ``available()`` tells whether this torch exposes the kernel."""

    def __init__(self, params, lr, betas=(0.9, 0.999), eps=1e-8):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.betas, self.eps = float(lr), betas, float(eps)
        self.exp_avg = [torch.zeros_like(p) for p in self.params]
        self.exp_avg_sq = [torch.zeros_like(p) for p in self.params]
        self.steps = [torch.zeros((), dtype=torch.float32, device=p.device) for p in self.params]

    @staticmethod
    def available():
        return hasattr(torch, "_fused_adam_") and hasattr(torch, "_foreach_add_")

    def zero_grad(self, set_to_none=True):
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    @torch.no_grad()
    def step(self):
        torch._foreach_add_(self.steps, 1)
        torch._fused_adam_(self.params, [p.grad for p in self.params], self.exp_avg, self.exp_avg_sq, [], self.steps, amsgrad=False,
                           lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], weight_decay=0.0, eps=self.eps, maximize=False,
                           grad_scale=None, found_inf=None)


def train(preset="small", table="replicated", rank=0, world=1, local_rank=0, epochs=3, min_timed_steps=0, batch_size=1024, lr=0.003,
          dropout=0.5, index_dtype="int64", max_steps=0, precision="tf32", ahead=True):
    """Train on the preset's synthetic data inside an already initialised process (and, for world > 1 or a sharded table,
    process group); returns the record rank 0 reports (every rank gets it).  The first epoch is a discarded warm-up; when
    ``min_timed_steps`` is set, enough further epochs are run to time at least that many steps per rank.  Per-phase device
    times come from CUDA events on the current stream (sample / exchange / forward / backward / optimizer)."""
    cfg = PRESETS[preset]
    device = torch.device("cuda", local_rank)
    idt = torch.int32 if index_dtype == "int32" else torch.int64
    indptr, indices, labels, train_ids, cm = build_data(cfg, device, idt, table)

    torch.manual_seed(0)
    model = sage.SAGE(cfg["feat"], cfg["hidden"], cfg["classes"], len(cfg["fan_out"]), dropout, cm).to(device)
    net = model
    flat_grad = None
    if world > 1:
        # Data parallel as the reference runs it (DistributedDataParallel, examples/train_graphsage_nodeclass.py:50-54): same
        # initial weights on every rank, gradients averaged over the ranks with an NCCL all-reduce every step.  The model has
        # ~0.1 M parameters, so the gradients live in ONE flat buffer (every p.grad is a view of it) and a step costs one
        # all-reduce and one scale instead of DDP's bucket and hook machinery (measured: 0.5-0.8 ms per step).
        params = [p for p in model.parameters() if p.requires_grad]
        for p in params:
            dist.broadcast(p.data, src=0)
        flat_grad = torch.zeros(sum(p.numel() for p in params), dtype=torch.float32, device=device)
        off = 0
        for p in params:
            p.grad = flat_grad[off:off + p.numel()].view_as(p)
            off += p.numel()
    # Adam lr 0.003 with an exponential decay of 0.978 per epoch (examples/train_graphsage_nodeclass.py:56-57); one fused
    # kernel for all parameters (the model is tiny)
    gamma = 0.978
    if DirectFusedAdam.available():
        optimizer, scheduler = DirectFusedAdam(net.parameters(), lr=lr), None
    else:
        optimizer = torch.optim.Adam(net.parameters(), lr=lr, fused=True)
        scheduler = torch.optim.lr_scheduler.ExponentialLR(optimizer, gamma=gamma)
    loader = sage.GPUSamplingDataloader(indptr, indices, train_ids, batch_size, cfg["fan_out"], rank, world, shuffle=True, ahead=ahead)
    # The reference trains in fp32 (examples/train_graphsage_nodeclass.py has no autocast).  "tf32": fp32 storage, matrix
    # products on the tensor cores with tf32 inputs and fp32 accumulation - no cast kernels at all, which matters because
    # the step is bound by the host's launch rate, not by the GPU.  "fp32": plain.  "bf16": the layers' products round their
    # operands to bf16 (sage.products_in), everything else stays fp32 - the mixed precision the two-level configuration names.
    if precision not in ("tf32", "fp32", "bf16"):
        raise ValueError("precision must be tf32, fp32 or bf16")
    product_dtype = torch.bfloat16 if precision == "bf16" else None
    tf32_before = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = precision == "tf32"
    steps = torch.tensor([len(loader)], device=device)
    if world > 1:
        dist.all_reduce(steps, op=dist.ReduceOp.MIN)  # every rank takes the same number of steps (gradient all-reduce)
    steps = int(steps.item())
    if max_steps:
        steps = min(steps, max_steps)
    if min_timed_steps:
        epochs = max(epochs, 1 + (min_timed_steps + steps - 1) // steps)

    phases = ("sample", "exchange", "forward", "backward", "optimizer")
    epoch_s, losses, edges = [], [], 0
    phase_ms = {k: 0.0 for k in phases}
    timed_steps = 0
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(steps)]
    for epoch in range(epochs):
        net.train()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        it = iter(loader)
        first_layer_edges = 0
        for step in range(steps):
            ev = marks[step]  # reused every epoch: creating six events costs the host as much as queueing four kernels
            ev[0].record()
            input_nodes, output_nodes, blocks = next(it)
            y = labels[output_nodes]
            ev[1].record()
            blocks[0]["first_layer_input"] = cm.for_block(blocks[0])  # sharded table: the row exchange of this minibatch
            ev[2].record()
            with sage.products_in(product_dtype):
                pred = net(blocks)
            loss = F.cross_entropy(pred, y)
            ev[3].record()
            loader.poke()  # next minibatch: one hop further on its own stream, if that needs no waiting
            if flat_grad is None:
                optimizer.zero_grad(set_to_none=True)
                with sage.products_in(product_dtype):
                    loss.backward()
            else:
                flat_grad.zero_()  # the views stay attached to the parameters
                with sage.products_in(product_dtype):
                    loss.backward()
                dist.all_reduce(flat_grad, op=dist.ReduceOp.AVG)  # NCCL divides inside the collective: no scale kernel
            ev[4].record()
            loader.poke()
            optimizer.step()
            ev[5].record()
            loader.poke()
            if epoch == epochs - 1:
                first_layer_edges += blocks[0]["n_edges"]  # the loader read it with the hop's other counters
        if scheduler is not None:
            scheduler.step()
        else:
            optimizer.lr *= gamma
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        epoch_s.append(time.perf_counter() - t0)
        if first_layer_edges:
            edges = float(first_layer_edges)
        losses.append(float(loss.detach()))
        if epoch > 0 or epochs == 1:
            timed_steps += steps
            for ev in marks:
                for i, k in enumerate(phases):
                    phase_ms[k] += ev[i].elapsed_time(ev[i + 1])
    timed = epoch_s[1:] if len(epoch_s) > 1 else epoch_s
    stats = torch.tensor([sum(timed) / len(timed), float(edges)] + [phase_ms[k] / max(timed_steps, 1) for k in phases], device=device,
                         dtype=torch.float64)
    if world > 1:
        mx = stats.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        stats = torch.cat([mx[:1], sm[1:2], mx[2:]])
    stats = stats.tolist()
    torch.backends.cuda.matmul.allow_tf32 = tf32_before
    if hasattr(cm, "close"):
        torch.cuda.synchronize()
        cm.close()
    return {
        "metric": "graphsage_epoch_seconds", "value": stats[0], "unit": "s/epoch", "n_gpus": world, "preset": preset,
        "steps_per_epoch_per_gpu": steps, "timed_steps_per_gpu": timed_steps, "batch_size": batch_size, "epochs_run": epochs,
        "epoch_seconds_all": [round(t, 4) for t in epoch_s], "ms_per_step": stats[0] / steps * 1e3,
        "breakdown_ms": {k: round(v, 4) for k, v in zip(phases, stats[2:])},
        "first_layer_edges_per_s": stats[1] / stats[0], "loss_last_step_per_epoch": [round(v, 4) for v in losses],
        "config": {k: (list(v) if isinstance(v, tuple) else v) for k, v in cfg.items()}, "index_dtype": index_dtype,
        "precision": precision, "blocks_built_ahead": bool(ahead), "table": table, "data": "synthetic", "scaling": "strong (train ids split over ranks)",
        "timing": "wall clock around barrier + synchronize delimited epochs, first epoch discarded, max over ranks; breakdown = CUDA "
                  "events on the current stream, mean per step, max over ranks"}


def pin_rank_cpus(local_rank, local_world):
    """Give every rank of the node its own share of the CPUs the process may run on.  With a gradient all-reduce per step
    every rank waits for the slowest host, and ranks (each with its autograd and NCCL threads) that wander over all cores
    get in one another's way: measured on a 4-GPU box with 32 CPUs, 1.71-1.76 ms per step pinned against 1.94-2.11 free.
    Only when a share has at least 8 CPUs: a rank runs its training thread, the autograd engine's thread and NCCL's proxy
    threads, and with 4 CPUs each (8 ranks on the same box) pinning made the epoch 5 % slower instead.
    Call it before CUDA and the process group start their threads (they inherit the mask).  Returns the mask, or None
    when nothing was changed."""
    if local_world <= 1 or not hasattr(os, "sched_setaffinity"):
        return None
    try:
        cpus = sorted(os.sched_getaffinity(0))
        per = len(cpus) // local_world
        if per < 8:
            return None
        mine = set(cpus[local_rank * per:(local_rank + 1) * per])
        os.sched_setaffinity(0, mine)
        return mine
    except OSError:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="small", choices=sorted(PRESETS))
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--batch-size", type=int, default=1024)
    ap.add_argument("--lr", type=float, default=0.003)
    ap.add_argument("--dropout", type=float, default=0.5)
    ap.add_argument("--index-dtype", default="int64", choices=["int32", "int64"])
    ap.add_argument("--max-steps", type=int, default=0, help="cut every epoch after this many steps (0 = whole epoch)")
    ap.add_argument("--min-timed-steps", type=int, default=0, help="run enough epochs to time at least this many steps")
    ap.add_argument("--precision", default="tf32", choices=["tf32", "fp32", "bf16"],
                    help="tf32: fp32 storage, tf32 tensor-core products (default); fp32: plain; bf16: product operands in bf16")
    ap.add_argument("--no-pin", action="store_true", help="do not give every rank its own share of the node's CPUs")
    ap.add_argument("--no-ahead", action="store_true", help="build every minibatch inside its step instead of one step early on a side stream")
    ap.add_argument("--table", default="replicated", choices=["replicated", "sharded", "sharded_peer"],
                    help="sharded: every table row-sharded over the ranks, rows fetched per minibatch with an all-to-all exchange; "
                         "sharded_peer: the same shards mapped into every rank, the fused kernel reads remote rows over NVLink")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if not args.no_pin:
        pin_rank_cpus(local_rank, int(os.environ.get("LOCAL_WORLD_SIZE", world)))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 or args.table != "replicated":
        if world == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("nccl", device_id=device, rank=rank, world_size=world)
    rec = train(args.preset, args.table, rank, world, local_rank, args.epochs, args.min_timed_steps, args.batch_size, args.lr,
                args.dropout, args.index_dtype, args.max_steps, args.precision, not args.no_ahead)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
