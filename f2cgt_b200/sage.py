"""DGL-free GraphSAGE over compressed features, mirroring the reference's training stack on top of the library:

* ``CompressionManager`` - what examples/compress.py keeps: codecs, codebooks and tables of a one- or two-level
  compressed feature matrix.  Here the tables stay resident in HBM and are addressed by GLOBAL node id, so there is
  no gathered copy of the codes per minibatch: ``aggregate`` is the fused decode + mean over a block's CSC,
  ``decode_rows`` decodes the rows of given nodes (the same fused kernel over an identity CSC: the mean of one
  neighbour is that neighbour, bit for bit).
* ``MySAGEConv`` - the fused first layer (examples/conv.py:9-76): ``fc_self(h_self) + fc_neigh(mean of decoded
  neighbours)``, ``fc_neigh`` without bias.
* ``SAGEConv`` - mean SAGE layer for hidden features (what the reference takes from DGL), aggregation through
  ``spmm_csr`` with a backward pass over the transposed block.
* ``SAGE`` - examples/models.py:10-42: ReLU + dropout between layers.
* ``GPUSamplingDataloader`` - examples/dataloader.py:154-192: per minibatch, hops in reversed(fan_out) order from the
  seeds with ``csr_sampling`` + ``tensor_relabel``; yields (input_nodes, output_nodes, blocks).

Blocks are dicts with ``indptr`` (CSC over the destination nodes), ``indices_local`` (positions in ``src_nodes``),
``indices_global``, ``src_nodes``, ``dst_nodes``; destination nodes are a prefix of the source nodes.
"""
import torch
from torch import nn

from . import ops


class CompressionManager:
    """methods: ["sq"] | ["vq"] | ["sq", "vq"] (two-level: level 0 = hot rows, level 1 = every row)."""

    def __init__(self, feat_dim, methods, configs, codebooks, tables, slot=None, hot_first=False):
        self.feat_dim = int(feat_dim)
        self.methods = list(methods)
        self.configs = list(configs)      # per level (column_slice, target_bits) as the reference stores them
        self.codebooks = list(codebooks)
        self.tables = list(tables)
        self.slot = slot                  # int32 [n_nodes]: row of the hot table, -1 for cold nodes (two-level only)
        self.is_two_level = len(self.methods) >= 2
        # hot_first: the graph is numbered so that the hot nodes are ids 0 .. len(tables[0]) - 1 (no slot array, one random
        # read less per edge)
        if self.is_two_level and (self.methods != ["sq", "vq"] or (slot is None and not hot_first)):
            raise ValueError("two-level compression is hot SQ rows over a VQ table, with a slot array or hot-first numbering")

    def aggregate(self, indptr, indices_global, dropout=None):
        if self.is_two_level:
            cs, bits = self.configs[0]
            return ops.two_level_decompress_spmm_csr(self.tables[0], self.codebooks[0], bits, cs, self.tables[1], self.codebooks[1],
                                                     self.slot, indptr, indices_global, self.feat_dim, dropout=dropout)
        if self.methods[0] == "vq":
            return ops.vq_decompress_spmm_csr(self.tables[0], self.codebooks[0], indptr, indices_global, self.feat_dim, dropout=dropout)
        cs, bits = self.configs[0]
        return ops.sq_decompress_spmm_csr(self.tables[0], self.codebooks[0], indptr, indices_global, bits, cs, self.feat_dim,
                                          dropout=dropout)

    def decode_rows(self, nodes):
        ident = torch.arange(nodes.numel() + 1, dtype=nodes.dtype, device=nodes.device)
        return self.aggregate(ident, nodes)

    def for_block(self, block):
        """(manager, neighbour ids, destination ids) with which the first layer reads this block: the resident tables
        are addressed by global id."""
        return self, block["indices_global"], block["dst_nodes"]


class ShardedCompressionManager:
    """The same compressed feature matrix with every table ROW-SHARDED over the ranks of the process group (rank r owns
    rows [r * ceil(n / world), ...) of the VQ table, of the slot array and - keyed by slot - of the hot SQ table).

    Per minibatch the rows of the block's source nodes are fetched from their owners with the all-to-all exchange of
    ``f2cgt_b200.shard.ShardedTable`` (ids out, rows back: NCCL over NVLink), which gives a block-local
    ``CompressionManager`` over gathered rows; the fused kernel then runs on block-local ids.  ``for_block`` is a
    collective: every rank calls it once per step."""

    def __init__(self, feat_dim, methods, configs, codebooks, local_tables, table_rows, local_slot=None, group=None):
        from . import shard
        self.feat_dim, self.methods, self.configs, self.codebooks = int(feat_dim), list(methods), list(configs), list(codebooks)
        self.is_two_level = len(self.methods) >= 2
        self.level2 = shard.ShardedTable(local_tables[-1], table_rows[-1], group)
        if self.is_two_level:
            if self.methods != ["sq", "vq"] or local_slot is None:
                raise ValueError("two-level compression is hot SQ rows over a VQ table, with a slot array")
            self.hot = shard.ShardedTable(local_tables[0], table_rows[0], group)
            self.slot = shard.ShardedTable(local_slot.reshape(-1, 1), table_rows[-1], group)

    def for_block(self, block):
        src = block["src_nodes"]
        n_dst = block["dst_nodes"].numel()
        plan = self.level2.plan(src)
        rows = self.level2.fetch_rows(plan)
        dst_local = torch.arange(n_dst, dtype=src.dtype, device=src.device)
        if not self.is_two_level:
            local = CompressionManager(self.feat_dim, self.methods, self.configs, self.codebooks, [rows])
            return local, block["indices_local"], dst_local
        slots = self.slot.fetch_rows(plan).reshape(-1)  # same ids, same row partition: the plan is shared
        hot_pos = (slots >= 0).nonzero().reshape(-1)
        hot_rows = self.hot.fetch(slots[hot_pos].to(src.dtype))
        local_slot = torch.full_like(slots, -1)
        local_slot[hot_pos] = torch.arange(hot_pos.numel(), dtype=slots.dtype, device=slots.device)
        local = CompressionManager(self.feat_dim, self.methods, self.configs, self.codebooks, [hot_rows, rows], local_slot)
        return local, block["indices_local"], dst_local


class PeerCompressionManager:
    """The same compressed feature matrix with every table row-sharded over the ranks AND mapped into every rank
    (``f2cgt_b200.shard.PeerTable``, CUDA IPC): the fused kernel reads the rows other ranks own over NVLink while it
    aggregates, so a minibatch needs no exchange step at all.  Construct and ``close`` it collectively.

    local_tables / table_rows as for ``ShardedCompressionManager``: [hot SQ shard, VQ shard] (two-level) or [VQ shard]."""

    def __init__(self, feat_dim, methods, configs, codebooks, local_tables, table_rows, local_slot=None, group=None):
        from . import shard
        self.feat_dim, self.methods, self.configs, self.codebooks = int(feat_dim), list(methods), list(configs), list(codebooks)
        self.is_two_level = len(self.methods) >= 2
        if self.methods not in (["vq"], ["sq", "vq"]):
            raise ValueError("the sharded kernel serves a VQ table, alone or under hot SQ rows")
        self.level2 = shard.PeerTable(local_tables[-1].contiguous(), table_rows[-1], group)
        self.hot = self.slot = None
        if self.is_two_level:
            self.hot = shard.PeerTable(local_tables[0].contiguous(), table_rows[0], group)
            if local_slot is not None:  # None: hot-first numbering
                self.slot = shard.PeerTable(local_slot.reshape(-1, 1).contiguous(), table_rows[-1], group)

    def aggregate(self, indptr, indices_global, dropout=None):
        cs, bits = self.configs[0] if self.is_two_level else (1, 8)
        return ops.two_level_decompress_spmm_csr_peer(self.hot, self.codebooks[0] if self.is_two_level else None, bits, cs, self.level2,
                                                      self.codebooks[-1], self.slot, indptr, indices_global, self.feat_dim, dropout=dropout)

    def decode_rows(self, nodes):
        ident = torch.arange(nodes.numel() + 1, dtype=nodes.dtype, device=nodes.device)
        return self.aggregate(ident, nodes)

    def for_block(self, block):
        return self, block["indices_global"], block["dst_nodes"]

    def close(self):
        for t in (self.slot, self.hot, self.level2):
            if t is not None:
                t.close()


def _bucket(n):
    """Row counts of sampled blocks change every step; the matrix products behind the Linear layers pick (and cache)
    their algorithms per shape, so inputs are zero-padded to a few recurring row counts."""
    step = 4096 if n > 16384 else 512 if n > 2048 else 128
    return (n + step - 1) // step * step


def _linear_rows(fc, x):
    n = x.shape[0]
    m = _bucket(n)
    if m != n:
        x = torch.nn.functional.pad(x, (0, 0, 0, m - n))
    return fc(x)[:n]


class _MeanAggregate(torch.autograd.Function):
    """out[d] = mean over the block's neighbours of h[src]; backward adds grad / deg to every neighbour's row."""

    @staticmethod
    def forward(ctx, h, indptr, indices, n_src):
        ctx.save_for_backward(indptr, indices)
        ctx.n_src = n_src
        return ops.spmm_csr(h, indptr, indices)

    @staticmethod
    def backward(ctx, grad_out):
        indptr, indices = ctx.saved_tensors
        # one scatter kernel (vector reductions into the source rows) instead of building the transposed block
        return ops.spmm_csr_backward(grad_out.float().contiguous(), indptr, indices, ctx.n_src), None, None, None


class MySAGEConv(nn.Module):
    def __init__(self, in_feats, out_feats, compression_manager, bias=True):
        super().__init__()
        self.fc_neigh = nn.Linear(in_feats, out_feats, bias=False)
        self.fc_self = nn.Linear(in_feats, out_feats, bias=bias)
        self.sm = compression_manager
        gain = nn.init.calculate_gain("relu")
        nn.init.xavier_uniform_(self.fc_self.weight, gain=gain)
        nn.init.xavier_uniform_(self.fc_neigh.weight, gain=gain)

    def forward(self, block, _unused=None):
        # (manager, neighbour ids, destination ids): fetched by the caller beforehand (so that a sharded table's row
        # exchange can be timed and overlapped on its own) or here
        sm, neighbours, dst = block.get("first_layer_input") or self.sm.for_block(block)
        h_neigh = sm.aggregate(block["indptr"], neighbours)  # raw codes in, no autograd through it
        h_self = sm.decode_rows(dst)
        return _linear_rows(self.fc_self, h_self) + _linear_rows(self.fc_neigh, h_neigh)


class SAGEConv(nn.Module):
    def __init__(self, in_feats, out_feats, bias=True):
        super().__init__()
        self.fc_neigh = nn.Linear(in_feats, out_feats, bias=False)
        self.fc_self = nn.Linear(in_feats, out_feats, bias=bias)
        gain = nn.init.calculate_gain("relu")
        nn.init.xavier_uniform_(self.fc_self.weight, gain=gain)
        nn.init.xavier_uniform_(self.fc_neigh.weight, gain=gain)

    def forward(self, block, h):
        n_dst = block["dst_nodes"].numel()
        h32 = h.float().contiguous()
        h_neigh = _MeanAggregate.apply(h32, block["indptr"], block["indices_local"], h.shape[0])
        return _linear_rows(self.fc_self, h[:n_dst]) + _linear_rows(self.fc_neigh, h_neigh)


class SAGE(nn.Module):
    def __init__(self, in_feats, n_hidden, n_classes, n_layers, dropout, cm):
        super().__init__()
        self.layers = nn.ModuleList()
        for i in range(n_layers):
            in_dim = in_feats if i == 0 else n_hidden
            out_dim = n_classes if i == n_layers - 1 else n_hidden
            self.layers.append(MySAGEConv(in_dim, out_dim, cm) if i == 0 else SAGEConv(in_dim, out_dim))
        self.dropout = nn.Dropout(dropout)

    def forward(self, blocks, x=None):
        h = x
        for i, (layer, block) in enumerate(zip(self.layers, blocks)):
            h = layer(block, h)
            if i != len(self.layers) - 1:
                h = self.dropout(torch.relu(h))
        return h


class GPUSamplingDataloader:
    """Seeds are split contiguously over the ranks (examples/dataloader.py:102-108), shuffled per epoch."""

    def __init__(self, indptr, indices, seeds, batchsize, num_picks, rank=0, world=1, shuffle=True, rng_seed=0):
        self.indptr, self.indices = indptr, indices
        self.batchsize, self.num_picks = int(batchsize), list(num_picks)
        self.shuffle, self.rng_seed, self.epoch = shuffle, rng_seed, 0
        per = (seeds.numel() + world - 1) // world
        self.seeds = seeds[rank * per:(rank + 1) * per]
        self.rank = rank

    def __len__(self):
        return (self.seeds.numel() + self.batchsize - 1) // self.batchsize

    def __iter__(self):
        self.curr = 0
        if self.shuffle:
            g = torch.Generator(device=self.seeds.device)
            g.manual_seed(self.rng_seed * 1000003 + self.epoch)
            self.order = self.seeds[torch.randperm(self.seeds.numel(), generator=g, device=self.seeds.device)]
        else:
            self.order = self.seeds
        self.epoch += 1
        return self

    def __next__(self):
        if self.curr >= len(self):
            raise StopIteration
        seeds = self.order[self.curr * self.batchsize:(self.curr + 1) * self.batchsize]
        step = self.curr
        self.curr += 1
        output_nodes = seeds
        blocks = []
        for hop, num_pick in enumerate(reversed(self.num_picks)):
            # one library call and one host read (the number of distinct nodes) per hop; the index tensors carry a tail
            # behind indptr[-1] that no kernel reads
            sub_indptr, sub_indices, unique, local = ops.sample_block(
                self.indptr, self.indices, seeds, num_pick,
                rng_seed=(self.rng_seed * 7919 + self.epoch) * 65536 + self.rank, rng_offset=step * 8 + hop)
            blocks.insert(0, dict(dst_nodes=seeds, src_nodes=unique, indptr=sub_indptr, indices_global=sub_indices, indices_local=local))
            seeds = unique
        return seeds, output_nodes, blocks
