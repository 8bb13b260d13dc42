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
``indices_global``, ``src_nodes``, ``dst_nodes``, ``n_edges`` (a host integer); destination nodes are a prefix of the
source nodes.
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

    def aggregate(self, indptr, indices_global, dropout=None, out_rows=None):
        """``out_rows``: allocate that many output rows (zero behind the block's own), see ``ops._block_out``."""
        if self.is_two_level:
            cs, bits = self.configs[0]
            return ops.two_level_decompress_spmm_csr(self.tables[0], self.codebooks[0], bits, cs, self.tables[1], self.codebooks[1],
                                                     self.slot, indptr, indices_global, self.feat_dim, dropout=dropout, out_rows=out_rows)
        if self.methods[0] == "vq":
            return ops.vq_decompress_spmm_csr(self.tables[0], self.codebooks[0], indptr, indices_global, self.feat_dim, dropout=dropout,
                                              out_rows=out_rows)
        cs, bits = self.configs[0]
        return ops.sq_decompress_spmm_csr(self.tables[0], self.codebooks[0], indptr, indices_global, bits, cs, self.feat_dim,
                                          dropout=dropout, out_rows=out_rows)

    def decode_rows(self, nodes, out_rows=None):
        return self.aggregate(_identity_offsets(nodes), nodes, out_rows=out_rows)

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
        if not self.is_two_level:
            self.level2 = shard.ShardedTable(local_tables[-1], table_rows[-1], group)
        else:
            if self.methods != ["sq", "vq"] or local_slot is None:
                raise ValueError("two-level compression is hot SQ rows over a VQ table, with a slot array")
            self.hot = shard.ShardedTable(local_tables[0], table_rows[0], group)
            codes = local_tables[-1]
            self.code_bytes = codes.shape[1] * codes.element_size()
            # a node's VQ code row and its slot travel as ONE row of code_bytes + 4 bytes: one gather and one exchange per
            # minibatch instead of two
            packed = torch.cat([codes.contiguous().view(torch.uint8).reshape(codes.shape[0], self.code_bytes),
                                local_slot.to(torch.int32).contiguous().view(torch.uint8).reshape(-1, 4)], dim=1)
            self.level2 = shard.ShardedTable(packed, table_rows[-1], group)
            self.code_dtype, self.code_width = codes.dtype, codes.shape[1]

    def for_block(self, block):
        src = block["src_nodes"]
        n_dst = block["dst_nodes"].numel()
        # Fetched rows are used where the exchange puts them (grouped by owner): the block's 8-byte indices are renumbered
        # to that order once instead of un-sorting every fetched table (4 .. 128 bytes per row, three tables).
        plan = self.level2.plan(src, check=False)  # ids straight from the sampler / slots from our own table
        arrival = plan["position"]
        rows = self.level2.fetch_rows(plan, ordered=False)
        dst_local = arrival[:n_dst].contiguous()
        neighbours = arrival[block["indices_local"]]
        if not self.is_two_level:
            local = CompressionManager(self.feat_dim, self.methods, self.configs, self.codebooks, [rows])
            return local, neighbours, dst_local
        slots = rows[:, self.code_bytes:].contiguous().view(torch.int32).reshape(-1)
        rows = rows[:, :self.code_bytes].contiguous().view(self.code_dtype).reshape(-1, self.code_width)
        hot_pos = (slots >= 0).nonzero().reshape(-1)
        hot_plan = self.hot.plan(slots[hot_pos].to(src.dtype), check=False)
        hot_rows = self.hot.fetch_rows(hot_plan, ordered=False)
        local_slot = torch.full_like(slots, -1)
        local_slot[hot_pos] = hot_plan["position"].to(slots.dtype)
        local = CompressionManager(self.feat_dim, self.methods, self.configs, self.codebooks, [hot_rows, rows], local_slot)
        return local, neighbours, dst_local


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

    def aggregate(self, indptr, indices_global, dropout=None, out_rows=None):
        cs, bits = self.configs[0] if self.is_two_level else (1, 8)
        return ops.two_level_decompress_spmm_csr_peer(self.hot, self.codebooks[0] if self.is_two_level else None, bits, cs, self.level2,
                                                      self.codebooks[-1], self.slot, indptr, indices_global, self.feat_dim, dropout=dropout,
                                                      out_rows=out_rows)

    def decode_rows(self, nodes, out_rows=None):
        return self.aggregate(_identity_offsets(nodes), nodes, out_rows=out_rows)

    def for_block(self, block):
        return self, block["indices_global"], block["dst_nodes"]

    def close(self):
        for t in (self.slot, self.hot, self.level2):
            if t is not None:
                t.close()


_CACHE = {}


def _identity_offsets(nodes):
    """[0, 1, ..., len(nodes)] in the dtype and on the device of ``nodes``: the CSC of "every row is its own only
    neighbour", under which a fused aggregation is a row decode.  One growing tensor per (device, dtype)."""
    key = ("ident", nodes.device, nodes.dtype)
    have = _CACHE.get(key)
    if have is None or have.numel() < nodes.numel() + 1:
        have = _CACHE[key] = torch.arange(max(2 * nodes.numel(), 4096) + 1, dtype=nodes.dtype, device=nodes.device)
    return have[:nodes.numel() + 1]


def _ones_row(m, like):
    key = ("ones", like.device, like.dtype)
    have = _CACHE.get(key)
    if have is None or have.shape[1] < m:
        have = _CACHE[key] = torch.ones((1, max(2 * m, 4096)), dtype=like.dtype, device=like.device)
    return have[:, :m]


def _bucket(n):
    """Row counts of sampled blocks change every step; the matrix products behind the Linear layers pick (and cache)
    their algorithms per shape, and the caching allocator keeps blocks per size, so the layers work on row counts rounded
    up to a few recurring values.  The extra rows are carried through the network instead of being cut off and padded
    again at every product: they never feed a real row (aggregation reads by index, below the block's row count), their
    gradients are zero, and only the final output is sliced."""
    step = 4096 if n > 16384 else 512 if n > 2048 else 128
    return (n + step - 1) // step * step


_PRODUCT_DTYPE = None  # None: the tensors' own dtype (fp32, or tf32 on the tensor cores when torch allows it)


class products_in:
    """``with products_in(torch.bfloat16):`` - the layers' matrix products round their operands to that dtype (storage,
    aggregation, bias and gradients stay fp32): the bf16 / fp32 mixed precision some configurations ask for.  It costs a
    cast kernel per operand, so it is slower than the default in a step that is bound by launches."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global _PRODUCT_DTYPE
        self.before, _PRODUCT_DTYPE = _PRODUCT_DTYPE, self.dtype

    def __exit__(self, *exc):
        global _PRODUCT_DTYPE
        _PRODUCT_DTYPE = self.before


def _mm(a, b):
    if _PRODUCT_DTYPE is None:
        return torch.mm(a, b)
    return torch.mm(a.to(_PRODUCT_DTYPE), b.to(_PRODUCT_DTYPE)).float()


def _affine(bias, a, b):
    if _PRODUCT_DTYPE is None:
        return torch.addmm(bias, a, b) if bias is not None else torch.mm(a, b)
    y = _mm(a, b)
    return y.add_(bias) if bias is not None else y


def _addmm_(y, a, b):
    return y.addmm_(a, b) if _PRODUCT_DTYPE is None else y.add_(_mm(a, b))


class _SageProduct(torch.autograd.Function):
    """y = x_self @ w_self^T + x_neigh @ w_neigh^T + bias for inputs that need no gradient (the decoded first layer)."""

    @staticmethod
    def forward(ctx, x_self, x_neigh, w_self, w_neigh, bias):
        ctx.save_for_backward(x_self, x_neigh)
        ctx.has_bias = bias is not None
        return _addmm_(_affine(bias, x_self, w_self.t()), x_neigh, w_neigh.t())

    @staticmethod
    def backward(ctx, dy):
        x_self, x_neigh = ctx.saved_tensors
        dy = dy.contiguous()
        dyt = dy.t()
        db = torch.mm(_ones_row(dy.shape[0], dy), dy).reshape(-1) if ctx.has_bias else None
        return None, None, _mm(dyt, x_self), _mm(dyt, x_neigh), db


class _SageLayer(torch.autograd.Function):
    """A hidden mean-SAGE layer in one autograd node: y = h[:m] @ w_self^T + mean_neigh(h) @ w_neigh^T + bias over m >= n_dst
    rows (rows behind n_dst: see ``_bucket``).  The backward pass is written out - five products, one scatter kernel - so a
    step queues a third of the kernels autograd would for the same layer built from Linear, slice and pad nodes."""

    @staticmethod
    def forward(ctx, h, indptr, indices, n_dst, m, w_self, w_neigh, bias):
        neigh = ops.spmm_csr(h, indptr, indices, out_rows=m)
        h_self = h[:m]
        y = _addmm_(_affine(bias, h_self, w_self.t()), neigh, w_neigh.t())
        ctx.save_for_backward(h, neigh, indptr, indices, w_self, w_neigh)
        ctx.n_dst, ctx.m, ctx.has_bias = n_dst, m, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        h, neigh, indptr, indices, w_self, w_neigh = ctx.saved_tensors
        n_dst, m = ctx.n_dst, ctx.m
        dy = dy.contiguous()
        dyt = dy.t()
        dw_self = _mm(dyt, h[:m])
        dw_neigh = _mm(dyt, neigh)
        db = torch.mm(_ones_row(m, dy), dy).reshape(-1) if ctx.has_bias else None
        dh = None
        if ctx.needs_input_grad[0]:
            d_neigh = _mm(dy, w_neigh)
            # one scatter kernel (vector reductions into the source rows) instead of building the transposed block
            dh = ops.spmm_csr_backward(d_neigh[:n_dst], indptr, indices, h.shape[0])
            _addmm_(dh[:m], dy, w_self)
        return dh, None, None, None, None, dw_self, dw_neigh, db


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

    def forward_padded(self, block, _unused=None):
        """[_bucket(n_dst), out]: the layer's output with the extra rows of ``_bucket`` left in place."""
        # (manager, neighbour ids, destination ids): fetched by the caller beforehand (so that a sharded table's row
        # exchange can be timed and overlapped on its own) or here
        sm, neighbours, dst = block.get("first_layer_input") or self.sm.for_block(block)
        m = _bucket(dst.numel())
        h_neigh = sm.aggregate(block["indptr"], neighbours, out_rows=m)  # raw codes in, no autograd through it
        h_self = sm.decode_rows(dst, out_rows=m)
        return _SageProduct.apply(h_self, h_neigh, self.fc_self.weight, self.fc_neigh.weight, self.fc_self.bias)

    def forward(self, block, _unused=None):
        return self.forward_padded(block)[:block["dst_nodes"].numel()]


class SAGEConv(nn.Module):
    def __init__(self, in_feats, out_feats, bias=True):
        super().__init__()
        self.fc_neigh = nn.Linear(in_feats, out_feats, bias=False)
        self.fc_self = nn.Linear(in_feats, out_feats, bias=bias)
        gain = nn.init.calculate_gain("relu")
        nn.init.xavier_uniform_(self.fc_self.weight, gain=gain)
        nn.init.xavier_uniform_(self.fc_neigh.weight, gain=gain)

    def forward_padded(self, block, h):
        """``h``: [>= n_src, in] float32 (rows behind the block's source nodes are ignored); returns [m, out] with
        m = min(_bucket(n_dst), rows of h)."""
        n_dst = block["dst_nodes"].numel()
        h = h.float().contiguous()
        m = min(_bucket(n_dst), h.shape[0])
        return _SageLayer.apply(h, block["indptr"], block["indices_local"], n_dst, m, self.fc_self.weight, self.fc_neigh.weight,
                                self.fc_self.bias)

    def forward(self, block, h):
        return self.forward_padded(block, h)[:block["dst_nodes"].numel()]


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
            h = layer.forward_padded(block, h)
            if i != len(self.layers) - 1:
                h = self.dropout(torch.relu(h))
        n_out = blocks[-1]["dst_nodes"].numel()
        return h if h.shape[0] == n_out else h[:n_out]


class GPUSamplingDataloader:
    """Seeds are split contiguously over the ranks (examples/dataloader.py:102-108), shuffled per epoch.

    ``ahead=True`` (default) builds every minibatch one step early on a CUDA stream of its own.  A block is a chain of
    small dependent kernels with one host read per hop; on the training stream that chain would sit on the critical path
    of every step although it needs nothing from the model.  Here ``__next__`` hands out the minibatch built during the
    previous step and queues the first hop of the next; each later hop is queued by ``poke()`` - which the training loop
    calls between its phases and which never blocks - or, at the latest, by the next ``__next__``.  The minibatches are
    the same either way: sampling draws are keyed by epoch, step and hop.  In this mode the loader works in two sets of
    buffers it allocates once (sized for the largest possible hop), used alternately: the tensors of a minibatch are
    views of one set and stay valid until the next-but-one ``__next__``."""

    def __init__(self, indptr, indices, seeds, batchsize, num_picks, rank=0, world=1, shuffle=True, rng_seed=0, ahead=True):
        # one check of the graph per loader (the sampling kernels trust it): offsets that wrapped in a too narrow integer
        # type show up here
        first, last = indptr[[0, -1]].tolist()
        if first != 0 or last != indices.numel():
            raise ValueError(f"indptr must run from 0 to len(indices) = {indices.numel()} (it runs from {first} to {last})")
        self.indptr, self.indices = indptr, indices
        self.batchsize, self.num_picks = int(batchsize), list(num_picks)
        self.shuffle, self.rng_seed, self.epoch = shuffle, rng_seed, 0
        per = (seeds.numel() + world - 1) // world
        self.seeds = seeds[rank * per:(rank + 1) * per]
        self.rank = rank
        self.side = torch.cuda.Stream(device=indptr.device) if ahead else None
        self._gen = self._result = self._wait = None
        self._sets, self._consumed, self._built = None, [None, None], 0

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
        self._gen = self._result = self._wait = None
        if self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream(self.indptr.device))  # the shuffled order is read over there
            self._start()
        return self

    def _buffer_sets(self):
        if self._sets is None:
            n_nodes, bound, sizes = self.indptr.numel() - 1, self.batchsize, []
            for num_pick in reversed(self.num_picks):
                sizes.append((bound, num_pick))
                bound = min(bound * (num_pick + 1), n_nodes)  # a hop's distinct nodes are the next hop's seeds
            self._sets = [[ops.BlockBuffers(b, k, self.indptr.dtype, self.indptr.device) for b, k in sizes] for _ in range(2)]
        return self._sets

    def _hops(self, seeds, step, buffers=None):
        """Generator over one minibatch: yields the pending hop after queueing it, returns the minibatch."""
        output_nodes, blocks = seeds, []
        for hop, num_pick in enumerate(reversed(self.num_picks)):
            # one library call and one host read (the number of distinct nodes) per hop; the index tensors carry a tail
            # behind indptr[-1] that no kernel reads
            pending = ops.sample_block_launch(self.indptr, self.indices, seeds, num_pick,
                                              rng_seed=(self.rng_seed * 7919 + self.epoch) * 65536 + self.rank, rng_offset=step * 8 + hop,
                                              buffers=None if buffers is None else buffers[hop])
            yield pending
            sub_indptr, sub_indices, unique, local = ops.sample_block_finish(pending)
            blocks.insert(0, dict(dst_nodes=seeds, src_nodes=unique, indptr=sub_indptr, indices_global=sub_indices, indices_local=local,
                                  n_edges=pending.n_edges))
            seeds = unique
        return seeds, output_nodes, blocks

    def _start(self):
        if self.curr >= len(self):
            self._gen = None
            return
        seeds = self.order[self.curr * self.batchsize:(self.curr + 1) * self.batchsize]
        which = self._built % 2
        self._built += 1
        if self._consumed[which] is not None:  # the minibatch that last lived in this set: its step must be through
            self.side.wait_event(self._consumed[which])
        self._gen = self._hops(seeds, self.curr, self._buffer_sets()[which])
        self.curr += 1
        self._advance()

    def _advance(self):
        """Finish the pending hop (blocks until the GPU is done with it) and queue the next one."""
        with torch.cuda.stream(self.side):
            try:
                self._wait = next(self._gen)
            except StopIteration as done:
                self._result, self._gen, self._wait = done.value, None, None

    def poke(self):
        """Move the minibatch under construction one hop forward if that needs no waiting; call it wherever the host has
        just queued a stretch of GPU work."""
        if self._gen is not None and self._wait is not None and self._wait.event.query():
            self._advance()

    def __next__(self):
        if self.side is None:
            if self.curr >= len(self):
                raise StopIteration
            gen = self._hops(self.order[self.curr * self.batchsize:(self.curr + 1) * self.batchsize], self.curr)
            self.curr += 1
            try:
                while True:
                    next(gen)
            except StopIteration as done:
                return done.value
        if self._gen is None and self._result is None:
            raise StopIteration
        while self._result is None:
            self._advance()
        batch, self._result = self._result, None
        cur = torch.cuda.current_stream(self.indptr.device)
        cur.wait_stream(self.side)
        # Everything queued on this stream so far belongs to earlier minibatches: once it has run, the set of the
        # minibatch handed out before this one may be overwritten (which is what the _start below goes on to do).
        previous = self._built % 2
        if self._consumed[previous] is None:
            self._consumed[previous] = torch.cuda.Event()
        self._consumed[previous].record(cur)
        self._start()
        return batch
