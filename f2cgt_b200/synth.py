"""Seeded synthetic workloads with the shapes of the graphs and tables the reference is run on
(ogbn-products / papers100M / Friendster sized, scripts/run_*.sh of gpzlx1/F2CGT), which cannot be
downloaded here: a power-law graph in CSC, sampled minibatch blocks, and compressed tables drawn
directly as codes so that fp32 features are never materialised for the large configurations.

Everything is generated on the device the caller names with a torch.Generator seeded by the caller.
"""
import math

import torch

from . import ops


def power_law_graph(num_nodes, avg_degree, exponent=2.1, seed=0, device="cuda", index_dtype=torch.int64, max_degree=None):
    """CSC (indptr, indices) of a directed graph whose in-degrees follow a Zipf(exponent) law rescaled to
    the requested mean and whose sources are drawn with probability proportional to (out-)degree."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    u = torch.rand(num_nodes, generator=g, device=device, dtype=torch.float64).clamp_min(1e-12)
    raw = u.pow(-1.0 / (exponent - 1.0))  # Pareto tail with P(X > x) ~ x^-(exponent-1)
    cap = float(max_degree if max_degree is not None else max(1, num_nodes // 20))
    raw = raw.clamp_max(cap)
    deg = torch.floor(raw * (avg_degree / float(raw.mean()))).to(torch.int64).clamp_(0, int(cap))
    indptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=device)
    torch.cumsum(deg, 0, out=indptr[1:])
    nnz = int(indptr[-1].item())
    if nnz > torch.iinfo(index_dtype).max:
        # the library's CSC has ONE integer type for offsets and ids; offsets beyond its range would wrap silently
        raise ValueError(f"{nnz} edges do not fit {index_dtype} offsets: build this graph with int64")
    # degree-proportional endpoints: pick a uniformly random stub, then the node that owns it
    indices = torch.empty(nnz, dtype=index_dtype, device=device)
    chunk = 1 << 26
    for s in range(0, nnz, chunk):
        e = min(s + chunk, nnz)
        stub = torch.randint(0, nnz, (e - s,), generator=g, device=device)
        indices[s:e] = (torch.searchsorted(indptr, stub, right=True) - 1).to(index_dtype)
    return indptr.to(index_dtype), indices


def sample_blocks(indptr, indices, seeds, fan_out, rng_seed=0):
    """Minibatch blocks as the reference's loader builds them (examples/dataloader.py:167-182): hops are taken
    in reversed(fan_out) order starting from the seeds; after each hop the frontier becomes
    [previous frontier, new nodes] so destination nodes are always a prefix of the source nodes.

    Returns a list ordered like the reference's ``blocks`` (blocks[0] = outermost hop, the one the fused
    first layer aggregates); each entry is a dict with
      dst_nodes / src_nodes  global ids (dst is a prefix of src),
      indptr                 CSC over the dst nodes,
      indices_global         neighbour ids in the graph's numbering (index the full table directly),
      indices_local          the same edges relabelled to positions in src_nodes (index gathered rows).
    """
    frontier = seeds
    blocks = []
    for hop, num_pick in enumerate(reversed(list(fan_out))):
        sub_indptr, sub_indices = ops.csr_sampling(indptr, indices, frontier, num_pick, False, rng_seed, hop)
        # relabel as the reference's loader does (examples/dataloader.py:176-177): distinct ids of [frontier,
        # sampled neighbours] in order of first occurrence, so the frontier stays a prefix
        src_nodes, (_, local) = ops.tensor_relabel([frontier, sub_indices])
        blocks.insert(0, dict(dst_nodes=frontier, src_nodes=src_nodes, indptr=sub_indptr, indices_global=sub_indices,
                              indices_local=local))
        frontier = src_nodes
    return blocks


def sq_codebook_from_sample(sample, column_slice):
    """Codebook rows [fmin, fmax, emin, emax, mean] by the reference recipe (tests/test_sq.py:8-21,
    examples/process_compress.py:55-68) for every column slice of a float32 sample [rows, D] (on any device)."""
    D = sample.shape[1]
    rows = []
    eps = 1e-5
    for b in range(0, D, column_slice):
        a = sample[:, b:b + column_slice].float().abs().flatten()
        from .compress import _percentiles
        q = _percentiles(a, (0.005, 0.995))
        fmin = max(float(q[0]), eps)
        fmax = max(float(q[1]), 2 * eps)
        mean = float(a.mean())
        if mean < 0.1:
            mean += 0.1
        rows.append([fmin, fmax, math.log2(fmin), math.log2(fmax) + eps, mean])
    return torch.tensor(rows, dtype=torch.float32, device=sample.device)


def sq_table_from_normal(num_rows, feat_dim, bits, column_slice, seed=0, device="cuda", chunk_rows=1 << 18):
    """SQ table of N(0,1) features: codebooks from a 250k-row sample (examples/process_compress.py:47), rows
    encoded chunk by chunk with the library's own sq_compress + packbits, never holding the fp32 matrix."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    sample = torch.randn((min(num_rows, 250_000), feat_dim), generator=g, device=device)
    cb = sq_codebook_from_sample(sample, column_slice)
    del sample
    g.manual_seed(seed + 1)
    parts = []
    for s in range(0, num_rows, chunk_rows):
        x = torch.randn((min(chunk_rows, num_rows - s), feat_dim), generator=g, device=device)
        c = ops.sq_compress(x, cb, bits, column_slice)
        if bits < 8:
            parts.append(ops.packbits(c.to(torch.uint8), bits))
        elif bits == 8:
            parts.append(c.to(torch.int8))
        else:
            parts.append(c.to(torch.int16))
    return torch.cat(parts), cb
