"""Offline feature compressor and the artefact format the trainer loads - the flow of the reference's
examples/process_compress.py on top of the library's operators, in one process or split over the ranks of a process
group the way the reference splits it (:82-107,192-196,225,236-238): codebook statistics by COLUMN slices (rank r
computes the codebook rows of its slices, then they are all-gathered), encoding by ROW ranges (rank r encodes rows
[r * ceil(n / world), ...) with all codebooks).  Who computes a slice does not change the result: samples and k-means
initialisations are seeded per column slice, so the split artefact equals the single-process one bit for bit.

* SQ (``target_compression_ratio <= element bits``): per column slice a codebook row
  ``[fmin, fmax, emin, emax, mean]`` from the 0.5 / 99.5 percentiles of |x| over a 250,000-row sample
  (:43-68), rows encoded in 1M-row batches with ``sq_compress`` and stored packed (:71-144).
* VQ (larger ratios): per column slice of width ``ratio / element bytes`` a cosine k-means over a 150,000-row sample
  from which the lowest-norm rows are dropped, centres rescaled to their mean norm (:16-18,145-181); codes =
  nearest centre under the cosine metric, uint8 / int16 by codebook size (:185-292).
* Two-level (``seeds`` given): the seed rows additionally as SQ at ``element bits / 8`` bits (:311-345).

``compress`` returns the dictionary the reference saves as ``compression_meta.pt`` (keys ``methods``, ``codebooks``,
``configs`` = (column_slice, target_bits) per level, ``feat_dim``, ``data``, ``seeds``) plus the tables;
``save`` / ``load`` write and read ``compression_meta.pt``, ``compression_data.pt`` and ``seeds_compression_data.pt``.
"""
import os

import torch

from . import ops


def normalize(data):
    """Centres rescaled to the mean of their norms (examples/process_compress.py:16-18)."""
    norm = data.norm(dim=1, p=2)
    return data / norm.reshape(-1, 1) * norm.mean()


def _sample_rows(num_items, sample_size, hotness, gen):
    if sample_size >= num_items:
        return torch.arange(num_items, device=gen.device)
    if hotness is None:
        return torch.randperm(num_items, generator=gen, device=gen.device)[:sample_size]
    p = hotness.to(gen.device, torch.float32)
    return torch.multinomial(p / p.sum(), sample_size, replacement=False, generator=gen)


def _percentiles(a, qs):
    """numpy.percentile (linear interpolation) of a 1-D tensor of any size, through one sort (torch.quantile stops at
    2^24 elements; the reference takes the percentiles of the whole 250,000 x slice sample, :55-58)."""
    v, _ = torch.sort(a)
    n = v.numel()
    out = []
    for q in qs:
        pos = q * (n - 1)
        lo = int(pos)
        hi = min(lo + 1, n - 1)
        out.append(float(v[lo].double() + (v[hi].double() - v[lo].double()) * (pos - lo)))
    return out


def sq_metadata(sample):
    """One codebook row from a sample of one column slice (examples/process_compress.py:43-68)."""
    eps = 1e-5
    a = sample.float().abs().flatten()
    q = _percentiles(a, (0.005, 0.995))
    fmin = max(float(q[0]), eps)
    fmax = max(float(q[1]), 2 * eps)
    mean = float(a.mean())
    if mean < 0.1:
        mean += 0.1
    # emin / emax are float32 values in the reference (torch.log2 of a float32 tensor, then + epsilon)
    emin = float(torch.log2(torch.tensor(fmin, dtype=torch.float32)))
    emax = float(torch.log2(torch.tensor(fmax, dtype=torch.float32)) + eps)
    return [fmin, fmax, emin, emax, mean]


# ---------------------------------------------------------------------------------------------- rank split (host logic)
def split_plan(n_rows, n_slices, world, rank):
    """What rank ``rank`` of ``world`` owns: (first, last+1) of its column slices and of its row range
    (examples/process_compress.py:82-83,105-107 for SQ, :192-196,236-238 for VQ: slices in contiguous groups of
    ceil(n_slices / world), rows in contiguous ranges of ceil(n_rows / world))."""
    per = (n_slices + world - 1) // world
    s_lo, s_hi = min(per * rank, n_slices), min(per * (rank + 1), n_slices)
    rpr = (n_rows + world - 1) // world
    r_lo, r_hi = min(rpr * rank, n_rows), min(rpr * (rank + 1), n_rows)
    return (s_lo, s_hi), (r_lo, r_hi)


def gather_parts(part, group):
    """Concatenation over the ranks, in rank order, of per-rank tensors whose leading sizes differ (codebook rows of a
    rank's column slices, or the encoded rows of its row range); a rank may contribute nothing."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = [None] * world
    dist.all_gather_object(sizes, int(part.shape[0]), group=group)
    most = max(max(sizes), 1)
    padded = torch.zeros((most,) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
    padded[:part.shape[0]] = part
    got = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(got, padded, group=group)
    return torch.cat([g[:k] for g, k in zip(got, sizes)], dim=0)


def _split(group):
    if group is None:
        return 1, 0
    import torch.distributed as dist
    return dist.get_world_size(group), dist.get_rank(group)


def sq_compress_features(features, target_bits, column_slice, hotness=None, sample_size=250_000, batch_rows=1_000_000, seed=0,
                         group=None, gather=True):
    """features [n, D] (any float dtype, on the GPU) -> (stored codes, codebooks [ceil(D / column_slice), 5]).

    With a process group: every rank passes the same features; rank r computes the codebook rows of its column slices and
    encodes its row range; ``gather=False`` returns only that row range of the table (a row shard), else the whole table."""
    n, D = features.shape
    world, rank = _split(group)
    n_slices = (D + column_slice - 1) // column_slice
    (s_lo, s_hi), (r_lo, r_hi) = split_plan(n, n_slices, world, rank)
    gen = torch.Generator(device=features.device)
    rows = []
    for i in range(s_lo, s_hi):
        gen.manual_seed(seed * 1000003 + i)  # per slice, so that the row is the same whichever rank computes it
        idx = _sample_rows(n, sample_size, hotness, gen)
        rows.append(sq_metadata(features[idx, i * column_slice:(i + 1) * column_slice]))
    codebooks = torch.tensor(rows, dtype=torch.float32, device=features.device).reshape(-1, 5)
    if group is not None:
        codebooks = gather_parts(codebooks, group)
    parts = []
    for s in range(r_lo, r_hi, batch_rows):
        x = features[s:min(s + batch_rows, r_hi)].float().contiguous()
        c = ops.sq_compress(x, codebooks, target_bits, column_slice)
        if target_bits < 8:
            parts.append(ops.packbits(c.to(torch.uint8), target_bits).view(torch.int8))  # stored as int8 (:109-111,141)
        elif target_bits == 8:
            parts.append(c.to(torch.int8))
        else:
            parts.append(c.to(torch.int16))
    width = (D * target_bits + 7) // 8 if target_bits <= 8 else D
    table = torch.cat(parts) if parts else torch.empty((0, width), dtype=torch.int8 if target_bits <= 8 else torch.int16,
                                                       device=features.device)
    if group is not None and gather:
        table = gather_parts(table, group)
    return table, codebooks


def vq_metadata(features, n_clusters, column_slice, hotness=None, sample_size=150_000, seed=0, max_iter=300, tol=5e-2, slices=None):
    """Codebooks [n_slices, n_clusters, column_slice] of the column slices ``slices`` = (first, last+1) (all by default)."""
    n, D = features.shape
    gen = torch.Generator(device=features.device)
    gen.manual_seed(seed)
    idx = _sample_rows(n, sample_size, hotness, gen)
    num_slice = (D + column_slice - 1) // column_slice
    s_lo, s_hi = slices if slices is not None else (0, num_slice)
    codebooks = torch.zeros((s_hi - s_lo, n_clusters, column_slice), dtype=torch.float32, device=features.device)
    for i in range(s_lo, s_hi):
        b, e = i * column_slice, min((i + 1) * column_slice, D)
        data = features[idx, b:e].float()
        dist = data.norm(dim=1, p=2)
        rim = torch.quantile(dist, min(1.0, 0.00625 * (data.shape[1] / 8)))
        data = data[dist >= rim].contiguous()
        km = ops.KMeans(n_clusters, data.shape[1], "cosine", max_iter=max_iter, tol=tol)
        torch.manual_seed(seed * 1000 + i)  # KMeans.fit draws its initial centres from torch's generator
        km.fit(data)
        codebooks[i - s_lo, :, :e - b] = normalize(km.get_centers())
    if torch.isnan(codebooks).any():
        raise ValueError("codebooks has nan")
    return codebooks


def vq_compress_features(features, n_clusters, column_slice, hotness=None, batch_rows=1_000_000, seed=0, group=None, gather=True,
                         **fit_args):
    n, D = features.shape
    world, rank = _split(group)
    num_slice = (D + column_slice - 1) // column_slice
    slices, (r_lo, r_hi) = split_plan(n, num_slice, world, rank)
    codebooks = vq_metadata(features, n_clusters, column_slice, hotness, seed=seed, slices=slices, **fit_args)
    if group is not None:
        codebooks = gather_parts(codebooks, group)
    dtype = torch.uint8 if n_clusters <= 256 else torch.int16
    if n_clusters > 32767:
        raise ValueError("the kernels address at most 32767 centres per slice (int16 codes)")
    codes = torch.empty((r_hi - r_lo, num_slice), dtype=dtype, device=features.device)
    for s in range(r_lo, r_hi, batch_rows):
        e_row = min(s + batch_rows, r_hi)
        for i in range(num_slice):
            b, e = i * column_slice, min((i + 1) * column_slice, D)
            data = torch.zeros((e_row - s, column_slice), dtype=torch.float32, device=features.device)
            data[:, :e - b] = features[s:e_row, b:e].float()
            labels = ops.kmeans_assign(data, codebooks[i].contiguous(), "cosine")
            codes[s - r_lo:e_row - r_lo, i] = labels.to(dtype)
    if group is not None and gather:
        codes = gather_parts(codes, group)
    return codes, codebooks


def compress(features, seeds=None, hotness=None, target_compression_ratio=32, n_clusters=256, world_size=None, seed=0, group=None,
             gather=True, **fit_args):
    """The decision logic of examples/process_compress.py:295-394.  Returns the meta dictionary with the tables added
    under ``compression_data`` / ``seeds_compression_data``.

    ``group``: split the work over that process group (see the module text); ``world_size`` then defaults to its size.
    ``world_size`` alone only sets the SQ column-slice width the reference derives from it (ceil(D / world) rounded up to
    8, :330,352), so a single process can reproduce the artefact of a ``world_size``-rank run.  ``gather=False`` leaves
    ``compression_data`` as this rank's row range (``meta["row_range"]``), which is what a row-sharded table wants."""
    n, feat_dim = features.shape
    if world_size is None:
        world_size = _split(group)[0]
    elem_bits = features.element_size() * 8
    meta = dict(methods=[], codebooks=[], configs=[], feat_dim=feat_dim, data={})

    def sq_slice():
        cs = (feat_dim + world_size - 1) // world_size
        return (cs + 7) // 8 * 8

    if seeds is not None:
        bits = elem_bits // 8
        cs = sq_slice()
        table, cb = sq_compress_features(features[seeds], bits, cs, None, seed=seed, group=group)  # the seed rows: always whole
        meta["methods"].append("sq")
        meta["configs"].append((cs, bits))
        meta["codebooks"].append(cb)
        meta["data"]["seeds_compression_data"] = (table.dtype, tuple(table.shape))
        meta["seeds"] = seeds
        meta["seeds_compression_data"] = table
    if target_compression_ratio <= elem_bits:
        bits = int(elem_bits / target_compression_ratio)
        cs = sq_slice()
        table, cb = sq_compress_features(features, bits, cs, hotness, seed=seed + 1, group=group, gather=gather)
        meta["methods"].append("sq")
        meta["configs"].append((cs, bits))
    else:
        cs = target_compression_ratio // features.element_size()
        if n_clusters > 256:
            cs *= 2
        table, cb = vq_compress_features(features, n_clusters, cs, hotness, seed=seed + 1, group=group, gather=gather, **fit_args)
        meta["methods"].append("vq")
        meta["configs"].append((cs, -1))
    meta["codebooks"].append(cb)
    meta["data"]["compression_data"] = (table.dtype, tuple(table.shape))
    meta["compression_data"] = table
    if group is not None and not gather:
        meta["row_range"] = split_plan(n, 1, *_split(group))[1]
    return meta


_TABLES = ("compression_data", "seeds_compression_data")


def save(meta, root):
    os.makedirs(root, exist_ok=True)
    small = {k: v for k, v in meta.items() if k not in _TABLES}
    small["codebooks"] = [c.cpu() for c in meta["codebooks"]]
    if "seeds" in small:
        small["seeds"] = small["seeds"].cpu()
    torch.save(small, os.path.join(root, "compression_meta.pt"))
    for name in _TABLES:
        if name in meta:
            torch.save(meta[name].cpu(), os.path.join(root, name + ".pt"))


def load(root, device="cuda"):
    meta = torch.load(os.path.join(root, "compression_meta.pt"), weights_only=False)
    for name in _TABLES:
        path = os.path.join(root, name + ".pt")
        if os.path.exists(path):
            meta[name] = torch.load(path, weights_only=False).to(device)
    meta["codebooks"] = [c.to(device) for c in meta["codebooks"]]
    if "seeds" in meta:
        meta["seeds"] = meta["seeds"].to(device)
    return meta


def to_manager(meta, num_nodes=None):
    """``sage.CompressionManager`` over the loaded artefact (tables by global node id; two-level: slot array from seeds)."""
    from . import sage
    tables, slot = [], None
    if len(meta["methods"]) >= 2 and meta["methods"] != ["sq", "vq"]:
        raise NotImplementedError("the single-launch two-level aggregation serves hot SQ rows over a VQ table")
    if len(meta["methods"]) >= 2:
        tables.append(meta["seeds_compression_data"])
        n = num_nodes if num_nodes is not None else meta["compression_data"].shape[0]
        slot = torch.full((n,), -1, dtype=torch.int32, device=meta["compression_data"].device)
        slot[meta["seeds"].long()] = torch.arange(meta["seeds"].numel(), dtype=torch.int32, device=slot.device)
    tables.append(meta["compression_data"])
    return sage.CompressionManager(meta["feat_dim"], meta["methods"], meta["configs"], meta["codebooks"], tables, slot)


def decompress(meta, level=-1):
    """Decoded fp32 matrix of one level of the artefact (for checks)."""
    method = meta["methods"][level]
    cb = meta["codebooks"][level]
    table = meta["compression_data"] if level in (-1, len(meta["methods"]) - 1) else meta["seeds_compression_data"]
    if method == "vq":
        return ops.vq_decompress(table, cb, meta["feat_dim"])
    cs, bits = meta["configs"][level]
    return ops.sq_decompress(table, cb, bits, cs, meta["feat_dim"])


__all__ = ["normalize", "sq_metadata", "split_plan", "gather_parts", "sq_compress_features", "vq_metadata", "vq_compress_features",
           "compress", "save", "load",
           "to_manager", "decompress"]
