"""Offline feature compressor and the artefact format the trainer loads - the flow of the reference's
examples/process_compress.py on top of the library's operators (one process; the reference additionally splits
columns / rows over ranks, which changes who computes a slice, not the result format):

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


def sq_metadata(sample):
    """One codebook row from a sample of one column slice (examples/process_compress.py:43-68)."""
    eps = 1e-5
    a = sample.float().abs().flatten()
    q = torch.quantile(a[:min(a.numel(), 1 << 24)].double(), torch.tensor([0.005, 0.995], dtype=torch.float64, device=a.device))
    fmin = max(float(q[0]), eps)
    fmax = max(float(q[1]), 2 * eps)
    mean = float(a.mean())
    if mean < 0.1:
        mean += 0.1
    # emin / emax are float32 values in the reference (torch.log2 of a float32 tensor, then + epsilon)
    emin = float(torch.log2(torch.tensor(fmin, dtype=torch.float32)))
    emax = float(torch.log2(torch.tensor(fmax, dtype=torch.float32)) + eps)
    return [fmin, fmax, emin, emax, mean]


def sq_compress_features(features, target_bits, column_slice, hotness=None, sample_size=250_000, batch_rows=1_000_000, seed=0):
    """features [n, D] (any float dtype, on the GPU) -> (stored codes, codebooks [ceil(D / column_slice), 5])."""
    n, D = features.shape
    gen = torch.Generator(device=features.device)
    gen.manual_seed(seed)
    rows = []
    for b in range(0, D, column_slice):
        idx = _sample_rows(n, sample_size, hotness, gen)
        rows.append(sq_metadata(features[idx, b:b + column_slice]))
    codebooks = torch.tensor(rows, dtype=torch.float32, device=features.device)
    parts = []
    for s in range(0, n, batch_rows):
        x = features[s:s + batch_rows].float().contiguous()
        c = ops.sq_compress(x, codebooks, target_bits, column_slice)
        if target_bits < 8:
            parts.append(ops.packbits(c.to(torch.uint8), target_bits).view(torch.int8))  # stored as int8 (:109-111,141)
        elif target_bits == 8:
            parts.append(c.to(torch.int8))
        else:
            parts.append(c.to(torch.int16))
    return torch.cat(parts), codebooks


def vq_metadata(features, n_clusters, column_slice, hotness=None, sample_size=150_000, seed=0, max_iter=300, tol=5e-2):
    n, D = features.shape
    gen = torch.Generator(device=features.device)
    gen.manual_seed(seed)
    idx = _sample_rows(n, sample_size, hotness, gen)
    num_slice = (D + column_slice - 1) // column_slice
    codebooks = torch.zeros((num_slice, n_clusters, column_slice), dtype=torch.float32, device=features.device)
    for i in range(num_slice):
        b, e = i * column_slice, min((i + 1) * column_slice, D)
        data = features[idx, b:e].float()
        dist = data.norm(dim=1, p=2)
        rim = torch.quantile(dist, min(1.0, 0.00625 * (data.shape[1] / 8)))
        data = data[dist >= rim].contiguous()
        km = ops.KMeans(n_clusters, data.shape[1], "cosine", max_iter=max_iter, tol=tol)
        torch.manual_seed(seed * 1000 + i)  # KMeans.fit draws its initial centres from torch's generator
        km.fit(data)
        codebooks[i, :, :e - b] = normalize(km.get_centers())
    if torch.isnan(codebooks).any():
        raise ValueError("codebooks has nan")
    return codebooks


def vq_compress_features(features, n_clusters, column_slice, hotness=None, batch_rows=1_000_000, seed=0, **fit_args):
    n, D = features.shape
    codebooks = vq_metadata(features, n_clusters, column_slice, hotness, seed=seed, **fit_args)
    num_slice = codebooks.shape[0]
    dtype = torch.uint8 if n_clusters <= 256 else torch.int16
    if n_clusters > 32767:
        raise ValueError("the kernels address at most 32767 centres per slice (int16 codes)")
    codes = torch.empty((n, num_slice), dtype=dtype, device=features.device)
    for s in range(0, n, batch_rows):
        for i in range(num_slice):
            b, e = i * column_slice, min((i + 1) * column_slice, D)
            data = torch.zeros((min(batch_rows, n - s), column_slice), dtype=torch.float32, device=features.device)
            data[:, :e - b] = features[s:s + batch_rows, b:e].float()
            labels = ops.kmeans_assign(data, codebooks[i].contiguous(), "cosine")
            codes[s:s + batch_rows, i] = labels.to(dtype)
    return codes, codebooks


def compress(features, seeds=None, hotness=None, target_compression_ratio=32, n_clusters=256, world_size=1, seed=0, **fit_args):
    """The decision logic of examples/process_compress.py:295-394.  Returns the meta dictionary with the tables added
    under ``compression_data`` / ``seeds_compression_data``."""
    n, feat_dim = features.shape
    elem_bits = features.element_size() * 8
    meta = dict(methods=[], codebooks=[], configs=[], feat_dim=feat_dim, data={})

    def sq_slice():
        cs = (feat_dim + world_size - 1) // world_size
        return (cs + 7) // 8 * 8

    if seeds is not None:
        bits = elem_bits // 8
        cs = sq_slice()
        table, cb = sq_compress_features(features[seeds], bits, cs, None, seed=seed)
        meta["methods"].append("sq")
        meta["configs"].append((cs, bits))
        meta["codebooks"].append(cb)
        meta["data"]["seeds_compression_data"] = (table.dtype, tuple(table.shape))
        meta["seeds"] = seeds
        meta["seeds_compression_data"] = table
    if target_compression_ratio <= elem_bits:
        bits = int(elem_bits / target_compression_ratio)
        cs = sq_slice()
        table, cb = sq_compress_features(features, bits, cs, hotness, seed=seed + 1)
        meta["methods"].append("sq")
        meta["configs"].append((cs, bits))
    else:
        cs = target_compression_ratio // features.element_size()
        if n_clusters > 256:
            cs *= 2
        table, cb = vq_compress_features(features, n_clusters, cs, hotness, seed=seed + 1, **fit_args)
        meta["methods"].append("vq")
        meta["configs"].append((cs, -1))
    meta["codebooks"].append(cb)
    meta["data"]["compression_data"] = (table.dtype, tuple(table.shape))
    meta["compression_data"] = table
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


__all__ = ["normalize", "sq_metadata", "sq_compress_features", "vq_metadata", "vq_compress_features", "compress", "save", "load",
           "to_manager", "decompress"]
