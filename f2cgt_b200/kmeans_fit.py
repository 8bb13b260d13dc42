"""Lloyd iterations for ``KMeans.fit`` (reference: RAFT ``kmeans::fit`` behind src/kmeans.cu:61-75, and
the torch loop around ``capi.pairwise_distance`` in examples/my_kmeans.py:73-113).

The assignment step - the n*k*d contraction - is the library's k-means kernel; torch only does the
O(n*d) centre update and the k-means++ / random initialisation.  Initial centres are random, so a fit
is comparable with the reference's by inertia only, never label by label.
"""
import torch

from . import ops


def _init_random(x, k, gen):
    # examples/my_kmeans.py:27-31: k distinct non-zero rows
    nz = (x != 0).any(dim=1).nonzero().squeeze(1)
    if nz.numel() < k:
        raise RuntimeError(f"KMeans.fit: need at least {k} non-zero rows, have {nz.numel()}")
    pick = nz[torch.randperm(nz.numel(), generator=gen, device=x.device)[:k]]
    return x[pick].clone()


def _init_kmeanspp(x, k, gen):
    n = x.shape[0]
    centers = torch.empty((k, x.shape[1]), dtype=torch.float32, device=x.device)
    first = int(torch.randint(0, n, (1,), generator=gen, device=x.device).item())
    centers[0] = x[first]
    d2 = ops.pairwise_distance(x, centers[:1].contiguous(), "l2").squeeze(1)
    for c in range(1, k):
        probs = d2.clamp_min(0)
        if float(probs.sum()) <= 0:
            probs = torch.ones_like(probs)
        nxt = int(torch.multinomial(probs, 1, generator=gen).item())
        centers[c] = x[nxt]
        d2 = torch.minimum(d2, ops.pairwise_distance(x, centers[c:c + 1].contiguous(), "l2").squeeze(1))
    return centers


def _update(x, labels, centers):
    """Mean of every cluster's points, deterministically (a scatter-add would sum in whatever order its atomics land, and
    a fit would not be reproducible): points sorted by label, float64 prefix sums, one difference per cluster."""
    k = centers.shape[0]
    order = torch.argsort(labels, stable=True)
    csum = torch.cumsum(x[order].double(), dim=0)
    cnt = torch.bincount(labels, minlength=k)
    end = torch.cumsum(cnt, 0)                      # one past the last point of every cluster, in sorted order
    zero = torch.zeros((1, x.shape[1]), dtype=torch.float64, device=x.device)
    padded = torch.cat([zero, csum], dim=0)         # padded[j] = sum of the first j sorted points
    sums = (padded[end] - padded[end - cnt]).float()
    cntf = cnt.to(torch.float32).unsqueeze(1)
    # empty clusters keep their previous centre (examples/my_kmeans.py:133-144)
    return torch.where(cntf > 0, sums / cntf.clamp_min(1), centers)


def _inertia(x, labels, centers, metric):
    c = centers[labels]
    if metric == "cosine":
        return float((1 - torch.nn.functional.cosine_similarity(x, c, dim=1)).sum())
    return float(((x - c) ** 2).sum())


def lloyd_fit(x, k, metric, init, init_centers, max_iter, tol, n_init, seed=None):
    gen = torch.Generator(device=x.device)
    gen.manual_seed(torch.initial_seed() if seed is None else seed)
    best, best_inertia = None, float("inf")
    for _ in range(max(1, n_init if init != "array" else 1)):
        if init == "array":
            centers = init_centers.float().clone()
        elif init == "random":
            centers = _init_random(x, k, gen)
        else:
            centers = _init_kmeanspp(x, k, gen)
        labels = None
        for _it in range(max_iter):
            labels = ops.kmeans_assign(x, centers.contiguous(), metric)
            new_centers = _update(x, labels, centers)
            shift = float(((new_centers - centers) ** 2).sum())
            centers = new_centers
            if shift <= tol:
                break
        labels = ops.kmeans_assign(x, centers.contiguous(), metric)
        inertia = _inertia(x, labels, centers, metric)
        if inertia < best_inertia:
            best, best_inertia = centers, inertia
    return best
