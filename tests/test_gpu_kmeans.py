"""GPU parity: pairwise distance and k-means assignment against the oracle (the reference's torch
restatement, examples/my_kmeans.py:43-64,116-125, evaluated in double)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def labels_match(oracle, x, c, metric, got):
    """Identical assignments, ignoring ties: where the label differs from the oracle's, the chosen
    centre must be as close as the best one up to fp32 rounding of the distance."""
    want, best, second = oracle.kmeans_assign(x, c, metric, with_margin=True)
    diff = np.nonzero(got != want)[0]
    if diff.size == 0:
        return True
    d = oracle.pairwise_distance(x[diff], c, metric).astype(np.float64)
    chosen = d[np.arange(diff.size), got[diff]]
    scale = np.maximum(np.abs(best[diff]), 1e-30) if metric != "cosine" else 1.0
    ok = np.abs(chosen - best[diff]) <= 4e-6 * scale + 1e-7
    return bool(ok.all()) and diff.size <= max(3, x.shape[0] // 2000)


@pytest.mark.parametrize("metric", ["l2", "cosine"])
@pytest.mark.parametrize("n,k,d", [(1000, 256, 8), (777, 256, 32), (513, 256, 64), (300, 17, 5), (64, 300, 100), (50, 40, 200), (1, 1, 1)])
def test_pairwise_distance(capi, oracle, metric, n, k, d):
    rng = np.random.default_rng(n + k + d)
    x = rng.standard_normal((n, d)).astype(np.float32)
    c = rng.standard_normal((k, d)).astype(np.float32)
    got = capi.pairwise_distance(dev(x), dev(c), metric).cpu().numpy()
    want = oracle.pairwise_distance(x, c, metric)
    assert got.shape == (n, k)
    assert np.allclose(got, want, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("metric", ["l2", "cosine"])
@pytest.mark.parametrize("n,k,d", [(20000, 256, 8), (9999, 256, 32), (5000, 256, 64), (3000, 17, 5), (700, 300, 100), (300, 40, 200)])
def test_kmeans_assign_identical_up_to_ties(capi, oracle, metric, n, k, d):
    rng = np.random.default_rng(n + k + d + 1)
    x = rng.standard_normal((n, d)).astype(np.float32)
    c = rng.standard_normal((k, d)).astype(np.float32)
    km = capi.KMeans(dev(c), metric)
    got = km.predict(dev(x)).cpu().numpy()
    assert got.dtype == np.int64 and got.shape == (n,)
    assert labels_match(oracle, x, c, metric, got)
    assert km.get_centers().data_ptr() == km.cluster_centers.data_ptr()


def test_kmeans_exact_ties_take_first_centre(capi):
    c = torch.randn(8, 16, device="cuda")
    c2 = torch.cat([c, c])  # every centre duplicated: the first copy must win
    x = torch.randn(500, 16, device="cuda")
    for metric in ("l2", "cosine"):
        lab = capi.KMeans(c2, metric).predict(x)
        assert int(lab.max()) < 8


def test_kmeans_zero_vectors_and_fit(capi):
    x = torch.randn(4000, 8, device="cuda")
    x[:5] = 0
    c = torch.randn(16, 8, device="cuda")
    d = capi.pairwise_distance(x, c, "cosine")
    assert torch.all(d[:5] == 1.0)  # NaN distances count as 1 (examples/my_kmeans.py:92-94)
    torch.manual_seed(0)
    for metric in ("l2", "cosine"):
        km = capi.KMeans(16, 8, metric, max_iter=30)
        km.fit(x)
        centers = km.get_centers()
        assert centers.shape == (16, 8) and bool(torch.isfinite(centers).all())
        lab = km.predict(x)
        # a fit must beat random centres on its own objective
        def inertia(cc, ll):
            if metric == "cosine":
                return float((1 - torch.nn.functional.cosine_similarity(x[5:], cc[ll[5:]], dim=1)).sum())
            return float(((x - cc[ll]) ** 2).sum())
        rnd = x[torch.randperm(4000, device="cuda")[:16]].contiguous()
        assert inertia(centers, lab) < inertia(rnd, capi.KMeans(rnd, metric).predict(x))


@pytest.mark.parametrize("metric", ["l2", "cosine"])
@pytest.mark.parametrize("n,k,d", [(100_000, 256, 8), (50_000, 256, 32), (30_000, 256, 64), (4097, 100, 5), (1000, 16, 24), (129, 256, 8),
                                   (20_000, 256, 40), (20_000, 200, 49), (10_000, 64, 33)])
def test_tensor_core_assignment_equals_exact_fp32_kernel(capi, oracle, metric, n, k, d):
    """The tcgen05 path must return the labels of the exact fp32 scorer, point for point: points it cannot
    decide within the error bound of the split product are re-scored by that scorer."""
    from f2cgt_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(n + k + d)
    x = torch.randn(n, d, device="cuda", generator=g)
    c = torch.randn(k, d, device="cuda", generator=g)
    x[:3] = 0                      # zero vectors: every distance ties
    c2 = c.clone()
    if k >= 8:
        c2[k // 2] = c2[1]         # an exact duplicate centre: the lower index must win
    for centers in (c, c2):
        tc = ops.kmeans_assign(x, centers, metric, scorer="tensor")  # the tensor-core path whatever the shape heuristic says
        undecided = ops.kmeans_assign.last_undecided
        exact = ops.kmeans_assign(x, centers, metric, scorer="exact")
        assert torch.equal(tc, exact), (metric, n, k, d, int((tc != exact).sum()))
        # the split product (3 x tf32 up to d = 32, 3 x bf16 up to d = 64) decides almost everything itself
        # (a duplicated centre makes every point that prefers it an exact tie: about 1/k of the points)
        assert undecided <= (0.02 if d <= 32 else 0.05) * n + 8 + (3.0 * n / k if centers is c2 else 0)
        if centers is c:
            assert labels_match(oracle, x.cpu().numpy(), c.cpu().numpy(), metric, tc.cpu().numpy())


@pytest.mark.parametrize("d", [8, 32, 64])
def test_tensor_core_assignment_at_table_scale(capi, d):
    """The sizes the k-means profile times: 2,449,029 sub-vectors against 256 centres (one VQ subspace of the
    2.4 M-row table), tensor-core labels == exact-scorer labels point for point, both metrics."""
    from f2cgt_b200 import ops
    n, k = 2_449_029, 256
    g = torch.Generator(device="cuda").manual_seed(d)
    x = torch.randn(n, d, device="cuda", generator=g)
    c = torch.randn(k, d, device="cuda", generator=g)
    for metric in ("l2", "cosine"):
        tc = ops.kmeans_assign(x, c, metric, scorer="tensor")
        assert ops.kmeans_assign.last_undecided <= (0.02 if d <= 32 else 0.05) * n
        exact = ops.kmeans_assign(x, c, metric, scorer="exact")
        assert torch.equal(tc, exact), (metric, d, int((tc != exact).sum()))
