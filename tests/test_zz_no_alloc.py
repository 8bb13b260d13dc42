"""GPU: the allocation-free k-means entry point against the regular one, through the C ABI.

`f2c_kmeans_assign_static` is for callers that cannot hand the library a device buffer - a worker thread next
to a framework allocator that already owns the GPU's memory, or a latency-critical path where an allocator
call would stall the device - so its scratch is a fixed array inside the library.  It must return exactly the
labels of `f2c_kmeans_assign` with a caller workspace.  Two calls in a row, the second smaller than the first,
also show that what one call leaves in the shared array does not leak into the next.  (This file is named so
that it is collected last: a run that stops at the first failure has then already run everything else.)"""
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _regular(lib, x, c, metric):
    n, d = x.shape
    k = c.shape[0]
    labels = torch.empty(n, dtype=torch.int64, device="cuda")
    ws = torch.zeros(lib.f2c_kmeans_assign_workspace(n, k, d), dtype=torch.uint8, device="cuda")
    rc = lib.f2c_kmeans_assign(x.data_ptr(), c.data_ptr(), labels.data_ptr(), n, k, d, metric, ws.data_ptr(), 0)
    assert rc == 0, lib.f2c_last_error()
    torch.cuda.synchronize()
    return labels


def _static(lib, x, c, metric):
    import ctypes
    n, d = x.shape
    labels = torch.full((n,), -1, dtype=torch.int64, device="cuda")
    rc = lib.f2c_kmeans_assign_static(x.data_ptr(), c.data_ptr(), labels.data_ptr(), n, c.shape[0], d, metric, 0)
    assert rc == 0, lib.f2c_last_error()
    # the caller cannot read the built-in array; the status call copies its header out after the stream has drained
    undecided, error = ctypes.c_int32(-1), ctypes.c_int32(-1)
    rc = lib.f2c_kmeans_assign_static_status(ctypes.byref(undecided), ctypes.byref(error), 0)
    assert rc == 0, lib.f2c_last_error()
    assert error.value == 0, "a bounded wait of the tensor-core kernel ran out"
    assert undecided.value >= 1, "the duplicated centre must leave exact ties to the exact scorer"
    return labels


def test_static_scratch_entry_point_matches_the_regular_one():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from f2cgt_b200 import _lib
    lib = _lib.lib
    g = torch.Generator(device="cuda").manual_seed(7)
    # d >= 16 so that the regular entry point also takes the tensor-core kernel with its scratch list
    for n, k, d, metric in ((300_000, 256, 32, _lib.L2), (70_001, 200, 16, _lib.COSINE)):
        x = torch.randn(n, d, device="cuda", generator=g)
        c = torch.randn(k, d, device="cuda", generator=g)
        c[k // 2] = c[3]  # a duplicated centre: exact ties land in the scratch list
        want = _regular(lib, x, c, metric)
        got = _static(lib, x, c, metric)
        assert torch.equal(got, want)
    # beyond the built-in capacity the call is refused with a clear message, nothing is launched
    big = (1 << 20) + 1
    rc = lib.f2c_kmeans_assign_static(x.data_ptr(), c.data_ptr(), got.data_ptr(), big, 200, 16, _lib.L2, 0)
    assert rc == 4 and b"exceed" in lib.f2c_last_error()
