"""Shared helpers of the test-suite: seeded inputs and comparison rules."""
import numpy as np


def ulp_diff(a, b):
    """Distance in units in the last place between two float32 arrays (same shape)."""
    a = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    b = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    a = np.where(a < 0, np.int64(-2**31) - a, a)
    b = np.where(b < 0, np.int64(-2**31) - b, b)
    return np.abs(a - b)


def random_csc(rng, n_dst, n_src, max_deg=12, empty_every=7, dtype=np.int64):
    deg = rng.integers(0, max_deg + 1, n_dst)
    if empty_every:
        deg[::empty_every] = 0
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(dtype)
    indices = rng.integers(0, n_src, int(indptr[-1])).astype(dtype)
    return indptr, indices


def sq_table(O, rng, rows, D, bits, column_slice, scale=1.0):
    """Seeded features -> codebooks (reference recipe) -> stored codes, all through the oracle."""
    x = (rng.standard_normal((rows, D)) * scale).astype(np.float32)
    cb = O.sq_codebooks(x, column_slice)
    stored = O.sq_codes_to_storage(O.sq_compress(x, cb, bits, column_slice), bits)
    return x, cb, stored


# tolerance of the aggregated outputs named by the task: 1e-5 relative / 1e-6 absolute in fp32
AGG_RTOL, AGG_ATOL = 1e-5, 1e-6
# decoded SQ values go through exp2f: GPU libdevice vs host libm may differ in the last bits
SQ_MAX_ULP = 2
