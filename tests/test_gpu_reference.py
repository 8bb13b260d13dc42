"""GPU: side by side with the reference's own kernels (extension built by oracle/build_ref.py from the
unmodified reference sources) on larger seeded inputs than the fixtures hold.  Skipped when that
extension was not built."""
import numpy as np
import pytest

from helpers import sq_table, random_csc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref
    try:
        return build_ref.load()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"reference extension unavailable: {e}")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 16])
def test_sq_bit_exact_against_reference_kernels(capi, ref, oracle, bits):
    rng = np.random.default_rng(bits)
    D, cs, n_src = 128, 32, 20000
    x = torch.randn(n_src, D, device="cuda")
    cb = dev(oracle.sq_codebooks(x[:4000].cpu().numpy(), cs))
    a, b = capi.sq_compress(x, cb, bits, cs), ref.sq_compress(x, cb, bits, cs)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    stored = ref.packbits(b.to(torch.uint8), bits) if bits < 8 else b.to(torch.int8 if bits == 8 else torch.int16)
    if bits < 8:
        assert torch.equal(capi.packbits(b.to(torch.uint8), bits), stored)
        assert torch.equal(capi.unpackbits(stored, bits, D), ref.unpackbits(stored, bits, D))
    da, db = capi.sq_decompress(stored, cb, bits, cs, D), ref.sq_decompress(stored, cb, bits, cs, D)
    torch.cuda.synchronize()
    assert torch.equal(da.view(torch.int32), db.view(torch.int32))
    indptr, indices = random_csc(rng, 5000, n_src, max_deg=15)
    ip, ix = dev(indptr), dev(indices)
    fa = capi.sq_decompress_spmm_csr(stored, cb, ip, ix, bits, cs, D)
    fb = ref.sq_decompress_spmm_csr(stored, cb, ip, ix, bits, cs, D)
    torch.cuda.synchronize()
    assert torch.equal(fa.view(torch.int32), fb.view(torch.int32))
    assert torch.equal(capi.spmm_csr(da, ip, ix), ref.spmm_csr(db, ip, ix))


def test_vq_bit_exact_against_reference_kernels(capi, ref):
    rng = np.random.default_rng(0)
    cbs = torch.randn(16, 256, 8, device="cuda")
    codes = torch.randint(0, 256, (20000, 16), dtype=torch.uint8, device="cuda")
    indptr, indices = random_csc(rng, 5000, 20000, max_deg=15)
    ip, ix = dev(indptr), dev(indices)
    assert torch.equal(capi.vq_decompress(codes, cbs, 128), ref.vq_decompress(codes, cbs, 128))
    a = capi.vq_decompress_spmm_csr(codes, cbs, ip, ix, 128)
    b = ref.vq_decompress_spmm_csr(codes, cbs, ip, ix, 128)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
