"""Drop-in for the reference's extension module: ``import F2CGTLib as capi`` (examples/conv.py:6,
tests/test_sq.py:3 of gpzlx1/F2CGT) resolves to the B200 implementation in ``f2cgt_b200.ops``."""
from f2cgt_b200.ops import (KMeans, dropout_inplace, fusion_decompress, kmeans_assign, packbits,  # noqa: F401
                            pairwise_distance, sq_compress, sq_decompress, sq_decompress_spmm_csr, spmm_csr,
                            two_level_decompress_spmm_csr, unpackbits, vq_decompress, vq_decompress_spmm_csr)
