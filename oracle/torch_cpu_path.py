"""TEST / BENCHMARK INFRASTRUCTURE ONLY - the reference's PyTorch-level CPU path for the fused operator,
timed on the host cores as the CPU baseline.  It is the reference's own torch restatement of its
kernels, applied the way its unfused pipeline does (examples/compress.py:58-72 gathers the rows of the
block's input nodes and decodes them; examples/conv.py:53-54 then aggregates):

  1. gather the compressed rows of the block's distinct source nodes;
  2. decode - SQ: shift/mask unpack in the bit order of src/packbits.cu:34-39, then
     sign * exp2(|c+0.5| * (emax-emin)/2^(bits-1) + emin), 1 bit: +-mean (tests/test_sq.py:75-111);
     VQ: index_select per codebook + cat (tests/test_vq.py:17-19,63-65);
  3. mean-aggregate with a CSR sparse matrix of 1/max(deg,1) weights times the decoded rows.

Never imported by the product package.
"""
import torch


def unpack_rows(packed_u8, bits, feat_dim):
    """[rows, ceil(D*bits/8)] uint8 -> [rows, D] uint8; element i of a byte at bit offset bits*i."""
    per = 8 // bits
    shifts = (torch.arange(per, dtype=torch.uint8) * bits).view(1, 1, per)
    u = (packed_u8.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return u.reshape(packed_u8.shape[0], -1)[:, :feat_dim]


def sq_decode_rows(stored, codebooks, bits, column_slice, feat_dim):
    if bits < 8:
        c = unpack_rows(stored.view(torch.uint8), bits, feat_dim).to(torch.float32)
    else:
        c = stored[:, :feat_dim].to(torch.float32)
    idx = torch.arange(feat_dim) // column_slice
    emin, emax, mean = codebooks[idx, 2], codebooks[idx, 3], codebooks[idx, 4]
    if bits == 1:
        return (c - 0.5) * (2 * mean)
    drange = float(2 ** (bits - 1))
    if bits < 8:
        c = c - drange
    c = c + 0.5
    sign = torch.where(c >= 0, 1.0, -1.0)
    return torch.exp2(c.abs() * ((emax - emin) / drange) + emin) * sign


def vq_decode_rows(codes, codebooks, feat_dim):
    parts = [torch.index_select(codebooks[s], 0, codes[:, s].long()) for s in range(codebooks.shape[0])]
    return torch.cat(parts, dim=1)[:, :feat_dim]


def mean_aggregate(decoded, indptr, local_indices, n_dst):
    deg = (indptr[1:] - indptr[:-1]).clamp_min(1).to(torch.float32)
    vals = torch.repeat_interleave(1.0 / deg, indptr[1:] - indptr[:-1])
    A = torch.sparse_csr_tensor(indptr, local_indices, vals, size=(n_dst, decoded.shape[0]))
    return A @ decoded


def relabel(indices):
    src, local = torch.unique(indices, return_inverse=True)
    return src, local


def sq_spmm(table, codebooks, indptr, indices, bits, column_slice, feat_dim):
    src, local = relabel(indices)
    decoded = sq_decode_rows(table[src], codebooks, bits, column_slice, feat_dim)
    return mean_aggregate(decoded, indptr, local, indptr.numel() - 1)


def vq_spmm(table, codebooks, indptr, indices, feat_dim):
    src, local = relabel(indices)
    return mean_aggregate(vq_decode_rows(table[src], codebooks, feat_dim), indptr, local, indptr.numel() - 1)
