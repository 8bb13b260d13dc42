"""Stand-in for the two operators of the reference's (absent, un-vendored) ShmTensor submodule that sit on the
minibatch path (examples/dataloader.py:174-177 of gpzlx1/F2CGT): ``csr_sampling`` and ``tensor_relabel``, served by the
B200 library.  The rest of ShmTensor (shared-memory tensors, UVA fetch, GPU cache) is outside the path."""
from f2cgt_b200.ops import csr_sampling, tensor_relabel  # noqa: F401
