// TEST INFRASTRUCTURE ONLY - never imported by the product path.
//
// Binding file for the UNMODIFIED reference CUDA sources (src/sq_quantization.cu,
// src/vq_quantization.cu, src/packbits.cu, src/fusion_spmm.cu, src/fusion_dropout.cu of
// gpzlx1/F2CGT), which are compiled where they lie in the read-only reference checkout by
// oracle/build_ref.py.  The reference's own binding file (src/pybind.cu) cannot be used because it
// also binds the RAFT-backed k-means wrappers, and RAFT is not available offline.  This file only
// declares the functions the reference sources define and exposes them under the reference's
// Python names, so fixtures produced through it are outputs of the reference's own kernels.
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "cuda_operators.h"  // reference header: prototypes of the bound operators

// Defined in the reference's src/fusion_dropout.cu:21 but missing from its header.
torch::Tensor dropout_inplace(torch::Tensor output, float p, bool is_training);

PYBIND11_MODULE(f2cgt_ref, m) {
  m.def("packbits", &packbits, py::arg("unpack"), py::arg("target_bits"));
  m.def("unpackbits", &unpackbits, py::arg("pack"), py::arg("target_bits"), py::arg("unpack_dim"));
  m.def("sq_compress", &sq_compress, py::arg("src"), py::arg("codebooks"), py::arg("target_bits"),
        py::arg("column_slice"));
  m.def("sq_decompress", &sq_decompress, py::arg("compress_data"), py::arg("codebooks"),
        py::arg("target_bits"), py::arg("column_slice"), py::arg("feat_dim"));
  m.def("vq_decompress", &vq_decompress, py::arg("index_tensor"), py::arg("codebooks"),
        py::arg("feat_dim"));
  m.def("spmm_csr", &SpMMCsr, py::arg("feat"), py::arg("indptr"), py::arg("indices"));
  m.def("vq_decompress_spmm_csr", &VqDecompressSpMMFusionCsr, py::arg("compress_feat"),
        py::arg("codebooks"), py::arg("indptr"), py::arg("indices"), py::arg("feat_dim"));
  m.def("sq_decompress_spmm_csr", &SqDecompressSpMMFusionCsr, py::arg("compress_feat"),
        py::arg("codebooks"), py::arg("indptr"), py::arg("indices"), py::arg("target_bit"),
        py::arg("column_slice"), py::arg("feat_dim"));
  m.def("dropout_inplace", &dropout_inplace, py::arg("output"), py::arg("p"),
        py::arg("is_training"));
}
