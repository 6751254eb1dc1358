// Python binding over the reference's OWN CUDA implementation files, compiled unmodified from
// the reference tree (see build_ref.py).  Test infrastructure only: the tier-2 oracle that the
// GPU parity tests compare this repository's kernels against, and the "reference on the same
// GPU" timing.  Nothing in the product imports it.  The functions bound are the kernel-level
// entry points the reference's gs::Graph methods call (src/graph.cc, src/batch_graph.cc).
#include <torch/extension.h>

#include "cuda/batch/batch_ops.h"
#include "cuda/fusion/column_row_slicing.h"
#include "cuda/fusion/node2vec.h"
#include "cuda/fusion/random_walk.h"
#include "cuda/fusion/slice_sampling.h"
#include "cuda/graph_ops.h"
#include "cuda/tensor_ops.h"

namespace ri = gs::impl;

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("slice_cols", &ri::OnIndptrSlicingCUDA);                         // src/cuda/slicing.cu:100-181
  m.def("slice_rows_on_indices", &ri::OnIndicesSlicingCUDA);             // src/cuda/slicing.cu:184-308
  m.def("batch_slice_cols", &ri::batch::BatchOnIndptrSlicingCUDA);       // src/cuda/batch/slicing.cu:11-120
  m.def("sample_cols", &ri::CSCColSamplingCUDA);                         // src/cuda/sampling.cu:17-172
  m.def("fused_slice_sample", &ri::fusion::FusedCSCColSlicingSamplingCUDA);  // src/cuda/fusion/slice_sampling.cu:13-177
  m.def("tensor_unique", &ri::TensorUniqueCUDA);                         // src/cuda/unique_reindex.cu:174-177
  m.def("tensor_relabel", &ri::TensorRelabelCUDA);                       // src/cuda/unique_reindex.cu:179-199
  m.def("batch_coo_relabel", &ri::batch::BatchCOORelabelCUDA);           // src/cuda/batch/batch_relabel.cu:376-499
  m.def("random_walk", &ri::fusion::FusedRandomWalkCUDA);                // src/cuda/fusion/random_walk.cu:10-70
  m.def("node2vec", &ri::fusion::FusedNode2VecCUDA);                     // src/cuda/fusion/node2vec.cu:20-162
  m.def("col_row_slicing", &ri::fusion::CSCColRowSlicingCUDA);           // src/cuda/fusion/column_row_slicing.cu:154-216
  m.def("batch_col_row_slicing", &ri::fusion::BatchCSCColRowSlicingCUDA);  // :266-362
}
