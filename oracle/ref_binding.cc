// Python binding over the reference's OWN CUDA implementation files, compiled unmodified from
// the reference tree (see build_ref.py).  Test infrastructure only: the tier-2 oracle that the
// GPU parity tests compare this repository's kernels against, and the "reference on the same
// GPU" timing.  Nothing in the product imports it.  The functions bound are the kernel-level
// entry points the reference's gs::Graph methods call (src/graph.cc, src/batch_graph.cc).
#include <torch/extension.h>

#include "cuda/batch/batch_ops.h"
#include "cuda/fusion/column_row_slicing.h"
#include "cuda/fusion/fused_coo_e_div_u_sum.h"
#include "cuda/fusion/fused_coo_e_square_sum.h"
#include "cuda/fusion/fused_coo_u_op_v.h"
#include "cuda/fusion/fused_csc_e_div_u_sum.h"
#include "cuda/fusion/fused_csc_e_square_sum.h"
#include "cuda/fusion/fused_csc_u_op_v.h"
#include "cuda/fusion/node2vec.h"
#include "cuda/fusion/random_walk.h"
#include "cuda/fusion/slice_sampling.h"
#include "cuda/graph_ops.h"
#include "cuda/tensor_ops.h"
#include "bcast.h"
#include "graph_storage.h"
#include "cuda/sddmm.h"
#include "cuda/spmm.h"

namespace ri = gs::impl;

// SpMM / SDDMM take the reference's graph structs and its broadcast table (src/bcast.cc:24-76),
// built here the way Graph::SpMM / Graph::SDDMM do (src/graph.cc:320-379).
static void spmm_csc(const std::string& op, const std::string& reduce, torch::Tensor indptr,
                     torch::Tensor indices, torch::Tensor ufeat, torch::Tensor efeat, torch::Tensor out,
                     torch::Tensor argu, torch::Tensor arge) {
  auto csc = std::make_shared<gs::CSC>(gs::CSC{indptr, indices, torch::nullopt});
  ri::SpMMCSC(op, reduce, gs::CalcBcastOff(op, ufeat, efeat), csc, ufeat, efeat, out, {argu, arge});
}
static void spmm_coo(const std::string& op, const std::string& reduce, torch::Tensor row, torch::Tensor col,
                     torch::Tensor ufeat, torch::Tensor efeat, torch::Tensor out, int64_t u_target,
                     torch::Tensor argu, torch::Tensor arge) {
  auto coo = std::make_shared<gs::COO>(gs::COO{row, col, torch::nullopt, false, false});
  ri::SpMMCOO(op, reduce, gs::CalcBcastOff(op, ufeat, efeat), coo, ufeat, efeat, out, u_target, {argu, arge});
}
static void sddmm_coo(const std::string& op, torch::Tensor row, torch::Tensor col, torch::Tensor lhs,
                      torch::Tensor rhs, torch::Tensor out, int64_t lhs_target, int64_t rhs_target) {
  auto coo = std::make_shared<gs::COO>(gs::COO{row, col, torch::nullopt, false, false});
  ri::SDDMMCOO(op, gs::CalcBcastOff(op, lhs, rhs), coo, lhs, rhs, out, (int)lhs_target, (int)rhs_target);
}

// The fused edge operators as Graph::FusedUOPV / FusedESquareSum / FusedEDivUSum call them
// (src/graph.cc:341-356,457-503).
static void fused_u_op_v_coo(const std::string& op, torch::Tensor row, torch::Tensor col, torch::Tensor lhs1,
                             torch::Tensor rhs1, torch::Tensor out1, torch::Tensor lhs2, torch::Tensor rhs2,
                             torch::Tensor out2) {
  auto coo = std::make_shared<gs::COO>(gs::COO{row, col, torch::nullopt, false, false});
  ri::fusion::FUSED_COO_U_OP_V(op, gs::CalcBcastOff(op, lhs1, rhs1), coo, lhs1, rhs1, out1, lhs2, rhs2, out2);
}
static void fused_u_op_v_csc(const std::string& op, torch::Tensor indptr, torch::Tensor indices,
                             torch::Tensor lhs1, torch::Tensor rhs1, torch::Tensor out1, torch::Tensor lhs2,
                             torch::Tensor rhs2, torch::Tensor out2) {
  auto csc = std::make_shared<gs::CSC>(gs::CSC{indptr, indices, torch::nullopt});
  ri::fusion::FUSED_CSC_U_OP_V(op, gs::CalcBcastOff(op, lhs1, rhs1), csc, lhs1, rhs1, out1, lhs2, rhs2, out2);
}
static void e_square_sum_csc(const std::string& op, const std::string& reduce, torch::Tensor indptr,
                             torch::Tensor indices, torch::Tensor ufeat, torch::Tensor efeat, torch::Tensor out,
                             torch::Tensor argu, torch::Tensor arge) {
  auto csc = std::make_shared<gs::CSC>(gs::CSC{indptr, indices, torch::nullopt});
  ri::fusion::ESquareSumCSC(op, reduce, gs::CalcBcastOff(op, ufeat, efeat), csc, ufeat, efeat, out, {argu, arge});
}
static void e_square_sum_coo(const std::string& op, const std::string& reduce, torch::Tensor row,
                             torch::Tensor col, torch::Tensor ufeat, torch::Tensor efeat, torch::Tensor out,
                             torch::Tensor argu, torch::Tensor arge) {
  auto coo = std::make_shared<gs::COO>(gs::COO{row, col, torch::nullopt, false, false});
  ri::fusion::ESquareSumCOO(op, reduce, gs::CalcBcastOff(op, ufeat, efeat), coo, ufeat, efeat, out, {argu, arge});
}
static void e_div_u_sum_csc(const std::string& op, const std::string& reduce, torch::Tensor indptr,
                            torch::Tensor indices, torch::Tensor ufeat, torch::Tensor efeat, torch::Tensor out,
                            torch::Tensor argu, torch::Tensor arge) {
  auto csc = std::make_shared<gs::CSC>(gs::CSC{indptr, indices, torch::nullopt});
  ri::fusion::EDivUSumCSC(op, reduce, gs::CalcBcastOff(op, ufeat, efeat), csc, ufeat, efeat, out, {argu, arge});
}
static void e_div_u_sum_coo(const std::string& op, const std::string& reduce, torch::Tensor row,
                            torch::Tensor col, torch::Tensor ufeat, torch::Tensor efeat, torch::Tensor out,
                            torch::Tensor argu, torch::Tensor arge) {
  auto coo = std::make_shared<gs::COO>(gs::COO{row, col, torch::nullopt, false, false});
  ri::fusion::EDivUSumCOO(op, reduce, gs::CalcBcastOff(op, ufeat, efeat), coo, ufeat, efeat, out, {argu, arge});
}

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
  m.def("sample_cols_probs", &ri::CSCColSamplingProbsCUDA);               // src/cuda/sampling_probs.cu:23-281
  m.def("list_sampling", &ri::ListSamplingCUDA);                          // src/cuda/list_sampling.cu:20-73
  m.def("list_sampling_probs", &ri::ListSamplingProbsCUDA);               // src/cuda/list_sampling_probs.cu:11-89
  m.def("batch_list_sampling_probs", &ri::batch::BatchListSamplingProbsCUDA);  // src/cuda/batch/list_sampling_probs.cu:29-107
  m.def("spmm_csc", &spmm_csc);                                           // src/cuda/spmm.cu:253-348
  m.def("spmm_coo", &spmm_coo);                                           // src/cuda/spmm.cu:170-250
  m.def("sddmm_coo", &sddmm_coo);                                         // src/cuda/sddmm.cu:120-200
  m.def("sort_indices", &ri::SortIndicesCUDA);                            // src/cuda/sort_indices.cu:11-37
  m.def("fused_u_op_v_coo", &fused_u_op_v_coo);                           // src/cuda/fusion/fused_coo_u_op_v.cu:21-137
  m.def("fused_u_op_v_csc", &fused_u_op_v_csc);                           // src/cuda/fusion/fused_csc_u_op_v.cu:21-150
  m.def("e_square_sum_csc", &e_square_sum_csc);                           // src/cuda/fusion/fused_csc_e_square_sum.cu
  m.def("e_square_sum_coo", &e_square_sum_coo);                           // src/cuda/fusion/fused_coo_e_square_sum.cu
  m.def("e_div_u_sum_csc", &e_div_u_sum_csc);                             // src/cuda/fusion/fused_csc_e_div_u_sum.cu
  m.def("e_div_u_sum_coo", &e_div_u_sum_coo);                             // src/cuda/fusion/fused_coo_e_div_u_sum.cu
}
