// Operators of gsb_host::Graph beyond slicing / sampling / relabel: the
// whole-sampler entry point, and the compute / walk operators.
#include <c10/cuda/CUDAGuard.h>

#include "graph.h"
#include "gsb200.h"
#include "ops.h"

namespace gsb_host {

static const int64_t* P(const torch::Tensor& t) { return t.data_ptr<int64_t>(); }

// L-layer GraphSAGE super-batch sampler in ONE call: the operator sequence
// A[:, seeds::ptr] -> individual_sampling(K) -> all_nodes -> to_dgl_block per
// layer (examples/graphsage/graphsage_e2e.py:37-44 in gSampler) with every
// intermediate size kept on the device.  Returns 9 tensors per layer
// (sub_indptr, rows, cols, select, edge_ptr, unique, unique_ptr, block_row,
// block_col), narrowed to their live sizes, followed by one CPU int64 tensor
// [3*L] = {S_l, E_l, U_l}.  The single synchronisation is the read of those
// counts at the end.
std::vector<torch::Tensor> Graph::BatchGraphSAGE(torch::Tensor seeds, torch::Tensor seeds_ptr,
                                                 std::vector<int64_t> fanouts) {
  CreateSparseFormat(kCSC);
  TORCH_CHECK(!csc_->e_ids.has_value(), "BatchGraphSAGE expects a CSC without edge-id indirection");
  CheckIds(seeds, "seeds");
  CheckIds(seeds_ptr, "seeds_ptr");
  c10::cuda::CUDAGuard guard(seeds.device());
  const int L = (int)fanouts.size();
  const int64_t B = seeds_ptr.numel() - 1, S0 = seeds.numel();
  TORCH_CHECK(L >= 1 && B >= 1, "need at least one layer and one minibatch");
  auto opt = torch::dtype(torch::kInt64).device(seeds.device());
  std::vector<gsb_layer_buffers> bufs((size_t)L);
  std::vector<torch::Tensor> keep;
  int64_t S_cap = S0;
  const int64_t nnz = csc_->indices.numel();
  for (int l = 0; l < L; ++l) {
    TORCH_CHECK(fanouts[l] >= 1, "fanout must be positive");
    int64_t E_cap = S_cap * fanouts[l];
    gsb_layer_buffers& b = bufs[(size_t)l];
    b.S_cap = S_cap;
    b.E_cap = E_cap;
    auto mk = [&](int64_t n) { keep.push_back(torch::empty({n}, opt)); return keep.back().data_ptr<int64_t>(); };
    b.sub_indptr = mk(S_cap + 1);
    b.rows = mk(E_cap);
    b.cols = mk(E_cap);
    b.sel = mk(E_cap);
    b.edge_ptr = mk(B + 1);
    b.unique = mk(S_cap + E_cap);
    b.unique_ptr = mk(B + 1);
    b.block_row = mk(E_cap);
    b.block_col = mk(E_cap);
    S_cap = S_cap + E_cap;
  }
  (void)nnz;
  auto counts = torch::zeros({3 * L + 1}, opt);  // last entry: device error word
  const size_t ws_bytes = gsb_graphsage_workspace_bytes(B, L, bufs.data(), fanouts.data());
  auto ws = NewWorkspace(ws_bytes, seeds.device());
  const int dtype = csc_->indices.scalar_type() == torch::kInt32 ? GSB_I32 : GSB_I64;
  CheckStatus(gsb_graphsage_sample(P(csc_->indptr), csc_->indices.data_ptr(), dtype, 0, P(seeds),
                                   P(seeds_ptr), B, S0, L, fanouts.data(), GetSeedU64(),
                                   bufs.data(), counts.data_ptr<int64_t>(), ws.data_ptr(),
                                   (size_t)ws.numel(),
                                   (int*)(counts.data_ptr<int64_t>() + 3 * L), CurrentStream()),
              "graphsage_sample");
  auto host = counts.cpu();
  const int64_t* c = host.data_ptr<int64_t>();
  CheckDeviceError((int)c[3 * L], "graphsage_sample");
  std::vector<torch::Tensor> out;
  for (int l = 0; l < L; ++l) {
    const int64_t S = c[3 * l], E = c[3 * l + 1], U = c[3 * l + 2];
    auto& k = keep;
    const size_t o = (size_t)l * 9;
    out.push_back(k[o + 0].narrow(0, 0, S + 1));
    out.push_back(k[o + 1].narrow(0, 0, E));
    out.push_back(k[o + 2].narrow(0, 0, E));
    out.push_back(k[o + 3].narrow(0, 0, E));
    out.push_back(k[o + 4]);
    out.push_back(k[o + 5].narrow(0, 0, U));
    out.push_back(k[o + 6]);
    out.push_back(k[o + 7].narrow(0, 0, E));
    out.push_back(k[o + 8].narrow(0, 0, E));
  }
  out.push_back(host.narrow(0, 0, 3 * L));
  return out;
}

#define GSB_NOT_YET(name) TORCH_CHECK(false, name ": not implemented in this build")

Graph::GraphAndIndex Graph::Compact(int64_t) { GSB_NOT_YET("Compact"); }
torch::Tensor Graph::RandomWalk(torch::Tensor, int64_t) { GSB_NOT_YET("RandomWalk"); }
torch::Tensor Graph::Node2Vec(torch::Tensor, int64_t, double, double) { GSB_NOT_YET("Node2Vec"); }
void Graph::SortCSCIndices() { GSB_NOT_YET("SortCSCIndices"); }
void Graph::SDDMM(const std::string&, torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int64_t,
                  int64_t) { GSB_NOT_YET("SDDMM"); }
void Graph::SpMM(const std::string&, const std::string&, torch::Tensor, torch::Tensor,
                 torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int64_t) { GSB_NOT_YET("SpMM"); }
void Graph::FusedUOPV(const std::string&, torch::Tensor, torch::Tensor, torch::Tensor,
                      torch::Tensor, torch::Tensor, torch::Tensor, int64_t) { GSB_NOT_YET("FusedUOPV"); }
void Graph::FusedESquareSum(const std::string&, const std::string&, torch::Tensor, torch::Tensor,
                            torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int64_t) {
  GSB_NOT_YET("FusedESquareSum");
}
void Graph::FusedEDivUSum(const std::string&, const std::string&, torch::Tensor, torch::Tensor,
                          torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int64_t) {
  GSB_NOT_YET("FusedEDivUSum");
}
Graph::GraphAndIndex Graph::BatchColRowSlcing(torch::Tensor, torch::Tensor, torch::Tensor,
                                              torch::Tensor) { GSB_NOT_YET("BatchColRowSlcing"); }
Graph::GraphAndIndex Graph::BatchRowSlicing(torch::Tensor, torch::Tensor) { GSB_NOT_YET("BatchRowSlicing"); }
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> Graph::SliceAcross(
    const Compressed&, torch::Tensor) { GSB_NOT_YET("row slicing on CSC"); }
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> Graph::SliceCoo(torch::Tensor, int64_t) {
  GSB_NOT_YET("slicing on COO");
}

torch::Tensor ListSampling(int64_t, int64_t, bool) { GSB_NOT_YET("ListSampling"); }
torch::Tensor ListSamplingProbs(torch::Tensor, int64_t, bool) { GSB_NOT_YET("ListSamplingWithProbs"); }
std::tuple<torch::Tensor, torch::Tensor> BatchListSamplingProbs(torch::Tensor, int64_t, bool,
                                                                torch::Tensor) {
  GSB_NOT_YET("BatchListSamplingWithProbs");
}
std::tuple<torch::Tensor, torch::Tensor> BatchListSampling(int64_t, bool, torch::Tensor) {
  GSB_NOT_YET("BatchListSampling");
}
torch::Tensor IndexSearch(torch::Tensor, torch::Tensor) { GSB_NOT_YET("IndexSearch"); }

}  // namespace gsb_host
