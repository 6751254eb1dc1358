// Host layer: the graph object behind torch.classes.gs_classes.Graph.
//
// Mirrors the operator surface of gSampler's gs::Graph (src/graph.h:11-232 in
// the gSampler tree: same method names, argument meaning and result layout) so
// that gs.Matrix / gs.BatchMatrix / gs.jit.compile run unchanged on top of it.
// The implementation is new: every operator validates its inputs, allocates
// its outputs through the torch caching allocator and calls the C ABI of
// include/gsb200.h on the current CUDA stream.  Errors are C++ exceptions
// (TORCH_CHECK), never a process abort, and there is no CPU path.
#pragma once
#include <torch/custom_class.h>
#include <torch/script.h>

#include <memory>
#include <string>
#include <tuple>
#include <vector>

namespace gsb_host {

constexpr int64_t kCOO = 1, kCSC = 2, kCSR = 4;  // format bits (src/graph_storage.h:31-33)

struct Compressed {  // CSC (offsets over columns) or CSR (offsets over rows)
  torch::Tensor indptr, indices;
  c10::optional<torch::Tensor> e_ids;
  torch::Tensor indptr32;   // lazily built 32-bit copy of the offsets (walks)
  torch::Tensor indices32;  // lazily built 32-bit copy of 64-bit indices (walks)
};

struct Coordinate {
  torch::Tensor row, col;
  c10::optional<torch::Tensor> e_ids;
  bool row_sorted = false, col_sorted = false;
};

class Graph : public torch::CustomClassHolder {
 public:
  using GraphPtr = c10::intrusive_ptr<Graph>;
  using GraphAndIndex = std::tuple<GraphPtr, torch::Tensor>;

  Graph(int64_t num_rows, int64_t num_cols) : num_rows_(num_rows), num_cols_(num_cols) {}

  // loaders / getters (src/graph.h:19-78)
  void LoadCSC(torch::Tensor indptr, torch::Tensor indices);
  void LoadCOO(torch::Tensor row, torch::Tensor col, bool row_sorted, bool col_sorted);
  void LoadCSR(torch::Tensor indptr, torch::Tensor indices);
  int64_t GetNumRows() { return num_rows_; }
  int64_t GetNumCols() { return num_cols_; }
  int64_t GetNumEdges() { return num_edges_; }
  torch::Tensor GetCSCIndptr();
  torch::Tensor GetCSCIndices();
  torch::Tensor GetCSCEids();
  torch::Tensor GetCOORows();
  torch::Tensor GetCOOCols();
  torch::Tensor GetCOOEids();
  torch::Tensor GetCSRIndptr();
  torch::Tensor GetCSRIndices();
  torch::Tensor GetCSREids();

  // extract / select operators (src/graph.h:81-125)
  GraphAndIndex Slicing(torch::Tensor seeds, int64_t axis, int64_t on_format, int64_t output_format);
  GraphAndIndex Sampling(int64_t axis, int64_t fanout, bool replace, int64_t on_format,
                         int64_t output_format);
  GraphAndIndex SamplingProbs(int64_t axis, torch::Tensor edge_probs, int64_t fanout, bool replace,
                              int64_t on_format, int64_t output_format);
  GraphAndIndex FusedSlicingSampling(int64_t axis, torch::Tensor seeds, int64_t fanout,
                                     bool replace, int64_t on_format, int64_t output_format);
  GraphAndIndex Compact(int64_t axis);
  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, c10::optional<torch::Tensor>>
  GraphRelabel(torch::Tensor col_seeds, torch::Tensor row_ids);
  torch::Tensor GetValidNodes(torch::Tensor col_seeds, torch::Tensor row_ids);
  torch::Tensor RandomWalk(torch::Tensor seeds, int64_t walk_length);
  torch::Tensor Node2Vec(torch::Tensor seeds, int64_t walk_length, double p, double q);
  void SortCSCIndices();

  // compute operators (feature tensors the chosen op does not read may be None)
  using OptTensor = c10::optional<torch::Tensor>;
  void SDDMM(const std::string& op, OptTensor lhs, OptTensor rhs, torch::Tensor out,
             int64_t lhs_target, int64_t rhs_target, int64_t on_format);
  void SpMM(const std::string& op, const std::string& reduce, OptTensor ufeat, OptTensor efeat,
            torch::Tensor out, OptTensor argu, OptTensor arge, int64_t u_target, int64_t on_format);
  void FusedUOPV(const std::string& op, OptTensor lhs1, OptTensor rhs1, torch::Tensor out1,
                 OptTensor lhs2, OptTensor rhs2, torch::Tensor out2, int64_t on_format);
  void FusedESquareSum(const std::string& op, const std::string& reduce, OptTensor ufeat,
                       OptTensor efeat, torch::Tensor out, OptTensor argu, OptTensor arge,
                       int64_t u_target, int64_t on_format);
  void FusedEDivUSum(const std::string& op, const std::string& reduce, OptTensor ufeat,
                     OptTensor efeat, torch::Tensor out, OptTensor argu, OptTensor arge,
                     int64_t u_target, int64_t on_format);

  // super-batch operators (src/graph.h:126-216)
  void SetEdgeBptr(torch::Tensor t) { edge_bptr_ = t; }
  void SetColBptr(torch::Tensor t) { col_bptr_ = t; }
  void SetRowBptr(torch::Tensor t) { row_bptr_ = t; }
  void SetOrigRowIds(torch::Tensor t) { orig_row_ids_ = t; }
  void SetOrigColIds(torch::Tensor t) { orig_col_ids_ = t; }
  torch::Tensor GetEdgeBptr() { return edge_bptr_; }
  torch::Tensor GetColBptr() { return col_bptr_; }
  torch::Tensor GetRowBptr() { return row_bptr_; }
  std::tuple<torch::Tensor, torch::Tensor> BatchGetRows() { return {orig_row_ids_, row_bptr_}; }
  std::tuple<torch::Tensor, torch::Tensor> BatchGetCols() { return {orig_col_ids_, col_bptr_}; }
  std::tuple<torch::Tensor, torch::Tensor> BatchGetCSCIndptr();
  std::tuple<torch::Tensor, torch::Tensor> BatchGetCSCIndices();
  std::tuple<torch::Tensor, torch::Tensor> BatchGetCSCEids();
  std::tuple<torch::Tensor, torch::Tensor> BatchGetCOORows();
  std::tuple<torch::Tensor, torch::Tensor> BatchGetCOOCols();
  std::tuple<torch::Tensor, torch::Tensor> BatchGetCOOEids();
  std::vector<int64_t> BatchGetColCounts();
  GraphAndIndex BatchColSlicing(torch::Tensor seeds, torch::Tensor col_bptr, bool encoding);
  GraphAndIndex BatchColRowSlcing(torch::Tensor col, torch::Tensor col_bptr, torch::Tensor row,
                                  torch::Tensor row_bptr);
  GraphAndIndex BatchRowSlicing(torch::Tensor row_ids, torch::Tensor row_bptr);
  GraphAndIndex BatchRowSampling(int64_t fanout, bool replace);
  GraphAndIndex BatchRowSamplingProbs(int64_t fanout, bool replace, torch::Tensor edge_probs);
  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor,
             c10::optional<torch::Tensor>, torch::Tensor>
  BatchGraphRelabel(torch::Tensor col_seeds, torch::Tensor row_ids);
  GraphAndIndex BatchFusedSlicingSampling(torch::Tensor seeds, torch::Tensor col_bptr,
                                          int64_t fanout, bool replace);
  std::tuple<torch::Tensor, torch::Tensor> BatchGetValidNodes(torch::Tensor col_seeds,
                                                              torch::Tensor row_ids);

  // Not part of the reference surface: the random stream used by the sampling
  // operators of this graph and of every graph derived from it.  The reference
  // hard-codes one seed (src/cuda/sampling.cu:143); here it is settable and a
  // call counter advances the stream so that repeated calls differ.
  void SetSeed(int64_t seed) {
    seed_ = (uint64_t)seed;
    *stream_counter_ = 0;
  }
  int64_t GetSeed() { return (int64_t)seed_; }
  uint64_t GetSeedU64() const { return seed_; }
  // The call counter that selects the random stream of the next operator.  Together with the seed
  // it is the whole random state of a graph and its descendants: a loop that is checkpointed saves
  // both and restores them to resume with the draws it would have made.
  int64_t GetStreamCounter() { return (int64_t)*stream_counter_; }
  void SetStreamCounter(int64_t counter) { *stream_counter_ = (uint32_t)counter; }
  // Whole L-layer GraphSAGE super-batch sampler in one call (no counterpart in
  // the reference, which composes it from per-layer operators).
  std::vector<torch::Tensor> BatchGraphSAGE(torch::Tensor seeds, torch::Tensor seeds_ptr,
                                            std::vector<int64_t> fanouts);
  // one whole LADIES layer (slice, row weights, collective sampling, renormalisation, block)
  std::vector<torch::Tensor> LadiesLayer(torch::Tensor seeds, int64_t K, torch::Tensor w);
  // enqueue only: tensors at capacity + the device-side counts (see graph_more.cc)
  std::vector<torch::Tensor> BatchGraphSAGEAsync(torch::Tensor seeds, torch::Tensor seeds_ptr,
                                                 std::vector<int64_t> fanouts);

  void CreateSparseFormat(int64_t format);

 private:
  GraphPtr Derive(int64_t rows, int64_t cols) const;
  uint32_t NextStream();
  uint32_t NextStreams(uint32_t n);
  torch::Tensor MapThroughEids(const c10::optional<torch::Tensor>& e_ids, torch::Tensor select);
  // returns (sub_indptr, rows, cols, select) of a sample/slice over `src`
  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> SampleCompressed(
      const Compressed& src, const c10::optional<torch::Tensor>& seeds, int64_t fanout,
      bool replace, const c10::optional<torch::Tensor>& probs, int64_t num_segments);
  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> SliceCompressed(
      const Compressed& src, torch::Tensor seeds, const c10::optional<torch::Tensor>& bptr,
      int64_t encoding_size);
  // row slicing of a CSC operand / column slicing of a CSR operand: keep the
  // entries whose id is in `ids`, relabelled to their position in `ids`
  // (`want_seg`: also the segment of every kept entry, i.e. the COO form)
  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> SliceAcross(
      const Compressed& src, torch::Tensor ids, int64_t nseg, int64_t id_bound, bool want_seg);
  void ReduceImpl(int opcode, const std::string& reduce, OptTensor ufeat, OptTensor efeat,
                  torch::Tensor out, OptTensor argu, OptTensor arge, int64_t u_target,
                  int64_t on_format, const char* who);
  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> SliceCoo(torch::Tensor ids, int64_t axis);
  void AttachSampled(bool is_csc, int64_t output_format, torch::Tensor sub_indptr,
                     torch::Tensor ids, torch::Tensor seg);
  void InheritBatch(const Graph& parent);
  using RelabelResult = std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>;
  RelabelResult RelabelImpl(torch::Tensor col_seeds, torch::Tensor seeds_ptr, torch::Tensor coo_row,
                            torch::Tensor coo_col, torch::Tensor edge_ptr, bool want_edges);
  RelabelResult BatchRelabelImpl(torch::Tensor col_seeds, torch::Tensor row_ids);
  struct RelabelCache {
    torch::Tensor col_seeds, row_ids;  // kept alive so that their addresses stay unique
    RelabelResult value;
  };
  std::shared_ptr<RelabelCache> relabel_cache_;

  int64_t num_rows_ = 0, num_cols_ = 0, num_edges_ = 0;
  std::shared_ptr<Compressed> csc_, csr_;
  std::shared_ptr<Coordinate> coo_;
  torch::Tensor col_bptr_, row_bptr_, edge_bptr_, orig_row_ids_, orig_col_ids_;
  int64_t row_encoding_size_ = 0;
  uint64_t seed_ = 7777;  // the reference's constant
  std::shared_ptr<uint32_t> stream_counter_ = std::make_shared<uint32_t>(0);
};

// helpers shared by graph.cc / ops.cc
void CheckStatus(int status, const char* what);
void CheckDeviceError(int err, const char* what);
torch::Tensor NewWorkspace(size_t bytes, const torch::Device& dev);
// per-device error word of the calls that do not synchronise (read by _CAPI_CheckAsyncErrors)
torch::Tensor& AsyncErrorWord(const torch::Device& dev);
void* CurrentStream();
void CheckIds(const torch::Tensor& t, const char* name);
torch::Device ComputeDevice(const torch::Tensor& t);

}  // namespace gsb_host
