// Operators of gsb_host::Graph beyond slicing / sampling / relabel: the
// whole-sampler entry point, and the compute / walk operators.
#include <c10/cuda/CUDAGuard.h>

#include "graph.h"
#include "gsb200.h"
#include "ops.h"

#include <c10/cuda/CUDAFunctions.h>

#include <atomic>
#include <map>
#include <mutex>

namespace gsb_host {

static const int64_t* P(const torch::Tensor& t) { return t.data_ptr<int64_t>(); }

// 32-bit copy of a CSC's 64-bit row ids, made on first use and kept with the format, for the
// kernels that gather row ids from random places (the sampler's picks, the walks' steps): the
// number of DRAM bursts such gathers cost falls with the bytes a column spans, and the share of the
// array that L2 holds doubles.  Costs half the array's size again in device memory; graphs with
// 2^31 rows or more, or kept in host memory, are read as they are.
struct IdArray { const void* ptr; int dtype; };
static IdArray NarrowIndices(Compressed& c, int64_t num_rows) {
  const int dt = c.indices.scalar_type() == torch::kInt32 ? GSB_I32 : GSB_I64;
  if (dt == GSB_I32 || !c.indices.is_cuda() || num_rows > (int64_t)0x7FFFFFFF)
    return {c.indices.data_ptr(), dt};
  static std::mutex mu;  // two host threads asking for the first time make one copy
  std::lock_guard<std::mutex> lock(mu);
  if (!c.indices32.defined()) {
    try {
      c.indices32 = c.indices.to(torch::kInt32);
    } catch (const c10::Error&) {  // no room for the copy: the 64-bit array serves as it is
      return {c.indices.data_ptr(), dt};
    }
  }
  return {c.indices32.data_ptr(), GSB_I32};
}

// L-layer GraphSAGE super-batch sampler in ONE call: the operator sequence
// A[:, seeds::ptr] -> individual_sampling(K) -> all_nodes -> to_dgl_block per
// layer (examples/graphsage/graphsage_e2e.py:37-44 in gSampler) with every
// intermediate size kept on the device.
//
// BatchGraphSAGEAsync only enqueues the work on the current stream and returns
// 9 tensors per layer (sub_indptr, rows, cols, select, edge_ptr, unique,
// unique_ptr, block_row, block_col) at their CAPACITY, followed by one device
// int64 tensor [3*L + 1] = {S_l, E_l, U_l}..., error word.  The caller reads
// the counts when it needs them (it can keep several super-batches in flight
// on different streams) and narrows the tensors itself.
std::vector<torch::Tensor> Graph::BatchGraphSAGEAsync(torch::Tensor seeds, torch::Tensor seeds_ptr,
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
  // Capacities first, then ONE allocation for the 9 L output arrays, the counts and the
  // workspace: a call costs the caching allocator a single block of a size that repeats from
  // call to call, instead of 28 blocks whose best-fit splitting keeps the pool from settling.
  std::vector<int64_t> sizes;  // int64 words of every output array, in return order
  int64_t S_cap = S0;
  for (int l = 0; l < L; ++l) {
    TORCH_CHECK(fanouts[l] >= 1, "fanout must be positive");
    const int64_t E_cap = S_cap * fanouts[l];
    bufs[(size_t)l].S_cap = S_cap;
    bufs[(size_t)l].E_cap = E_cap;
    for (int64_t n : {S_cap + 1, E_cap, E_cap, E_cap, B + 1, S_cap + E_cap, B + 1, E_cap, E_cap})
      sizes.push_back(n);
    S_cap = S_cap + E_cap;
  }
  sizes.push_back(3 * L + 1);  // counts; last entry: device error word
  auto round32 = [](int64_t words) { return (words + 31) & ~(int64_t)31; };  // 256-byte steps
  int64_t total_words = 0;
  for (int64_t n : sizes) total_words += round32(n);
  const size_t ws_bytes = gsb_graphsage_workspace_bytes(B, L, bufs.data(), fanouts.data());
  auto arena = torch::empty({total_words + (int64_t)((ws_bytes + 7) / 8)}, opt);
  std::vector<torch::Tensor> keep;
  int64_t at = 0;
  for (int64_t n : sizes) { keep.push_back(arena.narrow(0, at, n)); at += round32(n); }
  for (int l = 0; l < L; ++l) {
    gsb_layer_buffers& b = bufs[(size_t)l];
    const size_t o = (size_t)l * 9;
    b.sub_indptr = keep[o + 0].data_ptr<int64_t>();
    b.rows = keep[o + 1].data_ptr<int64_t>();
    b.cols = keep[o + 2].data_ptr<int64_t>();
    b.sel = keep[o + 3].data_ptr<int64_t>();
    b.edge_ptr = keep[o + 4].data_ptr<int64_t>();
    b.unique = keep[o + 5].data_ptr<int64_t>();
    b.unique_ptr = keep[o + 6].data_ptr<int64_t>();
    b.block_row = keep[o + 7].data_ptr<int64_t>();
    b.block_col = keep[o + 8].data_ptr<int64_t>();
  }
  auto counts = keep.back();
  counts.zero_();
  void* ws = arena.data_ptr<int64_t>() + total_words;
  const IdArray ids = NarrowIndices(*csc_, num_rows_);
  CheckStatus(gsb_graphsage_sample(P(csc_->indptr), ids.ptr, ids.dtype, num_cols_,
                                   std::max(num_rows_, num_cols_), P(seeds),
                                   P(seeds_ptr), B, S0, L, fanouts.data(), GetSeedU64(),
                                   NextStreams((uint32_t)L), bufs.data(), counts.data_ptr<int64_t>(), ws, ws_bytes,
                                   (int*)(counts.data_ptr<int64_t>() + 3 * L), CurrentStream()),
              "graphsage_sample");
  // every returned tensor is a view of the one arena (which therefore lives as long as any
  // of them); the workspace sits at its end
  return keep;
}

// The synchronous form: narrows the tensors to their live sizes and returns the
// counts as a CPU int64 tensor [3*L].  Its single synchronisation is the read
// of those counts at the end.
std::vector<torch::Tensor> Graph::BatchGraphSAGE(torch::Tensor seeds, torch::Tensor seeds_ptr,
                                                 std::vector<int64_t> fanouts) {
  auto k = BatchGraphSAGEAsync(seeds, seeds_ptr, fanouts);
  const int L = (int)fanouts.size();
  auto host = k.back().cpu();
  const int64_t* c = host.data_ptr<int64_t>();
  CheckDeviceError((int)c[3 * L], "graphsage_sample");
  std::vector<torch::Tensor> out;
  for (int l = 0; l < L; ++l) {
    const int64_t S = c[3 * l], E = c[3 * l + 1], U = c[3 * l + 2];
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


static int64_t* PM(torch::Tensor& t) { return t.data_ptr<int64_t>(); }
static torch::TensorOptions I64(const torch::Tensor& like) {
  return torch::dtype(torch::kInt64).device(ComputeDevice(like));
}
static int IdxDtype(const torch::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == torch::kInt32 || t.scalar_type() == torch::kInt64,
              "indices must be int32 or int64");
  return t.scalar_type() == torch::kInt32 ? GSB_I32 : GSB_I64;
}

// ------------------------------------------------------------------ slicing across / on COO
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> Graph::SliceAcross(
    const Compressed& src, torch::Tensor ids, int64_t nseg, int64_t id_bound, bool want_seg) {
  c10::cuda::CUDAGuard guard(ComputeDevice(src.indptr));
  CheckIds(ids, "ids");
  auto opt = I64(src.indptr);
  auto sub_indptr = torch::empty({nseg + 1}, opt);
  auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(ids.device()));
  const int64_t nnz_max = src.indices.numel();
  auto ws = NewWorkspace(gsb_slice_across_workspace_bytes(nnz_max, id_bound), ids.device());
  CheckStatus(gsb_slice_across_count(P(src.indptr), src.indices.data_ptr(), IdxDtype(src.indices),
                                     nseg, nnz_max, P(ids), ids.numel(), id_bound, PM(sub_indptr),
                                     ws.data_ptr(), (size_t)ws.numel(), err.data_ptr<int>(),
                                     CurrentStream()),
              "slice_across_count");
  const int64_t E = sub_indptr.narrow(0, nseg, 1).item<int64_t>();
  CheckDeviceError(err.item<int>(), "slice_across_count");
  auto out_ids = torch::empty({E}, opt), seg = torch::empty({want_seg ? E : 0}, opt), sel = torch::empty({E}, opt);
  if (E > 0) {
    CheckStatus(gsb_slice_across_fill(P(src.indptr), src.indices.data_ptr(), IdxDtype(src.indices),
                                      nseg, nnz_max, id_bound, PM(out_ids), want_seg ? PM(seg) : nullptr, PM(sel),
                                      ws.data_ptr(), (size_t)ws.numel(), err.data_ptr<int>(),
                                      CurrentStream()),
                "slice_across_fill");
  }
  return {sub_indptr, out_ids, seg, sel};
}

// src/graph_ops.cc:96-114: axis 0 filters on the rows, 1 on the columns
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> Graph::SliceCoo(torch::Tensor ids,
                                                                        int64_t axis) {
  c10::cuda::CUDAGuard guard(coo_->row.device());
  CheckIds(ids, "ids");
  const auto& key = axis == 0 ? coo_->row : coo_->col;
  const auto& other = axis == 0 ? coo_->col : coo_->row;
  const int64_t nnz = key.numel(), bound = axis == 0 ? num_rows_ : num_cols_;
  auto opt = I64(key);
  auto ok = torch::empty({nnz}, opt), oo = torch::empty({nnz}, opt), sel = torch::empty({nnz}, opt);
  auto scal = torch::zeros({2}, opt);
  auto ws = NewWorkspace(gsb_coo_filter_workspace_bytes(nnz, bound), key.device());
  CheckStatus(gsb_coo_filter(P(key), P(other), nnz, P(ids), ids.numel(), bound, PM(ok), PM(oo),
                             PM(sel), PM(scal), ws.data_ptr(), (size_t)ws.numel(),
                             (int*)(PM(scal) + 1), CurrentStream()),
              "coo_filter");
  auto host = scal.cpu();
  const int64_t E = host.data_ptr<int64_t>()[0];
  CheckDeviceError((int)host.data_ptr<int64_t>()[1], "coo_filter");
  ok = ok.narrow(0, 0, E); oo = oo.narrow(0, 0, E); sel = sel.narrow(0, 0, E);
  if (axis == 0) return {ok, oo, sel};
  return {oo, ok, sel};
}

// src/graph.cc:508-575 (sorted unique of one axis + remap, src/cuda/compact.cu:10-30).
// The ids of an axis lie below the graph's number of rows / columns, so the sorted unique is a
// presence table over that range (gsb_compact_rank / gsb_compact_apply): the rank table is built
// once from one of the formats' id arrays and every format's array is mapped through it.
Graph::GraphAndIndex Graph::Compact(int64_t axis) {
  TORCH_CHECK(axis == 0 || axis == 1, "Compact: axis must be 0 or 1");
  auto ret = Derive(num_rows_, num_cols_);
  const int64_t bound = axis == 0 ? num_rows_ : num_cols_;
  const torch::Tensor* first = nullptr;  // any array holding the axis' ids (they all hold the same set)
  if (coo_) first = axis == 0 ? &coo_->row : &coo_->col;
  else if (axis == 0 && csc_) first = &csc_->indices;
  else if (axis == 1 && csr_) first = &csr_->indices;
  TORCH_CHECK(first != nullptr, axis == 0 ? "Compact(0) needs a COO or CSC format" : "Compact(1) needs a COO or CSR format");
  TORCH_CHECK(first->is_cuda(), "Compact: the graph must be on the GPU");
  c10::cuda::CUDAGuard guard(first->device());
  const auto dev = first->device();
  auto ws = NewWorkspace(gsb_compact_workspace_bytes(bound), dev);
  auto count = torch::empty({1}, torch::dtype(torch::kInt64).device(dev));
  auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(dev));
  auto ids_of = [](const torch::Tensor& t) { return t.contiguous(); };
  {
    auto ids = ids_of(*first);
    CheckStatus(gsb_compact_rank(ids.data_ptr(), IdxDtype(ids), ids.numel(), bound, ws.data_ptr(),
                                 (size_t)ws.numel(), PM(count), err.data_ptr<int>(), CurrentStream()),
                "compact_rank");
  }
  const int64_t U = count.item<int64_t>();  // sizes the frontier list
  CheckDeviceError(err.item<int>(), "Compact");
  auto frontiers = torch::empty({U}, torch::dtype(torch::kInt64).device(dev));
  bool listed = false;
  auto compact = [&](const torch::Tensor& t) {
    auto ids = ids_of(t);
    auto mapped = torch::empty({ids.numel()}, torch::dtype(torch::kInt64).device(dev));
    CheckStatus(gsb_compact_apply(ws.data_ptr(), bound, listed ? nullptr : PM(frontiers), ids.data_ptr(),
                                  IdxDtype(ids), ids.numel(), PM(mapped), CurrentStream()),
                "compact_apply");
    listed = true;
    return mapped;
  };
  if (axis == 0) {
    if (coo_)
      ret->coo_ = std::make_shared<Coordinate>(
          Coordinate{compact(coo_->row), coo_->col, coo_->e_ids, coo_->row_sorted, coo_->col_sorted});
    if (csc_)
      ret->csc_ = std::make_shared<Compressed>(Compressed{csc_->indptr, compact(csc_->indices), csc_->e_ids});
    ret->num_rows_ = U;
  } else {
    if (coo_)
      ret->coo_ = std::make_shared<Coordinate>(
          Coordinate{coo_->row, compact(coo_->col), coo_->e_ids, coo_->row_sorted, coo_->col_sorted});
    if (csr_)
      ret->csr_ = std::make_shared<Compressed>(Compressed{csr_->indptr, compact(csr_->indices), csr_->e_ids});
    ret->num_cols_ = U;
  }
  if (!listed)  // U == 0 and no array: nothing to map
    CheckStatus(gsb_compact_apply(ws.data_ptr(), bound, PM(frontiers), nullptr, GSB_I64, 0, nullptr, CurrentStream()),
                "compact_apply");
  ret->num_edges_ = num_edges_;
  return {ret, frontiers};
}

torch::Tensor& AsyncErrorWord(const torch::Device& dev);  // per-device error word of the calls that do not synchronise

// 32-bit copy of a compressed format's offsets, made on first use and kept with the format, for
// the kernels that gather offsets at random (walks); null when the graph has 2^32 entries or more
// or does not live on the GPU.
static const uint32_t* Offsets32(Compressed& c) {
  if (!c.indptr.is_cuda() || c.indices.numel() >= (int64_t)0xFFFFFFFFll) return nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (!c.indptr32.defined()) c.indptr32 = c.indptr.to(torch::kInt32);  // wraps modulo 2^32: read back as unsigned
  return reinterpret_cast<const uint32_t*>(c.indptr32.data_ptr<int32_t>());
}

// ------------------------------------------------------------------ walks
// src/graph.cc:310-317.  The buffer is step-major [(L+1), N]; like the
// reference it is returned REINTERPRETED as [N, L+1] (a reshape, no transpose).
// The calls do not synchronise: a start node or row id that is not a column, or a rejection loop
// that ran out, ends the walk with -1 and raises a bit in the per-device word that
// _CAPI_CheckAsyncErrors reports.
torch::Tensor Graph::RandomWalk(torch::Tensor seeds, int64_t walk_length) {
  TORCH_CHECK(csc_, "RandomWalk needs the CSC format");
  c10::cuda::CUDAGuard guard(seeds.device());
  CheckIds(seeds, "seeds");
  const int64_t N = seeds.numel();
  auto out = torch::empty({N * (walk_length + 1)}, I64(seeds));
  const IdArray ix = NarrowIndices(*csc_, num_rows_);
  CheckStatus(gsb_random_walk(P(csc_->indptr), Offsets32(*csc_), ix.ptr, ix.dtype, num_cols_, P(seeds), N, walk_length, seed_, NextStream(), PM(out),
                              AsyncErrorWord(seeds.device()).data_ptr<int>(), CurrentStream()),
              "random_walk");
  return out.reshape({N, -1});
}

torch::Tensor Graph::Node2Vec(torch::Tensor seeds, int64_t walk_length, double p, double q) {
  TORCH_CHECK(csc_, "Node2Vec needs the CSC format (with sorted columns)");
  c10::cuda::CUDAGuard guard(seeds.device());
  CheckIds(seeds, "seeds");
  const int64_t N = seeds.numel();
  auto out = torch::empty({N * (walk_length + 1)}, I64(seeds));
  const IdArray ix = NarrowIndices(*csc_, num_rows_);
  CheckStatus(gsb_node2vec(P(csc_->indptr), Offsets32(*csc_), ix.ptr, ix.dtype, num_cols_, P(seeds), N, walk_length, p, q, seed_, NextStream(), PM(out),
                           AsyncErrorWord(seeds.device()).data_ptr<int>(), CurrentStream()),
              "node2vec");
  return out.reshape({N, -1});
}

// src/graph.cc:610-629.  Once-per-graph preprocessing: every column sorted in place by this
// library's per-segment sort (the reference calls CUB's segmented radix sort into a copy).
void Graph::SortCSCIndices() {
  TORCH_CHECK(csc_, "SortCSCIndices needs the CSC format");
  TORCH_CHECK(!csc_->e_ids.has_value(), "SortCSCIndices: the CSC carries edge ids");
  const int64_t nnz = csc_->indices.numel();
  if (nnz == 0) return;
  TORCH_CHECK(csc_->indices.is_cuda() && csc_->indptr.is_cuda(), "SortCSCIndices: the graph must be on the GPU");
  c10::cuda::CUDAGuard guard(csc_->indices.device());
  const int dt = IdxDtype(csc_->indices);
  auto ws = torch::empty({(int64_t)gsb_sort_segments_workspace_bytes(num_cols_, nnz, dt)},
                         torch::dtype(torch::kUInt8).device(csc_->indices.device()));
  auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(csc_->indices.device()));
  // a graph loaded from the caller's tensors shares them: sort a private copy
  csc_->indices = csc_->indices.clone();
  csc_->indices32 = torch::Tensor();
  CheckStatus(gsb_sort_segments(P(csc_->indptr), csc_->indices.data_ptr(), dt, num_cols_, nnz,
                                ws.data_ptr(), (size_t)ws.numel(), err.data_ptr<int>(), CurrentStream()),
              "sort_segments");
  TORCH_CHECK(err.item<int>() == 0, "SortCSCIndices: column offsets are not monotone");
  coo_.reset();
  csr_.reset();
}

// ------------------------------------------------------------------ SpMM / SDDMM
namespace {
enum { OP_ADD = 0, OP_SUB, OP_MUL, OP_DIV, OP_COPY_LHS, OP_COPY_RHS, OP_SQUARE_RHS, OP_RDIV };

int OpCode(const std::string& op) {
  if (op == "add") return OP_ADD;
  if (op == "sub") return OP_SUB;
  if (op == "mul") return OP_MUL;
  if (op == "div") return OP_DIV;
  if (op == "copy_lhs") return OP_COPY_LHS;
  if (op == "copy_rhs") return OP_COPY_RHS;
  TORCH_CHECK(false, "unsupported binary op '", op,
              "' (add, sub, mul, div, copy_lhs, copy_rhs; dot in SDDMM only)");
}
int ReduceCode(const std::string& r) {
  if (r == "sum") return 0;
  if (r == "max") return 1;
  if (r == "min") return 2;
  TORCH_CHECK(false, "unsupported reducer '", r, "' (sum, max, min)");
}
bool UsesLhs(int op) { return op != OP_COPY_RHS && op != OP_SQUARE_RHS; }
bool UsesRhs(int op) { return op != OP_COPY_LHS; }

struct Feature {
  const float* ptr = nullptr;
  int64_t len = 1;
  std::vector<int64_t> shape;  // trailing dims
};

Feature AsFeature(const c10::optional<torch::Tensor>& t, bool used, const char* name) {
  Feature f;
  if (!used) return f;
  TORCH_CHECK(t.has_value() && t.value().defined(), name, " is required by this op");
  const auto& x = t.value();
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kFloat32 && x.is_contiguous(), name,
              " must be a contiguous float32 CUDA tensor");
  f.ptr = x.data_ptr<float>();
  for (int64_t d = 1; d < x.dim(); ++d) { f.shape.push_back(x.size(d)); f.len *= x.size(d); }
  return f;
}

// Broadcast of the trailing feature dims (the role of src/bcast.cc:24-76):
// returns out_len and, when the shapes differ, per-output-element offsets.
struct Bcast {
  int64_t out_len = 1;
  torch::Tensor lhs_off, rhs_off;  // undefined = identity / scalar broadcast
};

Bcast MakeBcast(const Feature& l, bool ul, const Feature& r, bool ur, const torch::Device& dev) {
  Bcast b;
  if (!ul || !ur) { b.out_len = ul ? l.len : r.len; return b; }
  if (l.shape == r.shape || l.len == 1 || r.len == 1) { b.out_len = std::max(l.len, r.len); return b; }
  const size_t nd = std::max(l.shape.size(), r.shape.size());
  std::vector<int64_t> ls(nd, 1), rs(nd, 1), os(nd, 1);
  for (size_t i = 0; i < l.shape.size(); ++i) ls[nd - l.shape.size() + i] = l.shape[i];
  for (size_t i = 0; i < r.shape.size(); ++i) rs[nd - r.shape.size() + i] = r.shape[i];
  for (size_t i = 0; i < nd; ++i) {
    TORCH_CHECK(ls[i] == rs[i] || ls[i] == 1 || rs[i] == 1, "feature shapes do not broadcast");
    os[i] = std::max(ls[i], rs[i]);
    b.out_len *= os[i];
  }
  std::vector<int64_t> lo((size_t)b.out_len), ro((size_t)b.out_len);
  for (int64_t o = 0; o < b.out_len; ++o) {
    int64_t rem = o, lpos = 0, rpos = 0, lstride = 1, rstride = 1;
    for (size_t i = nd; i-- > 0;) {
      const int64_t c = rem % os[i];
      rem /= os[i];
      lpos += (ls[i] == 1 ? 0 : c) * lstride;
      rpos += (rs[i] == 1 ? 0 : c) * rstride;
      lstride *= ls[i];
      rstride *= rs[i];
    }
    lo[(size_t)o] = lpos;
    ro[(size_t)o] = rpos;
  }
  auto opt = torch::dtype(torch::kInt64);
  b.lhs_off = torch::tensor(lo, opt).to(dev);
  b.rhs_off = torch::tensor(ro, opt).to(dev);
  return b;
}

const int64_t* OffPtr(const torch::Tensor& t) { return t.defined() ? t.data_ptr<int64_t>() : nullptr; }
const int64_t* EidPtr(const c10::optional<torch::Tensor>& e) {
  return e.has_value() && e.value().defined() ? e.value().data_ptr<int64_t>() : nullptr;
}
int64_t* ArgPtr(const c10::optional<torch::Tensor>& t) {
  return t.has_value() && t.value().defined() ? t.value().data_ptr<int64_t>() : nullptr;
}
}  // namespace

// src/graph.cc:320-338.  Always evaluated on the COO view: the CSC / CSR
// flavours of the reference only differ in how they find an edge's endpoints.
void Graph::SDDMM(const std::string& op, OptTensor lhs, OptTensor rhs, torch::Tensor out,
                  int64_t lhs_target, int64_t rhs_target, int64_t on_format) {
  if (num_edges_ <= 0) return;
  TORCH_CHECK(on_format == kCOO || on_format == kCSC || on_format == kCSR, "SDDMM: bad format");
  CreateSparseFormat(kCOO);
  c10::cuda::CUDAGuard guard(out.device());
  if (op == "dot") {
    // contraction over the last feature dimension (src/cuda/functor.h:119-138); the leading
    // feature dimensions broadcast as for the other ops
    Feature l = AsFeature(lhs, true, "lhs"), r = AsFeature(rhs, true, "rhs");
    TORCH_CHECK(!l.shape.empty() && !r.shape.empty() && l.shape.back() == r.shape.back(),
                "SDDMM dot: operands need equal last dimensions");
    const int64_t reduce = l.shape.back();
    Feature lp = l, rp = r;
    lp.shape.pop_back(); rp.shape.pop_back();
    lp.len = l.len / reduce; rp.len = r.len / reduce;
    const Bcast bc = MakeBcast(lp, true, rp, true, out.device());
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kFloat32 && out.is_contiguous() &&
                    out.numel() == num_edges_ * bc.out_len,
                "SDDMM dot: out must be contiguous float32 [num_edges, ", bc.out_len, "(, 1)]");
    CheckStatus(gsb_sddmm_coo_dot(P(coo_->row), P(coo_->col), EidPtr(coo_->e_ids), coo_->row.numel(),
                                  l.ptr, l.len, (int)lhs_target, r.ptr, r.len, (int)rhs_target,
                                  OffPtr(bc.lhs_off), OffPtr(bc.rhs_off), reduce,
                                  out.data_ptr<float>(), bc.out_len, CurrentStream()),
                "sddmm_dot");
    return;
  }
  const int code = OpCode(op);
  const Feature l = AsFeature(lhs, UsesLhs(code), "lhs"), r = AsFeature(rhs, UsesRhs(code), "rhs");
  const Bcast bc = MakeBcast(l, UsesLhs(code), r, UsesRhs(code), out.device());
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kFloat32 && out.is_contiguous() &&
                  out.numel() == num_edges_ * bc.out_len,
              "SDDMM: out must be contiguous float32 [num_edges, ", bc.out_len, "]");
  CheckStatus(gsb_sddmm_coo(P(coo_->row), P(coo_->col), EidPtr(coo_->e_ids), coo_->row.numel(), code,
                            l.ptr, l.len, (int)lhs_target, r.ptr, r.len, (int)rhs_target,
                            OffPtr(bc.lhs_off), OffPtr(bc.rhs_off), out.data_ptr<float>(), bc.out_len,
                            CurrentStream()),
              "sddmm");
}

void Graph::ReduceImpl(int code, const std::string& reduce, OptTensor ufeat, OptTensor efeat,
                       torch::Tensor out, OptTensor argu, OptTensor arge, int64_t u_target,
                       int64_t on_format, const char* who) {
  if (num_edges_ <= 0) return;
  TORCH_CHECK(u_target == 0 || u_target == 2, who, ": u_target must be 0 or 2");
  c10::cuda::CUDAGuard guard(out.device());
  const int red = ReduceCode(reduce);
  const Feature u = AsFeature(ufeat, UsesLhs(code), "ufeat"), e = AsFeature(efeat, UsesRhs(code), "efeat");
  const Bcast bc = MakeBcast(u, UsesLhs(code), e, UsesRhs(code), out.device());
  const int64_t nout = u_target == 0 ? num_cols_ : num_rows_;
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kFloat32 && out.is_contiguous() &&
                  out.numel() == nout * bc.out_len,
              who, ": out must be contiguous float32 [", nout, ", ", bc.out_len, "]");
  // The compressed format that reduces along the wanted axis.  If it is not
  // there and building it would need a sort, a sum is accumulated with atomics
  // on the COO view instead (same result up to fp32 summation order).
  const int64_t want = u_target == 0 ? kCSC : kCSR;
  TORCH_CHECK(on_format == kCOO || on_format == want, who,
              ": format and u_target mismatch (CSC with u_target 0, CSR with 2)");
  TORCH_CHECK(coo_ || csc_ || csr_, who, ": graph holds no format");
  const bool have = want == kCSC ? (bool)csc_ : (bool)csr_;
  const bool sorted_coo = coo_ && (want == kCSC ? coo_->col_sorted : coo_->row_sorted);
  const bool segmented = have || sorted_coo || red != 0;
  if (!segmented) CreateSparseFormat(kCOO);
  if (segmented) {
    CreateSparseFormat(want);
    const auto& c = want == kCSC ? *csc_ : *csr_;
    CheckStatus(gsb_spmm_segmented(P(c.indptr), c.indices.data_ptr(), IdxDtype(c.indices),
                                   EidPtr(c.e_ids), nout, code, red, u.ptr, u.len, e.ptr, e.len,
                                   OffPtr(bc.lhs_off), OffPtr(bc.rhs_off), out.data_ptr<float>(),
                                   bc.out_len, ArgPtr(argu), ArgPtr(arge), CurrentStream()),
                who);
  } else {
    CheckStatus(gsb_spmm_coo_sum(P(coo_->row), P(coo_->col), EidPtr(coo_->e_ids), coo_->row.numel(),
                                 code, (int)u_target, u.ptr, u.len, e.ptr, e.len, OffPtr(bc.lhs_off),
                                 OffPtr(bc.rhs_off), out.data_ptr<float>(), bc.out_len,
                                 CurrentStream()),
                who);
  }
}

// src/graph.cc:359-379
void Graph::SpMM(const std::string& op, const std::string& reduce, OptTensor ufeat, OptTensor efeat,
                 torch::Tensor out, OptTensor argu, OptTensor arge, int64_t u_target,
                 int64_t on_format) {
  ReduceImpl(OpCode(op), reduce, ufeat, efeat, out, argu, arge, u_target, on_format, "SpMM");
}

// src/graph.cc:457-479: out[n] = sum of e^2 over the edges of n
void Graph::FusedESquareSum(const std::string&, const std::string& reduce, OptTensor ufeat,
                            OptTensor efeat, torch::Tensor out, OptTensor argu, OptTensor arge,
                            int64_t u_target, int64_t on_format) {
  ReduceImpl(OP_SQUARE_RHS, reduce, ufeat, efeat, out, argu, arge, u_target, on_format,
             "FusedESquareSum");
}

// src/graph.cc:482-503: out[n] = sum of e / u[other endpoint] over the edges of n
void Graph::FusedEDivUSum(const std::string&, const std::string& reduce, OptTensor ufeat,
                          OptTensor efeat, torch::Tensor out, OptTensor argu, OptTensor arge,
                          int64_t u_target, int64_t on_format) {
  ReduceImpl(OP_RDIV, reduce, ufeat, efeat, out, argu, arge, u_target, on_format, "FusedEDivUSum");
}

// src/graph.cc:341-356: two u-op-v edge maps over the same graph, one pass over the edges
void Graph::FusedUOPV(const std::string& op, OptTensor lhs1, OptTensor rhs1, torch::Tensor out1,
                      OptTensor lhs2, OptTensor rhs2, torch::Tensor out2, int64_t on_format) {
  if (num_edges_ <= 0) return;
  TORCH_CHECK(on_format == kCOO || on_format == kCSC, "FusedUOPV: CSC or COO format only");
  CreateSparseFormat(kCOO);   // the CSC flavour of the reference only differs in how it finds the endpoints
  c10::cuda::CUDAGuard guard(out1.device());
  const int code = OpCode(op);
  const Feature l1 = AsFeature(lhs1, UsesLhs(code), "lhs1"), r1 = AsFeature(rhs1, UsesRhs(code), "rhs1");
  const Feature l2 = AsFeature(lhs2, UsesLhs(code), "lhs2"), r2 = AsFeature(rhs2, UsesRhs(code), "rhs2");
  TORCH_CHECK(l1.shape == l2.shape && r1.shape == r2.shape, "FusedUOPV: both operand pairs need equal shapes");
  const Bcast bc = MakeBcast(l1, UsesLhs(code), r1, UsesRhs(code), out1.device());
  for (const torch::Tensor* o : {&out1, &out2})
    TORCH_CHECK(o->is_cuda() && o->scalar_type() == torch::kFloat32 && o->is_contiguous() &&
                    o->numel() == num_edges_ * bc.out_len,
                "FusedUOPV: outputs must be contiguous float32 [num_edges, ", bc.out_len, "]");
  CheckStatus(gsb_u_op_v_pair(P(coo_->row), P(coo_->col), EidPtr(coo_->e_ids), coo_->row.numel(), code,
                              l1.ptr, r1.ptr, out1.data_ptr<float>(), l2.ptr, r2.ptr,
                              out2.data_ptr<float>(), l1.len, r1.len, OffPtr(bc.lhs_off),
                              OffPtr(bc.rhs_off), bc.out_len, CurrentStream()),
              "u_op_v_pair");
}

// {0, n} on the device (a one-segment offset array)
static torch::Tensor OneSegment(int64_t n, const torch::Device& dev) {
  auto t = torch::empty({2}, torch::dtype(torch::kInt64).pinned_memory(true));
  t.data_ptr<int64_t>()[0] = 0;
  t.data_ptr<int64_t>()[1] = n;
  return t.to(dev, /*non_blocking=*/true);
}

// ------------------------------------------------------------------ whole LADIES layer
// One layer of the layer-wise (LADIES) sampler of gSampler's examples/ladies/ladies.py:7-21 in a
// single call:
//   subA = A[:, seeds];  p[r] = sum over the slice of w^2 per row r;  K rows by weight p
//   (collective sampling without replacement);  keep their edges;  w <- w / p[row];
//   w <- w / (column sum of w);  node list = first-occurrence unique of [seeds, rows];  block.
// The operator sequence is the one the Matrix API composes from Slicing / SpMM / ListSampling /
// row Slicing / SDDMM / GetValidNodes / GraphRelabel; doing it here leaves two host read-backs
// (the slice size and the kept-edge count, both needed to size outputs) instead of one per
// operator, and no Python between the launches.  Returns {node list, block rows, block cols,
// edge weights, selected row ids, edge positions in this graph, p of the selected rows}.
std::vector<torch::Tensor> Graph::LadiesLayer(torch::Tensor seeds, int64_t K, torch::Tensor w) {
  CreateSparseFormat(kCSC);
  TORCH_CHECK(!csc_->e_ids.has_value(), "LadiesLayer expects a CSC without edge-id indirection");
  CheckIds(seeds, "seeds");
  TORCH_CHECK(K >= 1, "K must be positive");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kFloat32 && w.is_contiguous() &&
                  w.numel() == csc_->indices.numel(),
              "LadiesLayer: weights must be a contiguous float32 CUDA tensor with one entry per edge");
  c10::cuda::CUDAGuard guard(seeds.device());
  const auto dev = seeds.device();
  auto i64 = torch::dtype(torch::kInt64).device(dev);
  auto f32 = torch::dtype(torch::kFloat32).device(dev);
  const int64_t S = seeds.numel(), R = num_rows_;
  auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(dev));
  int* d_err = err.data_ptr<int>();
  void* st = CurrentStream();
  const int idt = IdxDtype(csc_->indices);

  // 1. column slice (the one size that must come back before anything can be allocated)
  auto sub_indptr = torch::empty({S + 1}, i64);
  {
    auto ws = NewWorkspace(gsb_slice_cols_workspace_bytes(S), dev);
    CheckStatus(gsb_slice_cols_count(P(csc_->indptr), num_cols_, P(seeds), S, PM(sub_indptr), ws.data_ptr(),
                                     (size_t)ws.numel(), d_err, st),
                "slice_cols_count");
  }
  const int64_t Es = sub_indptr.narrow(0, S, 1).item<int64_t>();
  auto rows = torch::empty({Es}, i64), cols = torch::empty({Es}, i64), sel = torch::empty({Es}, i64);
  CheckStatus(gsb_slice_cols_fill(P(csc_->indptr), csc_->indices.data_ptr(), idt, P(seeds), S,
                                  P(sub_indptr), Es, PM(rows), PM(cols), PM(sel), nullptr, 0, 0, st),
              "slice_cols_fill");
  auto ws_e = torch::empty({Es}, f32);
  CheckStatus(gsb_gather_rows(w.data_ptr(), 4, w.numel(), P(sel), Es, ws_e.data_ptr(), d_err, st), "gather");

  // 2. p[r] = sum of w^2 over the slice's entries in row r
  auto prob = torch::zeros({R}, f32);
  if (Es > 0)
    CheckStatus(gsb_spmm_coo_sum(P(rows), P(cols), nullptr, Es, OP_SQUARE_RHS, /*u_target=*/2, nullptr, 1,
                                 ws_e.data_ptr<float>(), 1, nullptr, nullptr, prob.data_ptr<float>(), 1, st),
                "row sums");

  // 3. K of the R rows by weight p, without replacement
  const int64_t Ksel = std::min(K, R);
  auto range = OneSegment(R, dev);
  auto picked = torch::empty({Ksel}, i64), picked_ptr = torch::empty({2}, i64);
  {
    auto ws = NewWorkspace(gsb_list_sample_workspace_bytes(R, 1), dev);
    CheckStatus(gsb_list_sample(prob.data_ptr<float>(), P(range), 1, R, K, ListSamplingSeed(),
                                NextListStream(), PM(picked), PM(picked_ptr), ws.data_ptr(),
                                (size_t)ws.numel(), d_err, st),
                "list_sample");
  }

  // 4. keep the slice's entries whose row was picked (ordered compaction over the slice's
  //    edges, which stay in column order); row id -> position among the picked
  auto new_row = torch::empty({Es}, i64), seg = torch::empty({Es}, i64), sel2 = torch::empty({Es}, i64);
  auto kept = torch::zeros({1}, i64);
  {
    auto ws = NewWorkspace(gsb_coo_filter_workspace_bytes(Es, R), dev);
    CheckStatus(gsb_coo_filter(P(rows), P(cols), Es, P(picked), Ksel, R, PM(new_row), PM(seg), PM(sel2),
                               PM(kept), ws.data_ptr(), (size_t)ws.numel(), d_err, st),
                "coo_filter");
  }
  const int64_t E2 = kept.item<int64_t>();
  CheckDeviceError(err.item<int>(), "LadiesLayer");
  new_row = new_row.narrow(0, 0, E2); seg = seg.narrow(0, 0, E2); sel2 = sel2.narrow(0, 0, E2);

  // 5. w / p[row], then / column sum (division as multiplication by the reciprocal, like the
  //    Matrix API's div: python/gs/ops/sddmm.py:23-25)
  auto w2 = torch::empty({E2}, f32), p_sel = torch::empty({Ksel}, f32);
  CheckStatus(gsb_gather_rows(ws_e.data_ptr(), 4, Es, P(sel2), E2, w2.data_ptr(), d_err, st), "gather");
  CheckStatus(gsb_gather_rows(prob.data_ptr(), 4, R, P(picked), Ksel, p_sel.data_ptr(), d_err, st), "gather");
  auto inv_p = p_sel.reciprocal();
  auto w3 = torch::empty({E2}, f32), w4 = torch::empty({E2}, f32);
  auto colsum = torch::zeros({S}, f32);
  if (E2 > 0) {
    CheckStatus(gsb_sddmm_coo(P(new_row), P(seg), nullptr, E2, OP_MUL, w2.data_ptr<float>(), 1, 1,
                              inv_p.data_ptr<float>(), 1, 0, nullptr, nullptr, w3.data_ptr<float>(), 1, st),
                "sddmm");
    CheckStatus(gsb_spmm_coo_sum(P(new_row), P(seg), nullptr, E2, OP_COPY_RHS, /*u_target=*/0, nullptr, 1,
                                 w3.data_ptr<float>(), 1, nullptr, nullptr, colsum.data_ptr<float>(), 1, st),
                "column sums");
    auto inv_c = colsum.reciprocal();
    CheckStatus(gsb_sddmm_coo(P(new_row), P(seg), nullptr, E2, OP_MUL, w3.data_ptr<float>(), 1, 1,
                              inv_c.data_ptr<float>(), 1, 2, nullptr, nullptr, w4.data_ptr<float>(), 1, st),
                "sddmm");
  }

  // 6. node list and block: first-occurrence unique of [seeds, picked[new_row]]
  auto rows_global = torch::empty({E2}, i64), edge_pos = torch::empty({E2}, i64);
  CheckStatus(gsb_gather_rows(picked.data_ptr(), 8, Ksel, P(new_row), E2, rows_global.data_ptr(), d_err, st),
              "gather");
  CheckStatus(gsb_gather_rows(sel.data_ptr(), 8, Es, P(sel2), E2, edge_pos.data_ptr(), d_err, st), "gather");
  auto r = RelabelImpl(seeds, OneSegment(S, dev), rows_global, seg, OneSegment(E2, dev), true);
  CheckDeviceError(err.item<int>(), "LadiesLayer");
  return {std::get<0>(r), std::get<2>(r), std::get<3>(r), w4, picked, edge_pos, p_sel};
}

// ------------------------------------------------------------------ batch row slicing
// src/batch_graph.cc:144-157
Graph::GraphAndIndex Graph::BatchRowSlicing(torch::Tensor row_ids, torch::Tensor row_bptr) {
  auto r = Slicing(row_ids, 0, kCSC, kCSC + kCOO);
  auto g = std::get<0>(r);
  g->col_bptr_ = col_bptr_;
  g->row_bptr_ = row_bptr;
  g->orig_col_ids_ = orig_col_ids_;
  g->orig_row_ids_ = row_ids;
  g->row_encoding_size_ = row_encoding_size_;
  auto eb = torch::empty({col_bptr_.numel()}, I64(col_bptr_));
  CheckStatus(gsb_gather_i64(P(g->csc_->indptr), P(col_bptr_), col_bptr_.numel(), PM(eb),
                             CurrentStream()),
              "gather");
  g->edge_bptr_ = eb;
  return r;
}

// src/batch_graph.cc:107-141.  The returned index holds positions in THIS graph's
// edge order (mapped through e_ids when present), which is what the callers
// index the parent's edge data with (python/gs/matrix_api/batch_matrix.py:72-80).
Graph::GraphAndIndex Graph::BatchColRowSlcing(torch::Tensor col, torch::Tensor col_bptr,
                                              torch::Tensor row, torch::Tensor row_bptr) {
  CreateSparseFormat(kCSC);
  CheckIds(col, "col"); CheckIds(col_bptr, "col_bptr"); CheckIds(row, "row"); CheckIds(row_bptr, "row_bptr");
  TORCH_CHECK(col_bptr.numel() == row_bptr.numel() && col_bptr.numel() >= 2,
              "BatchColRowSlcing: col_bptr and row_bptr must have the same length >= 2");
  c10::cuda::CUDAGuard guard(ComputeDevice(csc_->indptr));
  const int64_t S = col.numel(), R = row.numel(), B = col_bptr.numel() - 1;
  auto opt = I64(csc_->indptr);
  auto sub_indptr = torch::empty({S + 1}, opt);
  auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(col.device()));
  auto ws = NewWorkspace(gsb_slice_cols_rows_workspace_bytes(S, R, B), col.device());
  CheckStatus(gsb_slice_cols_rows_count(P(csc_->indptr), csc_->indices.data_ptr(),
                                        IdxDtype(csc_->indices), num_cols_, P(col), P(col_bptr), S,
                                        P(row), P(row_bptr), R, B, PM(sub_indptr), ws.data_ptr(),
                                        (size_t)ws.numel(), err.data_ptr<int>(), CurrentStream()),
              "slice_cols_rows_count");
  const int64_t E = sub_indptr.narrow(0, S, 1).item<int64_t>();
  CheckDeviceError(err.item<int>(), "slice_cols_rows_count");
  auto ids = torch::empty({E}, opt), seg = torch::empty({E}, opt), sel = torch::empty({E}, opt);
  if (E > 0)
    CheckStatus(gsb_slice_cols_rows_fill(P(csc_->indptr), csc_->indices.data_ptr(),
                                         IdxDtype(csc_->indices), num_cols_, P(col), P(col_bptr), S,
                                         P(row_bptr), R, B, P(sub_indptr), PM(ids), PM(seg), PM(sel),
                                         ws.data_ptr(), CurrentStream()),
                "slice_cols_rows_fill");
  auto g = Derive(R, S);
  g->csc_ = std::make_shared<Compressed>(Compressed{sub_indptr, ids, c10::nullopt});
  g->coo_ = std::make_shared<Coordinate>(Coordinate{ids, seg, c10::nullopt, false, true});
  g->num_edges_ = E;
  g->col_bptr_ = col_bptr;
  g->row_bptr_ = row_bptr;
  g->orig_col_ids_ = col;
  g->orig_row_ids_ = row;
  auto eb = torch::empty({B + 1}, I64(col_bptr));
  CheckStatus(gsb_gather_i64(P(sub_indptr), P(col_bptr), B + 1, PM(eb), CurrentStream()), "gather");
  g->edge_bptr_ = eb;
  return {g, MapThroughEids(csc_->e_ids, sel)};
}

// ------------------------------------------------------------------ gs_ops

// `single_list`: the caller built `range` = [0, R] itself, so the number of picks is known on the
// host (min(K, R)) and nothing is read back; device-side errors go to the per-device word that
// CheckAsyncErrors reports.
static std::tuple<torch::Tensor, torch::Tensor> ListSampleImpl(const c10::optional<torch::Tensor>& probs,
                                                               torch::Tensor range, int64_t R,
                                                               int64_t K, const torch::Device& dev,
                                                               bool single_list = false) {
  c10::cuda::CUDAGuard guard(dev);
  const int64_t B = range.numel() - 1;
  auto opt = torch::dtype(torch::kInt64).device(dev);
  auto out_range = torch::empty({B + 1}, opt);
  auto out_idx = torch::empty({std::min(B * K, R)}, opt);
  auto err = single_list ? AsyncErrorWord(dev)
                         : torch::zeros({1}, torch::dtype(torch::kInt32).device(dev));
  // the uniform reservoir pass needs no scratch
  auto ws = NewWorkspace(probs.has_value() ? gsb_list_sample_workspace_bytes(R, B) : 256, dev);
  const float* pp = nullptr;
  if (probs.has_value()) {
    const auto& pr = probs.value();
    TORCH_CHECK(pr.is_cuda() && pr.scalar_type() == torch::kFloat32 && pr.is_contiguous(),
                "probs must be a contiguous float32 CUDA tensor");
    pp = pr.data_ptr<float>();
  }
  CheckStatus(gsb_list_sample(pp, P(range), B, R, K, ListSamplingSeed(), NextListStream(),
                              PM(out_idx), PM(out_range), ws.data_ptr(), (size_t)ws.numel(),
                              err.data_ptr<int>(), CurrentStream()),
              "list_sample");
  if (single_list) return {out_idx, out_range};
  const int64_t total = out_range.narrow(0, B, 1).item<int64_t>();
  CheckDeviceError(err.item<int>(), "list_sample");
  return {out_idx.narrow(0, 0, total), out_range};
}

static torch::Tensor Range2(int64_t n, const torch::Device& dev) {
  auto t = torch::empty({2}, torch::dtype(torch::kInt64).pinned_memory(true));
  t.data_ptr<int64_t>()[0] = 0;
  t.data_ptr<int64_t>()[1] = n;
  return t.to(dev, /*non_blocking=*/true);
}

static torch::Tensor ListReplaceImpl(const c10::optional<torch::Tensor>& probs, int64_t n, int64_t K,
                                     const torch::Device& dev) {
  c10::cuda::CUDAGuard guard(dev);
  TORCH_CHECK(n >= 1, "cannot draw from an empty list");
  auto out = torch::empty({K}, torch::dtype(torch::kInt64).device(dev));
  auto ws = NewWorkspace(gsb_list_sample_workspace_bytes(n, 1), dev);
  CheckStatus(gsb_list_sample_replace(probs.has_value() ? probs.value().data_ptr<float>() : nullptr, n,
                                      K, ListSamplingSeed(), NextListStream(), PM(out), ws.data_ptr(),
                                      (size_t)ws.numel(), CurrentStream()),
              "list_sample_replace");
  return out;
}

static torch::Device CurrentCudaDevice() { return torch::Device(torch::kCUDA, c10::cuda::current_device()); }

// src/tensor_ops.cc:6-8
torch::Tensor ListSampling(int64_t num_items, int64_t num_picks, bool replace) {
  const auto dev = CurrentCudaDevice();
  if (replace) return ListReplaceImpl(c10::nullopt, num_items, num_picks, dev);
  // one list whose length the host knows: no offsets go to the device, none come back
  TORCH_CHECK(num_items >= 0 && num_picks >= 0, "ListSampling: negative size");
  c10::cuda::CUDAGuard guard(dev);
  auto out = torch::empty({std::min(num_picks, num_items)}, torch::dtype(torch::kInt64).device(dev));
  CheckStatus(gsb_list_sample(nullptr, nullptr, 1, num_items, num_picks, ListSamplingSeed(), NextListStream(),
                              PM(out), nullptr, nullptr, 0, AsyncErrorWord(dev).data_ptr<int>(),
                              CurrentStream()),
              "list_sample");
  return out;
}

// src/tensor_ops.cc:10-13
torch::Tensor ListSamplingProbs(torch::Tensor probs, int64_t num_picks, bool replace) {
  TORCH_CHECK(probs.is_cuda() && probs.scalar_type() == torch::kFloat32, "probs must be float32 CUDA");
  probs = probs.contiguous();
  if (replace) return ListReplaceImpl(probs, probs.numel(), num_picks, probs.device());
  return std::get<0>(ListSampleImpl(probs, Range2(probs.numel(), probs.device()), probs.numel(),
                                    num_picks, probs.device(), /*single_list=*/true));
}

// src/tensor_ops.cc:15-19
std::tuple<torch::Tensor, torch::Tensor> BatchListSamplingProbs(torch::Tensor probs,
                                                                int64_t num_picks, bool replace,
                                                                torch::Tensor range) {
  TORCH_CHECK(!replace, "BatchListSamplingWithProbs: replace=True is not implemented "
                        "(nor is it in the reference, batch/list_sampling_probs.cu:38-39)");
  TORCH_CHECK(probs.is_cuda() && probs.scalar_type() == torch::kFloat32, "probs must be float32 CUDA");
  CheckIds(range, "range");
  return ListSampleImpl(probs.contiguous(), range, probs.numel(), num_picks, probs.device());
}

// src/tensor_ops.cc:21-28: uniform choice inside every segment
std::tuple<torch::Tensor, torch::Tensor> BatchListSampling(int64_t num_picks, bool replace,
                                                           torch::Tensor range) {
  TORCH_CHECK(!replace, "BatchListSampling: replace=True is not implemented");
  CheckIds(range, "range");
  const int64_t R = range.narrow(0, range.numel() - 1, 1).item<int64_t>();
  return ListSampleImpl(c10::nullopt, range, R, num_picks, range.device());
}

// src/tensor_ops.cc:30-38: position of every key in `origin_data`, -1 if absent (the smallest
// position when `origin_data` holds a value more than once).  Does not synchronise: a -1 inside
// `origin_data` (the table's empty key, as in the reference) is reported by CheckAsyncErrors.
torch::Tensor IndexSearch(torch::Tensor origin_data, torch::Tensor keys) {
  TORCH_CHECK(origin_data.is_cuda() && keys.is_cuda(), "IndexSearch: tensors must be on the GPU");
  TORCH_CHECK(origin_data.scalar_type() == torch::kInt64 && keys.scalar_type() == torch::kInt64,
              "IndexSearch: int64 tensors");
  c10::cuda::CUDAGuard guard(keys.device());
  auto data = origin_data.contiguous().reshape({-1});
  auto flat = keys.contiguous().reshape({-1});
  auto out = torch::empty_like(flat);
  auto ws = NewWorkspace(gsb_index_search_workspace_bytes(data.numel()), keys.device());
  CheckStatus(gsb_index_search(P(data), data.numel(), P(flat), flat.numel(), PM(out), ws.data_ptr(),
                               (size_t)ws.numel(), AsyncErrorWord(keys.device()).data_ptr<int>(), CurrentStream()),
              "index_search");
  return out.reshape(keys.sizes());
}

// ------------------------------------------------------------------ row gather
// One error word per device that the sync-free operators raise bits in; it is
// read (and cleared) by CheckAsyncErrors, the way CUDA reports kernel faults
// at the next synchronising call rather than at the launch.
torch::Tensor& AsyncErrorWord(const torch::Device& dev) {
  static std::mutex mu;
  // never destroyed: a static destructor would free device memory after the CUDA context is gone
  static auto* words = new std::map<int, torch::Tensor>();
  std::lock_guard<std::mutex> lock(mu);
  auto it = words->find(dev.index());
  if (it == words->end())
    it = words->emplace(dev.index(), torch::zeros({1}, torch::dtype(torch::kInt32).device(dev))).first;
  return it->second;
}

void CheckAsyncErrors() {
  const auto dev = CurrentCudaDevice();
  auto& w = AsyncErrorWord(dev);
  const int bits = w.item<int>();
  if (bits) w.zero_();
  CheckDeviceError(bits, "an earlier sync-free operator (row gather, single-list sampling, walks)");
}

// out[i, ...] = data[index[i], ...].  `data` lives on the GPU or in page-locked
// host memory (read in place, python/gs/matrix_api/matrix.py:19-23 and
// src/cuda/index_select_uvm.cu:22-41 in gSampler); no synchronisation.
torch::Tensor GatherRows(torch::Tensor data, torch::Tensor index) {
  CheckIds(index, "index");
  TORCH_CHECK(data.defined() && data.dim() >= 1 && data.is_contiguous(),
              "GatherRows: data must be a contiguous tensor with at least one dimension");
  TORCH_CHECK(data.is_cuda() ? data.device() == index.device() : data.is_pinned(),
              "GatherRows: data must be on the index's GPU or in pinned host memory");
  TORCH_CHECK(index.dim() == 1, "GatherRows: index must be one-dimensional");
  c10::cuda::CUDAGuard guard(index.device());
  auto sizes = data.sizes().vec();
  const int64_t src_rows = sizes[0];
  sizes[0] = index.numel();
  auto out = torch::empty(sizes, data.options().device(index.device()).pinned_memory(false));
  const int64_t row_bytes = src_rows == 0 ? 0 : data.nbytes() / src_rows;
  TORCH_CHECK(src_rows > 0 || index.numel() == 0, "GatherRows: data has no rows");
  CheckStatus(gsb_gather_rows(data.data_ptr(), row_bytes, src_rows, index.data_ptr<int64_t>(),
                              index.numel(), out.data_ptr(), AsyncErrorWord(index.device()).data_ptr<int>(),
                              CurrentStream()),
              "gather_rows");
  return out;
}

static std::atomic<uint64_t> g_list_seed{7777};
static std::atomic<uint32_t> g_list_calls{0};
uint64_t ListSamplingSeed() { return g_list_seed.load(); }
uint32_t NextListStream() { return g_list_calls.fetch_add(1); }
void SetListSamplingSeed(int64_t seed) {
  g_list_seed.store((uint64_t)seed);
  g_list_calls.store(0);
}

}  // namespace gsb_host
