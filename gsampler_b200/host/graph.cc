#include "graph.h"
#include "ops.h"

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "gsb200.h"

namespace gsb_host {

// ------------------------------------------------------------------ helpers
void CheckStatus(int status, const char* what) {
  if (status == GSB_OK) return;
  TORCH_CHECK(false, "gsb200: ", what, " failed: ", gsb_status_string(status),
              status == GSB_ERR_CUDA ? std::string(" (") + gsb_last_cuda_error() + ")" : std::string());
}

void CheckDeviceError(int err, const char* what) {
  if (err == 0) return;
  std::string msg;
  if (err & GSB_ERRBIT_LOOKBACK_TIMEOUT) msg += " tile-prefix wait timed out;";
  if (err & GSB_ERRBIT_TABLE_FULL) msg += " hash table full;";
  if (err & GSB_ERRBIT_KEY_MISSING) msg += " id missing from the node list;";
  if (err & GSB_ERRBIT_CAPACITY) msg += " output capacity exceeded;";
  if (err & GSB_ERRBIT_BAD_INPUT) msg += " id out of range or non-monotone offsets;";
  TORCH_CHECK(false, "gsb200: ", what, " reported a device-side error:", msg);
}

torch::Tensor NewWorkspace(size_t bytes, const torch::Device& dev) {
  return torch::empty({(int64_t)(bytes + 256)}, torch::dtype(torch::kUInt8).device(dev));
}

void* CurrentStream() { return (void*)c10::cuda::getCurrentCUDAStream().stream(); }

void CheckIds(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.defined(), name, " is undefined");
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(t.scalar_type() == torch::kInt64, name, " must be int64");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// The device a graph tensor is processed on: its own GPU, or -- for a graph kept
// in page-locked host memory, which the kernels read in place (src/graph_ops.cc:67,
// 159,192 and src/cuda/slicing.cu:128-130 in gSampler) -- the current GPU.
torch::Device ComputeDevice(const torch::Tensor& t) {
  if (t.is_cuda()) return t.device();
  TORCH_CHECK(t.is_pinned(), "graph tensors must live on a GPU or in pinned host memory");
  return torch::Device(torch::kCUDA, c10::cuda::current_device());
}

static void CheckGraphIndptr(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.defined(), name, " is undefined");
  TORCH_CHECK(t.is_cuda() || t.is_pinned(), name,
              " must be a CUDA tensor or a pinned host tensor (this library has no CPU path)");
  TORCH_CHECK(t.scalar_type() == torch::kInt64, name, " must be int64");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// Checked once at load time (one synchronisation): the offsets start at 0, never decrease, end at
// the number of entries and have one entry per segment plus one -- what every kernel relies on.
static void CheckOffsets(const torch::Tensor& indptr, int64_t nseg, int64_t nnz, const char* what) {
  TORCH_CHECK(indptr.numel() == nseg + 1, what, ": indptr has ", indptr.numel(), " entries, the graph has ",
              nseg, " segments (expected ", nseg + 1, ")");
  const bool ok = nseg == 0 ? indptr[0].item<int64_t>() == nnz
                            : (indptr[0].item<int64_t>() == 0 && indptr[nseg].item<int64_t>() == nnz &&
                               (indptr.narrow(0, 1, nseg) >= indptr.narrow(0, 0, nseg)).all().item<bool>());
  TORCH_CHECK(ok, what, ": indptr must start at 0, be non-decreasing and end at the number of entries (", nnz, ")");
}

static int IndicesDtype(const torch::Tensor& indices) {
  TORCH_CHECK((indices.is_cuda() || indices.is_pinned()) && indices.is_contiguous(),
              "indices must be contiguous, on a GPU or in pinned host memory");
  if (indices.scalar_type() == torch::kInt64) return GSB_I64;
  if (indices.scalar_type() == torch::kInt32) return GSB_I32;
  TORCH_CHECK(false, "indices must be int32 or int64");
}

static torch::TensorOptions I64(const torch::Tensor& like) {
  return torch::dtype(torch::kInt64).device(ComputeDevice(like));
}

static const int64_t* P(const torch::Tensor& t) { return t.data_ptr<int64_t>(); }
static int64_t* PM(torch::Tensor& t) { return t.data_ptr<int64_t>(); }

static torch::Tensor ExpandIndptr(const torch::Tensor& indptr, int64_t nnz) {
  auto out = torch::empty({nnz}, I64(indptr));
  CheckStatus(gsb_expand_indptr(P(indptr), indptr.numel() - 1, nnz, PM(out), CurrentStream()),
              "expand_indptr");
  return out;
}

static torch::Tensor AsI64(const torch::Tensor& t) {
  return t.scalar_type() == torch::kInt64 ? t : t.to(torch::kInt64);
}

// ------------------------------------------------------------------ loaders
void Graph::LoadCSC(torch::Tensor indptr, torch::Tensor indices) {
  CheckGraphIndptr(indptr, "indptr");
  IndicesDtype(indices);
  CheckOffsets(indptr, num_cols_, indices.numel(), "LoadCSC");
  csc_ = std::make_shared<Compressed>(Compressed{indptr, indices, c10::nullopt});
  num_edges_ = indices.numel();
}
void Graph::LoadCSR(torch::Tensor indptr, torch::Tensor indices) {
  CheckGraphIndptr(indptr, "indptr");
  IndicesDtype(indices);
  CheckOffsets(indptr, num_rows_, indices.numel(), "LoadCSR");
  csr_ = std::make_shared<Compressed>(Compressed{indptr, indices, c10::nullopt});
  num_edges_ = indices.numel();
}
void Graph::LoadCOO(torch::Tensor row, torch::Tensor col, bool row_sorted, bool col_sorted) {
  CheckIds(row, "row");
  CheckIds(col, "col");
  coo_ = std::make_shared<Coordinate>(Coordinate{row, col, c10::nullopt, row_sorted, col_sorted});
  num_edges_ = row.numel();
}

Graph::GraphPtr Graph::Derive(int64_t rows, int64_t cols) const {
  auto g = c10::make_intrusive<Graph>(rows, cols);
  g->seed_ = seed_;
  g->stream_counter_ = stream_counter_;
  return g;
}

uint32_t Graph::NextStream() { return (*stream_counter_)++; }
// `n` consecutive streams (one per layer of a whole-sampler call); returns the first
uint32_t Graph::NextStreams(uint32_t n) {
  const uint32_t first = *stream_counter_;
  *stream_counter_ += n;
  return first;
}

// Lazy format conversion (src/graph.cc:22-49, src/graph_ops.cc:14-61).
void Graph::CreateSparseFormat(int64_t format) {
  auto from_compressed = [&](const std::shared_ptr<Compressed>& c, bool is_csc) {
    auto seg = ExpandIndptr(c->indptr, c->indices.numel());
    auto ids = AsI64(c->indices);
    if (is_csc) return std::make_shared<Coordinate>(Coordinate{ids, seg, c->e_ids, false, true});
    return std::make_shared<Coordinate>(Coordinate{seg, ids, c->e_ids, true, false});
  };
  auto to_compressed = [&](const torch::Tensor& key, const torch::Tensor& val, bool sorted,
                           int64_t nkeys) {
    torch::Tensor k = key, v = val;
    c10::optional<torch::Tensor> e_ids = coo_->e_ids;
    if (!sorted && key.is_cuda() && key.numel() < (int64_t(1) << 31) &&
        std::max(num_rows_, num_cols_) <= (int64_t)0xFFFFFFFFll) {
      // unsorted COO on the GPU: this library's counting sort by key, stable in the entries' order
      // (the reference: a device-wide radix sort, src/cuda/format_transform.cu:66-86)
      c10::cuda::CUDAGuard guard(key.device());
      const int64_t nnz = key.numel();
      auto indptr = torch::empty({nkeys + 1}, I64(key));
      auto vals = torch::empty({nnz}, I64(key)), perm = torch::empty({nnz}, I64(key));
      auto ws = NewWorkspace(gsb_group_by_key_workspace_bytes(nnz, nkeys), key.device());
      CheckStatus(gsb_group_by_key(P(key), P(val), nnz, nkeys, PM(indptr), PM(vals), PM(perm), ws.data_ptr(),
                                   (size_t)ws.numel(), AsyncErrorWord(key.device()).data_ptr<int>(),
                                   CurrentStream()),
                  "group_by_key");
      e_ids = coo_->e_ids.has_value() ? coo_->e_ids.value().index_select(0, perm) : perm;
      return std::make_shared<Compressed>(Compressed{indptr, vals, e_ids});
    }
    if (!sorted) {
      // unsorted COO: stable sort by the key (src/cuda/format_transform.cu:66-86)
      auto perm = std::get<1>(key.sort(/*stable=*/true, /*dim=*/0, /*descending=*/false));
      k = key.index_select(0, perm);
      v = val.index_select(0, perm);
      e_ids = coo_->e_ids.has_value() ? coo_->e_ids.value().index_select(0, perm) : perm;
    }
    auto indptr = torch::empty({nkeys + 1}, I64(key));
    CheckStatus(gsb_indptr_from_sorted(P(k), k.numel(), nkeys, PM(indptr), CurrentStream()),
                "indptr_from_sorted");
    return std::make_shared<Compressed>(Compressed{indptr, v, e_ids});
  };
  if (format == kCOO) {
    if (coo_) return;
    TORCH_CHECK(csc_ || csr_, "graph holds no format");
    coo_ = csc_ ? from_compressed(csc_, true) : from_compressed(csr_, false);
  } else if (format == kCSC) {
    if (csc_) return;
    if (!coo_) { TORCH_CHECK(csr_, "graph holds no format"); coo_ = from_compressed(csr_, false); }
    csc_ = to_compressed(coo_->col, coo_->row, coo_->col_sorted, num_cols_);
  } else if (format == kCSR) {
    if (csr_) return;
    if (!coo_) { TORCH_CHECK(csc_, "graph holds no format"); coo_ = from_compressed(csc_, true); }
    csr_ = to_compressed(coo_->row, coo_->col, coo_->row_sorted, num_rows_);
  } else {
    TORCH_CHECK(false, "unsupported sparse format ", format);
  }
}

torch::Tensor Graph::GetCSCIndptr() { CreateSparseFormat(kCSC); return csc_->indptr; }
torch::Tensor Graph::GetCSCIndices() { CreateSparseFormat(kCSC); return csc_->indices; }
torch::Tensor Graph::GetCSCEids() {
  CreateSparseFormat(kCSC);
  return csc_->e_ids.has_value() ? csc_->e_ids.value() : torch::Tensor();
}
torch::Tensor Graph::GetCOORows() { CreateSparseFormat(kCOO); return coo_->row; }
torch::Tensor Graph::GetCOOCols() { CreateSparseFormat(kCOO); return coo_->col; }
torch::Tensor Graph::GetCOOEids() {
  CreateSparseFormat(kCOO);
  return coo_->e_ids.has_value() ? coo_->e_ids.value() : torch::Tensor();
}
torch::Tensor Graph::GetCSRIndptr() { CreateSparseFormat(kCSR); return csr_->indptr; }
torch::Tensor Graph::GetCSRIndices() { CreateSparseFormat(kCSR); return csr_->indices; }
torch::Tensor Graph::GetCSREids() {
  CreateSparseFormat(kCSR);
  return csr_->e_ids.has_value() ? csr_->e_ids.value() : torch::Tensor();
}

torch::Tensor Graph::MapThroughEids(const c10::optional<torch::Tensor>& e_ids,
                                    torch::Tensor select) {
  // src/graph.cc:169-176
  if (!e_ids.has_value()) return select;
  if (e_ids.value().is_pinned()) return GatherRows(e_ids.value(), select);  // read in place
  return e_ids.value().index_select(0, select);
}

// data[index] for a caller-supplied id map: bounds-checked on the device and reported here as an
// exception (never as a device assert).  The operators that use it synchronise anyway.
static torch::Tensor CheckedIdGather(const torch::Tensor& data, const torch::Tensor& index,
                                     const char* what) {
  CheckIds(data, what);
  CheckIds(index, "index");
  CheckAsyncErrors();  // do not blame this call for an older, unreported error
  auto out = GatherRows(data, index);
  CheckAsyncErrors();
  return out;
}

// ------------------------------------------------------------------ kernels glue
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> Graph::SampleCompressed(
    const Compressed& src, const c10::optional<torch::Tensor>& seeds, int64_t fanout, bool replace,
    const c10::optional<torch::Tensor>& probs, int64_t num_segments) {
  c10::cuda::CUDAGuard guard(ComputeDevice(src.indptr));
  TORCH_CHECK(fanout >= 1, "fanout must be positive");
  if (seeds.has_value()) CheckIds(seeds.value(), "seeds");
  const int64_t S = seeds.has_value() ? seeds.value().numel() : num_segments;
  int64_t E_cap = S * fanout;
  if (!replace && !seeds.has_value() && src.indices.numel() < E_cap) E_cap = src.indices.numel();
  auto opt = I64(src.indptr);
  auto sub_indptr = torch::empty({S + 1}, opt);
  auto rows = torch::empty({E_cap}, opt), cols = torch::empty({E_cap}, opt),
       sel = torch::empty({E_cap}, opt);
  auto scal = torch::zeros({2}, opt);  // [0] edge count, [1] device error word
  const uint32_t stream = NextStream();
  if (probs.has_value()) {
    const auto& pr = probs.value();
    TORCH_CHECK(pr.is_cuda() && pr.scalar_type() == torch::kFloat32 && pr.is_contiguous() &&
                    pr.numel() == src.indices.numel(),
                "edge_probs must be a contiguous float32 CUDA tensor with one entry per edge");
    auto ws = NewWorkspace(gsb_sample_cols_probs_workspace_bytes(S, fanout), ComputeDevice(src.indptr));
    CheckStatus(gsb_sample_cols_probs(
                    P(src.indptr), src.indices.data_ptr(), IndicesDtype(src.indices),
                    src.indptr.numel() - 1, pr.data_ptr<float>(), seeds.has_value() ? P(seeds.value()) : nullptr, S, nullptr,
                    fanout, replace, seed_, stream, PM(sub_indptr), PM(rows), PM(cols), PM(sel),
                    E_cap, PM(scal), ws.data_ptr(), (size_t)ws.numel(),
                    (int*)(PM(scal) + 1), CurrentStream()),
                "sample_cols_probs");
  } else {
    auto ws = NewWorkspace(gsb_sample_cols_workspace_bytes(S, fanout), ComputeDevice(src.indptr));
    CheckStatus(gsb_sample_cols(P(src.indptr), src.indices.data_ptr(), IndicesDtype(src.indices),
                                src.indptr.numel() - 1, seeds.has_value() ? P(seeds.value()) : nullptr, S, nullptr, fanout,
                                replace, seed_, stream, PM(sub_indptr), PM(rows), PM(cols), PM(sel),
                                E_cap, PM(scal), ws.data_ptr(), (size_t)ws.numel(),
                                (int*)(PM(scal) + 1), CurrentStream()),
                "sample_cols");
  }
  auto host = scal.cpu();  // the one synchronisation of this operator
  const int64_t E = host.data_ptr<int64_t>()[0];
  CheckDeviceError((int)host.data_ptr<int64_t>()[1], "sample_cols");
  return {sub_indptr, rows.narrow(0, 0, E), cols.narrow(0, 0, E), sel.narrow(0, 0, E)};
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> Graph::SliceCompressed(
    const Compressed& src, torch::Tensor seeds, const c10::optional<torch::Tensor>& bptr,
    int64_t encoding_size) {
  c10::cuda::CUDAGuard guard(ComputeDevice(src.indptr));
  CheckIds(seeds, "seeds");
  const int64_t S = seeds.numel();
  auto opt = I64(src.indptr);
  auto sub_indptr = torch::empty({S + 1}, opt);
  auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(seeds.device()));
  auto ws = NewWorkspace(gsb_slice_cols_workspace_bytes(S), seeds.device());
  CheckStatus(gsb_slice_cols_count(P(src.indptr), src.indptr.numel() - 1, P(seeds), S, PM(sub_indptr), ws.data_ptr(),
                                   (size_t)ws.numel(), err.data_ptr<int>(), CurrentStream()),
              "slice_cols_count");
  const int64_t E = sub_indptr.narrow(0, S, 1).item<int64_t>();  // sizes the outputs
  CheckDeviceError(err.item<int>(), "slice_cols_count");
  auto rows = torch::empty({E}, opt), cols = torch::empty({E}, opt), sel = torch::empty({E}, opt);
  const int64_t B = bptr.has_value() ? bptr.value().numel() - 1 : 0;
  CheckStatus(gsb_slice_cols_fill(P(src.indptr), src.indices.data_ptr(), IndicesDtype(src.indices),
                                  P(seeds), S, P(sub_indptr), E, PM(rows), PM(cols), PM(sel),
                                  bptr.has_value() ? P(bptr.value()) : nullptr, B, encoding_size,
                                  CurrentStream()),
              "slice_cols_fill");
  return {sub_indptr, rows, cols, sel};
}

// ------------------------------------------------------------------ Slicing
// axis 0 = rows, 1 = columns (src/graph.cc:90-179)
Graph::GraphAndIndex Graph::Slicing(torch::Tensor seeds, int64_t axis, int64_t on_format,
                                    int64_t output_format) {
  CreateSparseFormat(on_format);
  const int64_t new_rows = axis == 0 ? seeds.numel() : num_rows_;
  const int64_t new_cols = axis == 0 ? num_cols_ : seeds.numel();
  auto ret = Derive(new_rows, new_cols);
  torch::Tensor select;
  c10::optional<torch::Tensor> e_ids;
  const bool along_indptr = (on_format == kCSC && axis == 1) || (on_format == kCSR && axis == 0);
  if (on_format == kCSC || on_format == kCSR) {
    const bool is_csc = on_format == kCSC;
    TORCH_CHECK(output_format != (is_csc ? kCSR : kCSC),
                "Slicing: output format must include the operand's format or COO");
    const auto& src = is_csc ? *csc_ : *csr_;
    e_ids = src.e_ids;
    torch::Tensor sub_indptr, ids, seg;
    if (along_indptr) {
      std::tie(sub_indptr, ids, seg, select) = SliceCompressed(src, seeds, c10::nullopt, 0);
    } else {
      std::tie(sub_indptr, ids, seg, select) =
          SliceAcross(src, seeds, is_csc ? num_cols_ : num_rows_, is_csc ? num_rows_ : num_cols_,
                      (output_format & kCOO) != 0);
    }
    if (output_format & on_format) {
      auto c = std::make_shared<Compressed>(Compressed{sub_indptr, ids, c10::nullopt});
      if (is_csc) ret->csc_ = c; else ret->csr_ = c;
    }
    if (output_format & kCOO) {
      ret->coo_ = is_csc
                      ? std::make_shared<Coordinate>(Coordinate{ids, seg, c10::nullopt, false, true})
                      : std::make_shared<Coordinate>(Coordinate{seg, ids, c10::nullopt, true, false});
    }
  } else if (on_format == kCOO) {
    torch::Tensor r, c;
    std::tie(r, c, select) = SliceCoo(seeds, axis);
    e_ids = coo_->e_ids;
    ret->coo_ = std::make_shared<Coordinate>(
        Coordinate{r, c, c10::nullopt, coo_->row_sorted, coo_->col_sorted});
  } else {
    TORCH_CHECK(false, "Slicing: unsupported on_format ", on_format);
  }
  ret->num_edges_ = select.numel();
  return {ret, MapThroughEids(e_ids, select)};
}

// ------------------------------------------------------------------ Sampling
// src/graph.cc:182-244 (uniform), :246-308 (weighted)
static void CheckSamplingFormats(int64_t axis, int64_t on_format, int64_t output_format,
                                 const char* who) {
  TORCH_CHECK((axis == 1 && on_format == kCSC) || (axis == 0 && on_format == kCSR), who,
              ": not implemented for axis=", axis, " on_format=", on_format);
  TORCH_CHECK(output_format != (on_format == kCSC ? kCSR : kCSC), who,
              ": output format must include the operand's format or COO");
}

Graph::GraphAndIndex Graph::Sampling(int64_t axis, int64_t fanout, bool replace, int64_t on_format,
                                     int64_t output_format) {
  CheckSamplingFormats(axis, on_format, output_format, "Sampling");
  CreateSparseFormat(on_format);
  const bool is_csc = on_format == kCSC;
  const auto& src = is_csc ? *csc_ : *csr_;
  auto ret = Derive(num_rows_, num_cols_);
  torch::Tensor sub_indptr, ids, seg, select;
  std::tie(sub_indptr, ids, seg, select) =
      SampleCompressed(src, c10::nullopt, fanout, replace, c10::nullopt, is_csc ? num_cols_ : num_rows_);
  ret->AttachSampled(is_csc, output_format, sub_indptr, ids, seg);
  ret->num_edges_ = select.numel();
  return {ret, MapThroughEids(src.e_ids, select)};
}

Graph::GraphAndIndex Graph::SamplingProbs(int64_t axis, torch::Tensor edge_probs, int64_t fanout,
                                          bool replace, int64_t on_format, int64_t output_format) {
  CheckSamplingFormats(axis, on_format, output_format, "SamplingProbs");
  CreateSparseFormat(on_format);
  const bool is_csc = on_format == kCSC;
  const auto& src = is_csc ? *csc_ : *csr_;
  // probabilities are given per edge id; bring them into storage order
  torch::Tensor probs = src.e_ids.has_value() ? edge_probs.index_select(0, src.e_ids.value())
                                              : edge_probs;
  auto ret = Derive(num_rows_, num_cols_);
  torch::Tensor sub_indptr, ids, seg, select;
  std::tie(sub_indptr, ids, seg, select) = SampleCompressed(
      src, c10::nullopt, fanout, replace, probs.contiguous(), is_csc ? num_cols_ : num_rows_);
  ret->AttachSampled(is_csc, output_format, sub_indptr, ids, seg);
  ret->num_edges_ = select.numel();
  return {ret, MapThroughEids(src.e_ids, select)};
}

// src/graph.cc:383-454
Graph::GraphAndIndex Graph::FusedSlicingSampling(int64_t axis, torch::Tensor seeds, int64_t fanout,
                                                 bool replace, int64_t on_format,
                                                 int64_t output_format) {
  CheckSamplingFormats(axis, on_format, output_format, "FusedSlicingSampling");
  CreateSparseFormat(on_format);
  const bool is_csc = on_format == kCSC;
  const auto& src = is_csc ? *csc_ : *csr_;
  auto ret = is_csc ? Derive(num_rows_, seeds.numel()) : Derive(seeds.numel(), num_cols_);
  torch::Tensor sub_indptr, ids, seg, select;
  std::tie(sub_indptr, ids, seg, select) =
      SampleCompressed(src, seeds, fanout, replace, c10::nullopt, 0);
  ret->AttachSampled(is_csc, output_format, sub_indptr, ids, seg);
  ret->num_edges_ = select.numel();
  return {ret, MapThroughEids(src.e_ids, select)};
}

void Graph::AttachSampled(bool is_csc, int64_t output_format, torch::Tensor sub_indptr,
                          torch::Tensor ids, torch::Tensor seg) {
  if (output_format & (is_csc ? kCSC : kCSR)) {
    auto c = std::make_shared<Compressed>(Compressed{sub_indptr, ids, c10::nullopt});
    if (is_csc) csc_ = c; else csr_ = c;
  }
  if (output_format & kCOO) {
    coo_ = is_csc ? std::make_shared<Coordinate>(Coordinate{ids, seg, c10::nullopt, false, true})
                  : std::make_shared<Coordinate>(Coordinate{seg, ids, c10::nullopt, true, false});
  }
}

// ------------------------------------------------------------------ relabel
// Shared implementation of GraphRelabel / GetValidNodes / Batch* (B >= 1).
// Returns (unique, unique_ptr, out_row, out_col); out_* undefined when
// !want_edges.
Graph::RelabelResult Graph::RelabelImpl(
    torch::Tensor col_seeds, torch::Tensor seeds_ptr, torch::Tensor coo_row, torch::Tensor coo_col,
    torch::Tensor edge_ptr, bool want_edges) {
  c10::cuda::CUDAGuard guard(col_seeds.device());
  CheckIds(col_seeds, "col_seeds");
  CheckIds(seeds_ptr, "seeds_ptr");
  CheckIds(coo_row, "rows");
  CheckIds(edge_ptr, "edge_ptr");
  const int64_t S = col_seeds.numel(), E = coo_row.numel(), B = seeds_ptr.numel() - 1;
  TORCH_CHECK(B >= 1 && edge_ptr.numel() == B + 1, "batch pointers must have B+1 entries");
  auto opt = I64(col_seeds);
  auto unique = torch::empty({S + E}, opt);
  auto unique_ptr = torch::empty({B + 1}, opt);
  torch::Tensor out_row, out_col;
  if (want_edges) {
    CheckIds(coo_col, "cols");
    out_row = torch::empty({E}, opt);
    out_col = torch::empty({E}, opt);
  }
  auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(col_seeds.device()));
  auto ws = NewWorkspace(gsb_batch_relabel_workspace_bytes(S, E, B), col_seeds.device());
  CheckStatus(gsb_batch_relabel(P(col_seeds), P(seeds_ptr), B, S, P(coo_row),
                                want_edges ? P(coo_col) : nullptr, P(edge_ptr), E,
                                /*id_bound=*/0, PM(unique), S + E,
                                PM(unique_ptr), want_edges ? PM(out_row) : nullptr,
                                want_edges ? PM(out_col) : nullptr, ws.data_ptr(), (size_t)ws.numel(),
                                err.data_ptr<int>(), CurrentStream()),
              "batch_relabel");
  const int64_t U = unique_ptr.narrow(0, B, 1).item<int64_t>();  // sizes the node list
  CheckDeviceError(err.item<int>(), "batch_relabel");
  return {unique.narrow(0, 0, U), unique_ptr, out_row, out_col};
}

static torch::Tensor Ptr2(int64_t n, const torch::Tensor& like) {
  auto t = torch::empty({2}, torch::dtype(torch::kInt64).pinned_memory(true));
  t.data_ptr<int64_t>()[0] = 0;
  t.data_ptr<int64_t>()[1] = n;
  return t.to(like.device(), /*non_blocking=*/true);
}

// src/graph.cc:577-591
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, c10::optional<torch::Tensor>>
Graph::GraphRelabel(torch::Tensor col_seeds, torch::Tensor row_ids) {
  CreateSparseFormat(kCOO);
  TORCH_CHECK(col_seeds.numel() == num_cols_ || coo_->col.numel() == 0,
              "GraphRelabel: col_seeds must hold one id per column");
  torch::Tensor coo_row = row_ids.numel() > 0 ? CheckedIdGather(row_ids, coo_->row, "row_ids") : coo_->row;
  auto r = RelabelImpl(col_seeds, Ptr2(col_seeds.numel(), col_seeds), coo_row, coo_->col,
                       Ptr2(coo_row.numel(), col_seeds), true);
  return {std::get<0>(r), std::get<2>(r), std::get<3>(r), coo_->e_ids};
}

// src/graph.cc:593-608
torch::Tensor Graph::GetValidNodes(torch::Tensor col_seeds, torch::Tensor row_ids) {
  torch::Tensor rows;
  if (csc_) {
    rows = AsI64(csc_->indices);
  } else {
    CreateSparseFormat(kCOO);
    rows = coo_->row;
  }
  if (row_ids.numel() > 0) rows = CheckedIdGather(row_ids, rows, "row_ids");
  auto r = RelabelImpl(col_seeds, Ptr2(col_seeds.numel(), col_seeds), rows, torch::Tensor(),
                       Ptr2(rows.numel(), col_seeds), false);
  return std::get<0>(r);
}

// ------------------------------------------------------------------ batch
void Graph::InheritBatch(const Graph& parent) {
  col_bptr_ = parent.col_bptr_;
  row_bptr_ = parent.row_bptr_;
  orig_col_ids_ = parent.orig_col_ids_;
  orig_row_ids_ = parent.orig_row_ids_;
  row_encoding_size_ = parent.row_encoding_size_;
}

static torch::Tensor GatherPtr(const torch::Tensor& indptr, const torch::Tensor& bptr) {
  CheckIds(bptr, "batch pointer");
  auto out = torch::empty({bptr.numel()}, I64(indptr));
  CheckStatus(gsb_gather_i64(P(indptr), P(bptr), bptr.numel(), PM(out), CurrentStream()),
              "gather");
  return out;
}

std::tuple<torch::Tensor, torch::Tensor> Graph::BatchGetCSCIndptr() {
  CreateSparseFormat(kCSC);
  return {csc_->indptr, col_bptr_};
}
std::tuple<torch::Tensor, torch::Tensor> Graph::BatchGetCSCIndices() {
  CreateSparseFormat(kCSC);
  return {csc_->indices, edge_bptr_};
}
std::tuple<torch::Tensor, torch::Tensor> Graph::BatchGetCSCEids() {
  CreateSparseFormat(kCSC);
  if (csc_->e_ids.has_value()) return {csc_->e_ids.value(), edge_bptr_};
  return {torch::Tensor(), torch::Tensor()};
}
std::tuple<torch::Tensor, torch::Tensor> Graph::BatchGetCOORows() {
  CreateSparseFormat(kCOO);
  return {coo_->row, edge_bptr_};
}
std::tuple<torch::Tensor, torch::Tensor> Graph::BatchGetCOOCols() {
  CreateSparseFormat(kCOO);
  return {coo_->col, edge_bptr_};
}
std::tuple<torch::Tensor, torch::Tensor> Graph::BatchGetCOOEids() {
  CreateSparseFormat(kCOO);
  if (coo_->e_ids.has_value()) return {coo_->e_ids.value(), edge_bptr_};
  return {torch::Tensor(), torch::Tensor()};
}

std::vector<int64_t> Graph::BatchGetColCounts() {
  TORCH_CHECK(col_bptr_.defined(), "graph has no column batch pointer");
  auto host = col_bptr_.cpu();
  const int64_t* p = host.data_ptr<int64_t>();
  std::vector<int64_t> out(host.numel() - 1);
  for (size_t i = 0; i < out.size(); ++i) out[i] = p[i + 1] - p[i];
  return out;
}

// src/batch_graph.cc:13-104
Graph::GraphAndIndex Graph::BatchColSlicing(torch::Tensor seeds, torch::Tensor col_bptr,
                                            bool encoding) {
  CreateSparseFormat(kCSC);
  CheckIds(col_bptr, "col_bptr");
  const int64_t B = col_bptr.numel() - 1;
  torch::Tensor sub_indptr, ids, seg, select;
  std::tie(sub_indptr, ids, seg, select) =
      SliceCompressed(*csc_, seeds, col_bptr, encoding ? num_rows_ : 0);
  torch::Tensor row_bptr, orig_row_ids;
  if (encoding) {
    // sorted unique of the encoded ids + remap (src/cuda/compact.cu:10-30), then
    // split the unique list per minibatch (src/cuda/batch/encoding_decoding.cu:99-122)
    torch::Tensor enc;
    const int64_t bound = num_rows_ * B;  // the encoded ids lie below it
    if (ids.is_cuda() && num_rows_ > 0 && bound / num_rows_ == B && bound < (int64_t(1) << 40)) {
      // presence table over the encoded range (gsb_compact_*): 3/8 of a byte per possible id
      c10::cuda::CUDAGuard guard(ids.device());
      ids = ids.to(torch::kInt64).contiguous();
      auto ws = NewWorkspace(gsb_compact_workspace_bytes(bound), ids.device());
      auto count = torch::empty({1}, I64(ids));
      auto err = torch::zeros({1}, torch::dtype(torch::kInt32).device(ids.device()));
      CheckStatus(gsb_compact_rank(ids.data_ptr(), GSB_I64, ids.numel(), bound, ws.data_ptr(), (size_t)ws.numel(),
                                   PM(count), err.data_ptr<int>(), CurrentStream()),
                  "compact_rank");
      const int64_t U = count.item<int64_t>();  // sizes the list of distinct ids
      CheckDeviceError(err.item<int>(), "BatchColSlicing");
      enc = torch::empty({U}, I64(ids));
      auto mapped = torch::empty({ids.numel()}, I64(ids));
      CheckStatus(gsb_compact_apply(ws.data_ptr(), bound, PM(enc), ids.data_ptr(), GSB_I64, ids.numel(),
                                    PM(mapped), CurrentStream()),
                  "compact_apply");
      ids = mapped;
    } else {  // not on the GPU, or an encoded range of 2^40 and more: the library's sorted unique
      auto uq = torch::_unique2(ids, /*sorted=*/true, /*return_inverse=*/true, false);
      enc = std::get<0>(uq);
      ids = std::get<1>(uq);
    }
    auto batch_of = torch::floor_divide(enc, num_rows_);
    orig_row_ids = enc - batch_of * num_rows_;
    row_bptr = torch::empty({B + 1}, I64(enc));
    CheckStatus(gsb_indptr_from_sorted(P(batch_of), batch_of.numel(), B, PM(row_bptr), CurrentStream()),
                "indptr_from_sorted");
  }
  auto ret = Derive(encoding ? orig_row_ids.numel() : num_rows_ * B, seeds.numel());
  ret->csc_ = std::make_shared<Compressed>(Compressed{sub_indptr, ids, c10::nullopt});
  ret->coo_ = std::make_shared<Coordinate>(Coordinate{ids, seg, c10::nullopt, false, true});
  ret->num_edges_ = select.numel();
  ret->col_bptr_ = col_bptr;
  ret->orig_col_ids_ = seeds;
  ret->edge_bptr_ = GatherPtr(sub_indptr, col_bptr);
  if (encoding) {
    ret->row_bptr_ = row_bptr;
    ret->orig_row_ids_ = orig_row_ids;
    ret->row_encoding_size_ = num_rows_;
  }
  return {ret, MapThroughEids(csc_->e_ids, select)};
}

// src/batch_graph.cc:159-172
Graph::GraphAndIndex Graph::BatchRowSampling(int64_t fanout, bool replace) {
  auto r = Sampling(1, fanout, replace, kCSC, kCSC + kCOO);
  auto g = std::get<0>(r);
  g->InheritBatch(*this);
  g->edge_bptr_ = GatherPtr(g->csc_->indptr, col_bptr_);
  return r;
}

// src/batch_graph.cc:174-188
Graph::GraphAndIndex Graph::BatchRowSamplingProbs(int64_t fanout, bool replace,
                                                  torch::Tensor edge_probs) {
  auto r = SamplingProbs(1, edge_probs, fanout, replace, kCSC, kCSC + kCOO);
  auto g = std::get<0>(r);
  g->InheritBatch(*this);
  g->edge_bptr_ = GatherPtr(g->csc_->indptr, col_bptr_);
  return r;
}

// src/batch_graph.cc:190-212
Graph::GraphAndIndex Graph::BatchFusedSlicingSampling(torch::Tensor seeds, torch::Tensor col_bptr,
                                                      int64_t fanout, bool replace) {
  auto r = FusedSlicingSampling(1, seeds, fanout, replace, kCSC, kCSC + kCOO);
  auto g = std::get<0>(r);
  g->col_bptr_ = col_bptr;
  g->orig_col_ids_ = seeds;
  g->edge_bptr_ = GatherPtr(g->csc_->indptr, col_bptr);
  return r;
}

// Shared by BatchGraphRelabel / BatchGetValidNodes (src/batch_graph.cc:214-284).
// The reference runs the whole relabel for each of the two calls; here the
// first call of a pair computes everything and the second one is served from
// the cached result (keyed by the identity of the argument tensors).
Graph::RelabelResult Graph::BatchRelabelImpl(torch::Tensor col_seeds, torch::Tensor row_ids) {
  TORCH_CHECK(edge_bptr_.defined() && edge_bptr_.numel() > 0,
              "batch relabel needs the edge batch pointer (slice with seeds::ptr first)");
  CreateSparseFormat(kCOO);
  TORCH_CHECK(coo_->col_sorted, "batch relabel requires a column-sorted COO");
  auto same = [](const torch::Tensor& a, const torch::Tensor& b) {
    return a.numel() == b.numel() && (a.numel() == 0 || a.data_ptr() == b.data_ptr());
  };
  if (relabel_cache_ && same(relabel_cache_->col_seeds, col_seeds) &&
      same(relabel_cache_->row_ids, row_ids))
    return relabel_cache_->value;
  torch::Tensor coo_row = coo_->row;
  if (row_ids.numel() > 0) {
    // encoded row ids: decode back to graph ids (encoding_decoding.cu:99-122)
    auto enc = CheckedIdGather(row_ids, coo_->row, "row_ids");
    coo_row = row_encoding_size_ > 0 ? torch::remainder(enc, row_encoding_size_) : enc;
  }
  auto r = RelabelImpl(col_seeds, col_bptr_, coo_row, coo_->col, edge_bptr_, true);
  relabel_cache_ = std::make_shared<RelabelCache>(RelabelCache{col_seeds, row_ids, r});
  return r;
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, c10::optional<torch::Tensor>,
           torch::Tensor>
Graph::BatchGraphRelabel(torch::Tensor col_seeds, torch::Tensor row_ids) {
  auto r = BatchRelabelImpl(col_seeds, row_ids);
  return {std::get<0>(r), std::get<1>(r), std::get<2>(r), std::get<3>(r), coo_->e_ids, edge_bptr_};
}

std::tuple<torch::Tensor, torch::Tensor> Graph::BatchGetValidNodes(torch::Tensor col_seeds,
                                                                   torch::Tensor row_ids) {
  auto r = BatchRelabelImpl(col_seeds, row_ids);
  return {std::get<0>(r), std::get<1>(r)};
}

}  // namespace gsb_host
