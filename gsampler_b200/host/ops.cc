#include "ops.h"

#include <c10/cuda/CUDAGuard.h>

#include "graph.h"
#include "gsb200.h"

namespace gsb_host {

// src/cuda/batch/batch_split.cu:107-119: one D2H of the sizes, then views.
std::vector<torch::Tensor> SplitByOffset(torch::Tensor data, torch::Tensor offset) {
  auto host = offset.to(torch::kCPU, torch::kInt64);
  const int64_t* p = host.data_ptr<int64_t>();
  std::vector<int64_t> sizes((size_t)host.numel() - 1);
  for (size_t i = 0; i < sizes.size(); ++i) sizes[i] = p[i + 1] - p[i];
  return torch::split_with_sizes(data, sizes);
}

// src/cuda/batch/batch_split.cu:50-95: piece b = indptr[off[b] .. off[b+1]]
// rebased to start at zero (off[b+1]-off[b]+1 entries).
std::vector<torch::Tensor> SplitIndptrByOffset(torch::Tensor indptr, torch::Tensor offsets) {
  CheckIds(indptr, "indptr");
  auto host = offsets.to(torch::kCPU, torch::kInt64);
  const int64_t* p = host.data_ptr<int64_t>();
  std::vector<torch::Tensor> out;
  for (int64_t b = 0; b + 1 < host.numel(); ++b) {
    auto piece = indptr.narrow(0, p[b], p[b + 1] - p[b] + 1);
    out.push_back(piece - piece.narrow(0, 0, 1));
  }
  return out;
}

}  // namespace gsb_host
