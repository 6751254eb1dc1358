// Free operators behind torch.ops.gs_ops.* (src/pybind.cc:69-78,
// src/tensor_ops.h:18-30, src/cuda/batch/batch_ops.h:22-23,77-78 in gSampler).
#pragma once
#include <torch/script.h>

#include <tuple>
#include <vector>

namespace gsb_host {

torch::Tensor ListSampling(int64_t num_items, int64_t num_picks, bool replace);
torch::Tensor ListSamplingProbs(torch::Tensor probs, int64_t num_picks, bool replace);
std::tuple<torch::Tensor, torch::Tensor> BatchListSamplingProbs(torch::Tensor probs,
                                                                int64_t num_picks, bool replace,
                                                                torch::Tensor range);
std::tuple<torch::Tensor, torch::Tensor> BatchListSampling(int64_t num_picks, bool replace,
                                                           torch::Tensor range);
std::vector<torch::Tensor> SplitByOffset(torch::Tensor data, torch::Tensor offset);
std::vector<torch::Tensor> SplitIndptrByOffset(torch::Tensor indptr, torch::Tensor offsets);
torch::Tensor IndexSearch(torch::Tensor origin_data, torch::Tensor keys);
// row gather from GPU or pinned host memory (src/cuda/index_select_uvm.cu:22-49); sync-free:
// a bad index raises a bit that CheckAsyncErrors reports
torch::Tensor GatherRows(torch::Tensor data, torch::Tensor index);
void CheckAsyncErrors();
// random stream of the list-sampling operators (the reference hard-codes 7777,
// src/cuda/list_sampling.cu:36); a per-process call counter advances the stream
uint64_t ListSamplingSeed();
uint32_t NextListStream();
void SetListSamplingSeed(int64_t seed);

}  // namespace gsb_host
