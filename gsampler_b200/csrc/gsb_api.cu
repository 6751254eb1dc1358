// Library-level entry points: version, status strings, and the multi-layer
// GraphSAGE sampler that chains the per-stage launches on one stream without
// any host synchronisation (all intermediate sizes stay on the device).
#include <atomic>
#include <mutex>
#include <vector>

#include "gsb_common.cuh"

namespace gsb {

static thread_local const char* g_last_cuda_error = "";


// ---------------------------------------------------------------- launch accounting
static const char* const kKernelNames[KID_NUM] = {
    "sample_tile", "sample_probs", "count", "slice_fill", "gather", "expand_indptr",
    "indptr_from_sorted", "relabel_setup", "relabel_pcount", "relabel_pscan", "relabel_scatter",
    "relabel_dedupe", "relabel_mark", "relabel_prefix", "relabel_rank", "relabel_emit",
    "slice_rows", "edge_sum", "edge_op", "list_sample", "walk", "sort", "sample_probs_short",
    "sample_probs_long", "misc"};

struct TimedLaunch {
  int id, tag;
  cudaEvent_t start, stop;
};

static std::atomic<unsigned long long> g_launches{0};
static std::mutex g_timing_mutex;
static bool g_timing_on = false;
static int g_timing_tag = 0;
static std::vector<TimedLaunch> g_timed;      // events of the current collection window
static std::vector<cudaEvent_t> g_event_pool;  // recycled events

static cudaEvent_t pool_event() {
  if (!g_event_pool.empty()) {
    cudaEvent_t e = g_event_pool.back();
    g_event_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

LaunchScope::LaunchScope(int id_, cudaStream_t st_) : id(id_), st(st_), slot(-1) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_timing_on) return;
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  TimedLaunch t{id, g_timing_tag, pool_event(), pool_event()};
  if (!t.start || !t.stop) return;
  cudaEventRecord(t.start, st);
  g_timed.push_back(t);
  slot = (int)g_timed.size() - 1;
}

LaunchScope::~LaunchScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  if (slot < (int)g_timed.size()) cudaEventRecord(g_timed[(size_t)slot].stop, st);
}

void set_timing_tag(int tag) { g_timing_tag = tag; }

int sm_count() {
  constexpr int MAX_DEV = 64;
  static std::atomic<int> cached[MAX_DEV];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) return 148;
  cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_abi_version(void) { return 1; }

extern "C" uint64_t gsb_kernel_launches(void) { return g_launches.load(); }

extern "C" int gsb_timing_enable(int on) {
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  for (auto& t : g_timed) { g_event_pool.push_back(t.start); g_event_pool.push_back(t.stop); }
  g_timed.clear();
  g_timing_on = on != 0;
  g_timing_tag = 0;
  return GSB_OK;
}

extern "C" int gsb_timing_collect(int max_entries, const char** names, int* tags, double* total_ms,
                                  int64_t* launches) {
  if (max_entries < 0 || (max_entries > 0 && (!names || !tags || !total_ms || !launches))) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  int n = 0;
  for (auto& t : g_timed) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, t.start, t.stop) != cudaSuccess) continue;
    int k = 0;
    for (; k < n; ++k)
      if (names[k] == kKernelNames[t.id] && tags[k] == t.tag) break;
    if (k == n) {
      if (n == max_entries) continue;
      names[n] = kKernelNames[t.id]; tags[n] = t.tag; total_ms[n] = 0; launches[n] = 0;
      ++n;
    }
    total_ms[k] += ms;
    launches[k] += 1;
  }
  return n;
}

extern "C" const char* gsb_status_string(int status) {
  switch (status) {
    case GSB_OK: return "ok";
    case GSB_ERR_INVALID: return "invalid argument";
    case GSB_ERR_UNSUPPORTED: return "request outside the supported range";
    case GSB_ERR_WORKSPACE: return "workspace missing or too small";
    case GSB_ERR_CUDA: return "CUDA runtime error";
    case GSB_ERR_SCRATCH_LIMIT: return "size exceeds the fixed scratch of this entry point";
    default: return "unknown status";
  }
}

extern "C" const char* gsb_last_cuda_error(void) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) g_last_cuda_error = cudaGetErrorString(e);
  return g_last_cuda_error;
}

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

extern "C" size_t gsb_graphsage_workspace_bytes(int64_t B, int num_layers,
                                                const gsb_layer_buffers* layers,
                                                const int64_t* fanouts) {
  if (!layers || !fanouts || num_layers < 1 || B < 1) return 0;
  size_t need = 0;
  for (int l = 0; l < num_layers; ++l) {
    size_t a = align256(gsb_sample_cols_workspace_bytes(layers[l].S_cap, fanouts[l]));
    size_t b = align256(gsb_batch_relabel_workspace_bytes(layers[l].S_cap, layers[l].E_cap, B));
    if (a + b > need) need = a + b;
  }
  return need;
}

extern "C" int gsb_graphsage_sample(const int64_t* indptr, const void* indices, int indices_dtype,
                                    int64_t num_cols, int64_t id_bound, const int64_t* seeds,
                                    const int64_t* seeds_ptr, int64_t B, int64_t S0,
                                    int num_layers, const int64_t* fanouts, uint64_t seed,
                                    uint32_t stream_base, const gsb_layer_buffers* layers,
                                    int64_t* d_counts,
                                    void* workspace, size_t workspace_bytes, int* d_err,
                                    void* cuda_stream) {
  if (!indptr || !indices || !seeds_ptr || !layers || !fanouts || !d_counts || num_layers < 1 ||
      B < 1 || S0 < 0 || (S0 > 0 && !seeds))
    return GSB_ERR_INVALID;
  if (workspace_bytes < gsb_graphsage_workspace_bytes(B, num_layers, layers, fanouts) || !workspace)
    return GSB_ERR_WORKSPACE;
  // The node lists of layer l are the seeds of layer l+1.  S_cap[l+1] >=
  // S_cap[l] + E_cap[l] can never overflow; smaller capacities are accepted and
  // checked on the device (GSB_ERRBIT_CAPACITY).
  if (layers[0].S_cap < S0) return GSB_ERR_INVALID;

  const int64_t* cur_seeds = seeds;
  const int64_t* cur_ptr = seeds_ptr;
  // the live seed count is read on the device for every layer (seeds_ptr[B] for the first one),
  // so S0 is only an upper bound: a recorded CUDA graph can be replayed on a shorter super-batch
  const int64_t* d_S = seeds_ptr + B;
  for (int l = 0; l < num_layers; ++l) {
    const gsb_layer_buffers& L = layers[l];
    const int64_t S_max = l == 0 ? S0 : L.S_cap;
    set_timing_tag(l);
    const size_t ws_a = align256(gsb_sample_cols_workspace_bytes(L.S_cap, fanouts[l]));
    // the sampler also writes block_col = slot - first slot of the minibatch, which is the
    // relabelled column wherever the minibatch's seeds are distinct (the relabel stage rewrites
    // the other minibatches)
    int rc = sample_launch(indptr, indices, indices_dtype, num_cols, cur_seeds, S_max, d_S, fanouts[l], 0,
                           seed, stream_base + (uint32_t)l, L.sub_indptr, L.rows, L.cols, L.sel, L.E_cap,
                           d_counts + 3 * l + 1, cur_ptr, B, L.block_col, L.S_cap, workspace, ws_a, d_err,
                           cuda_stream);
    if (rc != GSB_OK) return rc;
    // edge_ptr = sub_indptr[seeds_ptr] and the {S, U} counts are produced inside the relabel passes
    rc = relabel_launch(cur_seeds, cur_ptr, B, S_max, L.rows, L.cols, nullptr, L.sub_indptr,
                        L.edge_ptr, L.E_cap, id_bound, L.unique, L.S_cap + L.E_cap, L.unique_ptr,
                        L.block_row, L.block_col, d_counts + 3 * l, 1, (char*)workspace + ws_a,
                        workspace_bytes - ws_a, d_err, cuda_stream);
    if (rc != GSB_OK) return rc;
    cur_seeds = L.unique;
    cur_ptr = L.unique_ptr;
    d_S = L.unique_ptr + B;
  }
  set_timing_tag(0);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
