// Random walks over the in-neighbour lists of a CSC graph: uniform walks and
// node2vec (second-order, rejection sampled).
//
// A thread owns a walker for all its steps (the steps are sequentially
// dependent).  The walker keeps its current and previous node in registers --
// the trace in global memory is write-only -- and consumes the draws of its own
// counter-based stream in order, so a trace depends only on (seed, stream,
// walker index), never on the launch geometry.  Traces are stored step-major,
// trace[s * N + w], which makes every step's store coalesced across walkers.
#include "gsb_common.cuh"

namespace gsb {

constexpr int WALK_THREADS = 256;

template <typename IndexT>
__global__ void __launch_bounds__(WALK_THREADS)
random_walk_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices,
                   i64 num_nodes, const i64* __restrict__ seeds, i64 N, int L, u64 seed,
                   u32 stream, i64* __restrict__ out, int* err) {
  for (i64 w = (i64)blockIdx.x * WALK_THREADS + threadIdx.x; w < N;
       w += (i64)gridDim.x * WALK_THREADS) {
    i64 cur = seeds[w];
    out[w] = cur;
    if (cur >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); cur = -1; }
    StreamReader rng;
    rng.init(seed, stream, (u64)w);
    for (int s = 0; s < L; ++s) {
      i64 pick = -1;
      if (cur >= 0) {
        const i64 st = __ldg(indptr + cur);
        const i64 deg = __ldg(indptr + cur + 1) - st;
        if (deg > 0) pick = load_index<IndexT>(indices, st + (i64)__umulhi(rng.next(), (u32)deg));
        // a row id that is not a column (more rows than columns) ends the walk instead of
        // indexing the offsets out of bounds
        if (pick >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); pick = -1; }
      }
      out[(i64)(s + 1) * N + w] = pick;
      cur = pick;
    }
  }
}

// is `dst` an entry of column `src`?  Columns must be sorted ascending.
template <typename IndexT>
__device__ __forceinline__ bool column_contains(const i64* __restrict__ indptr,
                                                const void* __restrict__ indices, i64 num_nodes,
                                                i64 src, i64 dst) {
  if (src < 0 || src >= num_nodes) return false;
  i64 lo = __ldg(indptr + src);
  const i64 end = __ldg(indptr + src + 1);
  i64 hi = end;
  while (lo < hi) {
    const i64 mid = (lo + hi) >> 1;
    if (load_index<IndexT>(indices, mid) < dst) lo = mid + 1; else hi = mid;
  }
  return lo < end && load_index<IndexT>(indices, lo) == dst;
}

template <typename IndexT>
__global__ void __launch_bounds__(WALK_THREADS)
node2vec_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 num_nodes,
                const i64* __restrict__ seeds, i64 N, int L, double p, double q, u64 seed,
                u32 stream, i64* __restrict__ out, int* err) {
  const double max_scale = p > q ? p : q;
  const double reject_from = max_scale > 1.0 ? max_scale : 1.0;
  double accept_below = p < q ? p : q;
  if (accept_below > 1.0) accept_below = 1.0;
  const double inv32 = 1.0 / 4294967296.0;
  for (i64 w = (i64)blockIdx.x * WALK_THREADS + threadIdx.x; w < N;
       w += (i64)gridDim.x * WALK_THREADS) {
    i64 cur = seeds[w];
    i64 last = w;  // the reference starts the "previous node" at the walker's index
    out[w] = cur;
    if (cur >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); cur = -1; }
    StreamReader rng;
    rng.init(seed, stream, (u64)w);
    for (int s = 0; s < L; ++s) {
      i64 pick = -1;
      if (cur >= 0) {
        const i64 st = __ldg(indptr + cur);
        const i64 deg = __ldg(indptr + cur + 1) - st;
        if (deg == 1) {
          pick = load_index<IndexT>(indices, st);
        } else if (deg > 1) {
          // bounded rejection loop: the acceptance probability is at least
          // min(1, 1/max(p,q)) per round, so 1<<16 rounds never run out in practice
          for (int round = 0; round < (1 << 16); ++round) {
            const double u1 = ((double)rng.next() + 1.0) * inv32;
            const int y = (int)floor(u1 * max_scale);
            if ((double)y >= reject_from) continue;
            const double u2 = ((double)rng.next() + 1.0) * inv32;
            i64 x = (i64)floor(u2 * (double)deg);
            if (x >= deg) x = deg - 1;
            const i64 cand = load_index<IndexT>(indices, st + x);
            if ((double)y < accept_below) { pick = cand; break; }
            // h = p for a return, q for a neighbour of the previous node, 1
            // otherwise.  The membership search only matters when q and 1 lie
            // on different sides of y; for (p, q) = (2, 0.5) it never runs.
            double h;
            if (cand == last) h = p;
            else if (((double)y < q) == ((double)y < 1.0)) h = 1.0;
            else if (column_contains<IndexT>(indptr, indices, num_nodes, last, cand)) h = q;
            else h = 1.0;
            if ((double)y < h) { pick = cand; break; }
          }
          if (pick < 0) raise(err, ERRBIT_LOOKBACK_TIMEOUT);
        }
        if (pick >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); pick = -1; }
      }
      out[(i64)(s + 1) * N + w] = pick;
      last = cur;
      cur = pick;
    }
  }
}

static int walk_grid(i64 N) {
  i64 blocks = (N + WALK_THREADS - 1) / WALK_THREADS;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_random_walk(const int64_t* indptr, const void* indices, int indices_dtype,
                               int64_t num_nodes, const int64_t* seeds, int64_t N,
                               int64_t walk_length, uint64_t seed, uint32_t stream, int64_t* out,
                               int* d_err, void* cuda_stream) {
  if (N == 0) return GSB_OK;
  if (!indptr || !indices || !seeds || !out || N < 0 || walk_length < 0 || num_nodes < 0)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (walk_length > (1 << 30)) return GSB_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_WALK, st);
  if (indices_dtype == GSB_I32)
    random_walk_kernel<int><<<walk_grid(N), WALK_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_nodes, (const i64*)seeds, N, (int)walk_length, seed, stream,
        (i64*)out, d_err);
  else
    random_walk_kernel<i64><<<walk_grid(N), WALK_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_nodes, (const i64*)seeds, N, (int)walk_length, seed, stream,
        (i64*)out, d_err);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_node2vec(const int64_t* indptr, const void* indices, int indices_dtype,
                            int64_t num_nodes, const int64_t* seeds, int64_t N,
                            int64_t walk_length, double p, double q, uint64_t seed,
                            uint32_t stream, int64_t* out, int* d_err, void* cuda_stream) {
  if (N == 0) return GSB_OK;
  if (!indptr || !indices || !seeds || !out || N < 0 || walk_length < 0 || num_nodes < 0)
    return GSB_ERR_INVALID;
  if (!(p > 0.0) || !(q > 0.0)) return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (walk_length > (1 << 30)) return GSB_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_WALK, st);
  if (indices_dtype == GSB_I32)
    node2vec_kernel<int><<<walk_grid(N), WALK_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_nodes, (const i64*)seeds, N, (int)walk_length, p, q, seed,
        stream, (i64*)out, d_err);
  else
    node2vec_kernel<i64><<<walk_grid(N), WALK_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_nodes, (const i64*)seeds, N, (int)walk_length, p, q, seed,
        stream, (i64*)out, d_err);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
