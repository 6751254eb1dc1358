// Random walks over the in-neighbour lists of a CSC graph: uniform walks and
// node2vec (second-order, rejection sampled).
//
// A thread owns a walker for all its steps (the steps are sequentially
// dependent).  The walker keeps its current and previous node in registers --
// the trace in global memory is write-only -- and consumes the draws of its own
// counter-based stream in order, so a trace depends only on (seed, stream,
// walker index), never on the launch geometry.  Traces are stored step-major,
// trace[s * N + w], which makes every step's store coalesced across walkers.
//
// A step is two dependent random accesses: the offsets pair of the current node, then one row
// id.  The offsets array is small (4 or 8 bytes per node) and every walker reads it at random
// at every step, so it is loaded with an evict-last policy and the trace stores -- never read
// again -- are marked evict-first: the offsets then stay in L2 and a step costs one DRAM access
// instead of two.  What is left is the rate at which the memory system serves random 32-byte
// gathers from the row-id array, which grows with the share of that array L2 holds: hence the
// 32-bit copies of offsets and row ids the caller may pass, and the normal (not evict-first)
// policy on the gathers.
#include "gsb_common.cuh"

namespace gsb {

constexpr int WALK_THREADS = 256;
#ifndef GSB_WALK_MIN_CTAS
#define GSB_WALK_MIN_CTAS 4
#endif

// The two offsets of a node, kept in L2.  With 32-bit offsets (a copy the caller keeps when the
// graph has fewer than 2^32 entries) the array every walker gathers from at every step is half
// the size.
__device__ __forceinline__ void load_bounds(const i64* p, i64 node, u64 keep_pol, i64& st, i64& deg) {
  st = ld_i64_keep(p + node, keep_pol);
  deg = ld_i64_keep(p + node + 1, keep_pol) - st;
}
__device__ __forceinline__ void load_bounds(const u32* p, i64 node, u64 keep_pol, i64& st, i64& deg) {
  u32 a, b;
  asm volatile("ld.global.nc.L1::evict_last.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(a) : "l"(p + node), "l"(keep_pol));
  asm volatile("ld.global.nc.L1::evict_last.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(b) : "l"(p + node + 1), "l"(keep_pol));
  st = (i64)a;
  deg = (i64)(b - a);
}

// L2 policy of the row-id gathers: 0 evict-first, 1 evict-last, 2 normal.  The gathers land at
// random places of an array several times the size of L2; the share of it that L2 happens to hold
// is the only reuse there is, and marking the lines evict-first lowers it (1 000 000 walkers x 80
// steps on a 124 M-entry graph: 1.78 ms with 0, 1.71 ms with 1 or 2).
#ifndef GSB_WALK_GATHER
#define GSB_WALK_GATHER 2
#endif
__device__ __forceinline__ u64 walk_gather_policy() {
#if GSB_WALK_GATHER == 0
  return l2_policy_stream();
#elif GSB_WALK_GATHER == 1
  return l2_policy_keep();
#else
  u64 pol;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
#endif
}

template <typename IndexT, typename OffT>
__global__ void __launch_bounds__(WALK_THREADS, GSB_WALK_MIN_CTAS)
random_walk_kernel(const OffT* __restrict__ indptr, const void* __restrict__ indices,
                   i64 num_nodes, const i64* __restrict__ seeds, i64 N, int L, u64 seed,
                   u32 stream, i64* __restrict__ out, int* err) {
  const u64 keep_pol = l2_policy_keep(), stream_pol = l2_policy_stream();
  const u64 gather_pol = walk_gather_policy();
  for (i64 w = (i64)blockIdx.x * WALK_THREADS + threadIdx.x; w < N;
       w += (i64)gridDim.x * WALK_THREADS) {
    i64 cur = seeds[w];
    st_i64_stream(out + w, cur, stream_pol);
    if (cur >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); cur = -1; }
    StreamReader rng;
    rng.init(seed, stream, (u64)w);
    for (int s = 0; s < L; ++s) {
      i64 pick = -1;
      if (cur >= 0) {
        i64 st, deg;
        load_bounds(indptr, cur, keep_pol, st, deg);
        if (deg > 0)
          pick = load_index_stream<IndexT>(indices, st + (i64)__umulhi(rng.next(), (u32)deg), gather_pol);
        // a row id that is not a column (more rows than columns) ends the walk instead of
        // indexing the offsets out of bounds
        if (pick >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); pick = -1; }
      }
      st_i64_stream(out + (i64)(s + 1) * N + w, pick, stream_pol);
      cur = pick;
    }
  }
}

// is `dst` an entry of column `src`?  Columns must be sorted ascending.
template <typename IndexT, typename OffT>
__device__ __forceinline__ bool column_contains(const OffT* __restrict__ indptr,
                                                const void* __restrict__ indices, i64 num_nodes,
                                                i64 src, i64 dst, u64 keep_pol) {
  if (src < 0 || src >= num_nodes) return false;
  i64 lo, len;
  load_bounds(indptr, src, keep_pol, lo, len);
  const i64 end = lo + len;
  i64 hi = end;
  while (lo < hi) {
    const i64 mid = (lo + hi) >> 1;
    if (load_index<IndexT>(indices, mid) < dst) lo = mid + 1; else hi = mid;
  }
  return lo < end && load_index<IndexT>(indices, lo) == dst;
}

template <typename IndexT, typename OffT>
__global__ void __launch_bounds__(WALK_THREADS, GSB_WALK_MIN_CTAS)
node2vec_kernel(const OffT* __restrict__ indptr, const void* __restrict__ indices, i64 num_nodes,
                const i64* __restrict__ seeds, i64 N, int L, double p, double q, u64 seed,
                u32 stream, i64* __restrict__ out, int* err) {
  const double max_scale = p > q ? p : q;
  const double reject_from = max_scale > 1.0 ? max_scale : 1.0;
  double accept_below = p < q ? p : q;
  if (accept_below > 1.0) accept_below = 1.0;
  const double inv32 = 1.0 / 4294967296.0;
  const u64 keep_pol = l2_policy_keep(), stream_pol = l2_policy_stream();
  const u64 gather_pol = walk_gather_policy();
  for (i64 w = (i64)blockIdx.x * WALK_THREADS + threadIdx.x; w < N;
       w += (i64)gridDim.x * WALK_THREADS) {
    i64 cur = seeds[w];
    i64 last = w;  // the reference starts the "previous node" at the walker's index
    st_i64_stream(out + w, cur, stream_pol);
    if (cur >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); cur = -1; }
    StreamReader rng;
    rng.init(seed, stream, (u64)w);
    for (int s = 0; s < L; ++s) {
      i64 pick = -1;
      if (cur >= 0) {
        i64 st, deg;
        load_bounds(indptr, cur, keep_pol, st, deg);
        if (deg == 1) {
          pick = load_index_stream<IndexT>(indices, st, gather_pol);
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
            const i64 cand = load_index_stream<IndexT>(indices, st + x, gather_pol);
            if ((double)y < accept_below) { pick = cand; break; }
            // h = p for a return, q for a neighbour of the previous node, 1
            // otherwise.  The membership search only matters when q and 1 lie
            // on different sides of y; for (p, q) = (2, 0.5) it never runs.
            double h;
            if (cand == last) h = p;
            else if (((double)y < q) == ((double)y < 1.0)) h = 1.0;
            else if (column_contains<IndexT>(indptr, indices, num_nodes, last, cand, keep_pol)) h = q;
            else h = 1.0;
            if ((double)y < h) { pick = cand; break; }
          }
          if (pick < 0) raise(err, ERRBIT_LOOKBACK_TIMEOUT);
        }
        if (pick >= num_nodes) { raise(err, ERRBIT_BAD_INPUT); pick = -1; }
      }
      st_i64_stream(out + (i64)(s + 1) * N + w, pick, stream_pol);
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

extern "C" int gsb_random_walk(const int64_t* indptr, const uint32_t* indptr32, const void* indices,
                               int indices_dtype, int64_t num_nodes, const int64_t* seeds, int64_t N,
                               int64_t walk_length, uint64_t seed, uint32_t stream, int64_t* out,
                               int* d_err, void* cuda_stream) {
  if (N == 0) return GSB_OK;
  if ((!indptr && !indptr32) || !indices || !seeds || !out || N < 0 || walk_length < 0 || num_nodes < 0)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (walk_length > (1 << 30)) return GSB_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_WALK, st);
  auto go = [&](auto kernel, auto offsets) {
    kernel<<<walk_grid(N), WALK_THREADS, 0, st>>>(offsets, indices, num_nodes, (const i64*)seeds, N,
                                                  (int)walk_length, seed, stream, (i64*)out, d_err);
  };
  if (indptr32) {
    if (indices_dtype == GSB_I32) go(random_walk_kernel<int, u32>, (const u32*)indptr32);
    else go(random_walk_kernel<i64, u32>, (const u32*)indptr32);
  } else {
    if (indices_dtype == GSB_I32) go(random_walk_kernel<int, i64>, (const i64*)indptr);
    else go(random_walk_kernel<i64, i64>, (const i64*)indptr);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_node2vec(const int64_t* indptr, const uint32_t* indptr32, const void* indices,
                            int indices_dtype, int64_t num_nodes, const int64_t* seeds, int64_t N,
                            int64_t walk_length, double p, double q, uint64_t seed,
                            uint32_t stream, int64_t* out, int* d_err, void* cuda_stream) {
  if (N == 0) return GSB_OK;
  if ((!indptr && !indptr32) || !indices || !seeds || !out || N < 0 || walk_length < 0 || num_nodes < 0)
    return GSB_ERR_INVALID;
  if (!(p > 0.0) || !(q > 0.0)) return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (walk_length > (1 << 30)) return GSB_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_WALK, st);
  auto go = [&](auto kernel, auto offsets) {
    kernel<<<walk_grid(N), WALK_THREADS, 0, st>>>(offsets, indices, num_nodes, (const i64*)seeds, N,
                                                  (int)walk_length, p, q, seed, stream, (i64*)out, d_err);
  };
  if (indptr32) {
    if (indices_dtype == GSB_I32) go(node2vec_kernel<int, u32>, (const u32*)indptr32);
    else go(node2vec_kernel<i64, u32>, (const u32*)indptr32);
  } else {
    if (indices_dtype == GSB_I32) go(node2vec_kernel<int, i64>, (const i64*)indptr);
    else go(node2vec_kernel<i64, i64>, (const i64*)indptr);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
