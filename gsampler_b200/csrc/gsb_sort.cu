// Per-segment sort of the ids of a CSC / CSR (every column's row ids ascending), in place.
//
// The segments of a sampling graph are short (tens of entries) with a few hubs, so the work is
// split by length instead of running one general segmented sort over everything:
//   short  (<= 256 entries): one WARP per segment -- the entries go to the warp's slice of shared
//          memory, a bitonic network runs there with warp-level barriers only, and the sorted run
//          is written back coalesced;
//   medium (<= 4096)       : one CTA per segment, the same network over the whole CTA;
//   long                   : one CTA per segment: the value range [min, max] is cut into 256
//          equal intervals, the entries are partitioned by interval into a scratch copy (a stable
//          order is not needed: equal ids are indistinguishable), every interval is then sorted in
//          shared memory and written back; an interval that still exceeds the shared tile (ids
//          crowded into a narrow range) is sorted where it lies by a bitonic network in global
//          memory -- slow, correct, and not met on graphs whose ids are spread.
// The first kernel walks all segments, sorts the short ones and appends the others to two work
// lists, so no CTA of the later kernels sits idle on segments it does not own.
#include "gsb_common.cuh"

namespace gsb {

constexpr int SORT_THREADS = 256;           // 8 warps
constexpr int SORT_WARP_CAP = 256;          // entries a warp sorts in its shared slice
constexpr int SORT_CTA_CAP = 4096;          // entries a CTA sorts in shared memory
constexpr int SORT_CTA_THREADS = 512;
constexpr int SORT_PARTS = 256;             // intervals of the long-segment partition

template <typename T>
struct SortLimits;
template <>
struct SortLimits<int> { static __device__ __forceinline__ int max() { return 0x7FFFFFFF; } };
template <>
struct SortLimits<i64> { static __device__ __forceinline__ i64 max() { return 0x7FFFFFFFFFFFFFFFll; } };

struct SortParams {
  const i64* indptr;
  void* indices;
  i64 nseg;
  i64* mid_list;   // [nseg] segments for the CTA kernel
  i64* long_list;  // [nseg] segments for the partition kernel
  int* list_n;     // {mid count, long count}
  void* scratch;   // one entry per entry of the graph (long segments only)
  int* err;
};

// Sorting network over a[0..n) for ANY n, run by `nthreads` threads with ids `tid`; `sync`
// separates the stages (a warp- or CTA-level barrier).  It is the bitonic network over the next
// power of two P written with ascending comparators only (the first stage of every merge pairs
// position x with its mirror image inside the block, the others pair x with x + j): positions
// >= n behave as +infinity, which an ascending comparator never moves, so a comparator whose
// upper end lies beyond n is simply skipped and no padding is stored anywhere.
template <typename T, typename Sync>
__device__ __forceinline__ void bitonic_any(T* a, u32 n, u32 tid, u32 nthreads, Sync sync) {
  u32 P = 2;
  while (P < n) P <<= 1;
  u32 lh = 0;  // log2 of half the merge width
  for (u32 k = 2; k <= P; k <<= 1, ++lh) {
    const u32 h = k >> 1;
    for (u32 t = tid; t < (P >> 1); t += nthreads) {
      const u32 blk = t >> lh, off = t & (h - 1);
      const u32 i = (blk << (lh + 1)) + off, q = (blk << (lh + 1)) + (k - 1 - off);
      if (q < n) {
        const T x = a[i], y = a[q];
        if (x > y) { a[i] = y; a[q] = x; }
      }
    }
    sync();
    for (u32 j = h >> 1; j > 0; j >>= 1) {
      for (u32 t = tid; t < (P >> 1); t += nthreads) {
        const u32 i = ((t & ~(j - 1)) << 1) | (t & (j - 1)), q = i | j;
        if (q < n) {
          const T x = a[i], y = a[q];
          if (x > y) { a[i] = y; a[q] = x; }
        }
      }
      sync();
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(SORT_THREADS) sort_short_kernel(const SortParams p) {
  __shared__ T s_all[(SORT_THREADS / 32) * SORT_WARP_CAP];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  T* s = s_all + wid * SORT_WARP_CAP;
  T* ids = reinterpret_cast<T*>(p.indices);
  const i64 warp0 = (i64)blockIdx.x * (SORT_THREADS / 32) + wid;
  const i64 nwarps = (i64)gridDim.x * (SORT_THREADS / 32);
  auto sync = [] { __syncwarp(); };
  // 32 consecutive segments per warp and step: their bounds come from one coalesced load
  for (i64 seg0 = warp0 * 32; seg0 < p.nseg; seg0 += nwarps * 32) {
    const i64 mine = seg0 + lane;
    i64 lo = 0, hi = 0;
    if (mine < p.nseg) { lo = __ldg(p.indptr + mine); hi = __ldg(p.indptr + mine + 1); }
    if (hi < lo) { raise(p.err, ERRBIT_BAD_INPUT); hi = lo; }
    const i64 len = hi - lo;
    if (len > SORT_WARP_CAP) {
      if (len <= SORT_CTA_CAP) p.mid_list[atomicAdd(p.list_n, 1)] = mine;
      else p.long_list[atomicAdd(p.list_n + 1, 1)] = mine;
    }
    const unsigned todo = __ballot_sync(0xffffffffu, len > 1 && len <= SORT_WARP_CAP);
    for (unsigned m = todo; m; m &= m - 1) {
      const int src = __ffs(m) - 1;
      const i64 b = __shfl_sync(0xffffffffu, lo, src);
      const int n = (int)__shfl_sync(0xffffffffu, len, src);
      for (int i = lane; i < n; i += 32) s[i] = ids[b + i];
      __syncwarp();
      bitonic_any(s, (u32)n, (u32)lane, 32u, sync);
      for (int i = lane; i < n; i += 32) ids[b + i] = s[i];
      __syncwarp();
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(SORT_CTA_THREADS) sort_mid_kernel(const SortParams p) {
  __shared__ T s[SORT_CTA_CAP];
  T* ids = reinterpret_cast<T*>(p.indices);
  const int count = p.list_n[0];
  auto sync = [] { __syncthreads(); };
  for (int w = blockIdx.x; w < count; w += gridDim.x) {
    const i64 seg = p.mid_list[w];
    const i64 b = p.indptr[seg];
    const int n = (int)(p.indptr[seg + 1] - b);
    for (int i = threadIdx.x; i < n; i += SORT_CTA_THREADS) s[i] = ids[b + i];
    __syncthreads();
    bitonic_any(s, (u32)n, threadIdx.x, (u32)SORT_CTA_THREADS, sync);
    for (int i = threadIdx.x; i < n; i += SORT_CTA_THREADS) ids[b + i] = s[i];
    __syncthreads();
  }
}

// interval of value v in [vmin, vmax] cut into SORT_PARTS equal parts
template <typename T>
__device__ __forceinline__ int part_of(T v, T vmin, u64 width) {
  return (int)(((u64)((i64)v - (i64)vmin)) / width);
}

template <typename T>
__global__ void __launch_bounds__(SORT_CTA_THREADS) sort_long_kernel(const SortParams p) {
  __shared__ T s[SORT_CTA_CAP];
  __shared__ u32 s_cnt[SORT_PARTS + 1];
  __shared__ u32 s_fill[SORT_PARTS];
  __shared__ T s_min, s_max;
  __shared__ T s_red[2 * (SORT_CTA_THREADS / 32)];
  T* ids = reinterpret_cast<T*>(p.indices);
  T* tmp = reinterpret_cast<T*>(p.scratch);
  const int count = p.list_n[1];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  auto sync = [] { __syncthreads(); };
  for (int w = blockIdx.x; w < count; w += gridDim.x) {
    const i64 seg = p.long_list[w];
    const i64 b = p.indptr[seg];
    const i64 n = p.indptr[seg + 1] - b;
    // value range
    T vmin = SortLimits<T>::max(), vmax = -SortLimits<T>::max() - 1;
    for (i64 i = threadIdx.x; i < n; i += SORT_CTA_THREADS) {
      const T v = ids[b + i];
      vmin = v < vmin ? v : vmin;
      vmax = v > vmax ? v : vmax;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const T a = __shfl_xor_sync(0xffffffffu, vmin, d), c = __shfl_xor_sync(0xffffffffu, vmax, d);
      vmin = a < vmin ? a : vmin;
      vmax = c > vmax ? c : vmax;
    }
    if (lane == 0) { s_red[wid] = vmin; s_red[SORT_CTA_THREADS / 32 + wid] = vmax; }
    for (int k = threadIdx.x; k <= SORT_PARTS; k += SORT_CTA_THREADS) s_cnt[k] = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
      T a = s_red[0], c = s_red[SORT_CTA_THREADS / 32];
      for (int k = 1; k < SORT_CTA_THREADS / 32; ++k) {
        a = s_red[k] < a ? s_red[k] : a;
        c = s_red[SORT_CTA_THREADS / 32 + k] > c ? s_red[SORT_CTA_THREADS / 32 + k] : c;
      }
      s_min = a; s_max = c;
    }
    __syncthreads();
    vmin = s_min; vmax = s_max;
    const u64 width = ((u64)((i64)vmax - (i64)vmin)) / SORT_PARTS + 1;   // part_of(vmax) <= SORT_PARTS - 1
    // histogram, exclusive scan, partition into the scratch copy
    for (i64 i = threadIdx.x; i < n; i += SORT_CTA_THREADS) atomicAdd(&s_cnt[part_of(ids[b + i], vmin, width)], 1u);
    __syncthreads();
    if (wid == 0) {
      u32 carry = 0;
      for (int k0 = 0; k0 < SORT_PARTS; k0 += 32) {
        const u32 c = s_cnt[k0 + lane];
        u32 inc = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const u32 t = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += t;
        }
        s_cnt[k0 + lane] = carry + inc - c;
        s_fill[k0 + lane] = carry + inc - c;
        carry += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) s_cnt[SORT_PARTS] = carry;
    }
    __syncthreads();
    for (i64 i = threadIdx.x; i < n; i += SORT_CTA_THREADS) {
      const T v = ids[b + i];
      tmp[b + atomicAdd(&s_fill[part_of(v, vmin, width)], 1u)] = v;
    }
    __syncthreads();
    // every interval: sort and write back to its place in the segment
    for (int k = 0; k < SORT_PARTS; ++k) {
      const u32 o = s_cnt[k], m = s_cnt[k + 1] - o;
      if (m == 0) continue;  // uniform over the CTA
      if (m <= (u32)SORT_CTA_CAP) {
        for (u32 i = threadIdx.x; i < m; i += SORT_CTA_THREADS) s[i] = tmp[b + o + i];
        __syncthreads();
        if (m > 1) bitonic_any(s, m, threadIdx.x, (u32)SORT_CTA_THREADS, sync);
        for (u32 i = threadIdx.x; i < m; i += SORT_CTA_THREADS) ids[b + o + i] = s[i];
        __syncthreads();
      } else {
        // crowded interval (ids packed into a narrow range): the same network where the entries
        // lie, in global memory
        T* g = tmp + b + o;
        bitonic_any(g, m, threadIdx.x, (u32)SORT_CTA_THREADS, sync);
        for (u32 i = threadIdx.x; i < m; i += SORT_CTA_THREADS) ids[b + o + i] = g[i];
        __syncthreads();
      }
    }
  }
}

struct SortLayout {
  size_t lists, counters, scratch, total;
};

static SortLayout sort_layout(i64 nseg, i64 nnz, int elem) {
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  SortLayout L;
  size_t o = 0;
  L.counters = o; o = up(o + 256);
  L.lists = o; o = up(o + sizeof(i64) * 2 * (size_t)(nseg + 1));
  L.scratch = o; o = up(o + (size_t)elem * (size_t)(nnz + 1));
  L.total = o;
  return L;
}

template <typename T>
static int sort_launch(const SortParams& p, cudaStream_t st) {
  const i64 warps_needed = (p.nseg + 31) / 32;
  i64 g = (warps_needed + SORT_THREADS / 32 - 1) / (SORT_THREADS / 32);
  if (g > sm_count() * 32) g = sm_count() * 32;
  if (g < 1) g = 1;
  { LaunchScope ls(KID_SORT, st); sort_short_kernel<T><<<(int)g, SORT_THREADS, 0, st>>>(p); }
  { LaunchScope ls(KID_SORT, st); sort_mid_kernel<T><<<sm_count() * 4, SORT_CTA_THREADS, 0, st>>>(p); }
  { LaunchScope ls(KID_SORT, st); sort_long_kernel<T><<<sm_count() * 2, SORT_CTA_THREADS, 0, st>>>(p); }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_sort_segments_workspace_bytes(int64_t nseg, int64_t nnz, int indices_dtype) {
  if (nseg < 0 || nnz < 0) return 0;
  return sort_layout(nseg, nnz, indices_dtype == GSB_I32 ? 4 : 8).total;
}

extern "C" int gsb_sort_segments(const int64_t* indptr, void* indices, int indices_dtype, int64_t nseg,
                                 int64_t nnz, void* workspace, size_t workspace_bytes, int* d_err,
                                 void* cuda_stream) {
  if (nseg == 0 || nnz == 0) return GSB_OK;
  if (!indptr || !indices || nseg < 0 || nnz < 0) return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  const SortLayout L = sort_layout(nseg, nnz, indices_dtype == GSB_I32 ? 4 : 8);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  GSB_CUDA_OK(cudaMemsetAsync(ws + L.counters, 0, 256, st));
  SortParams p;
  p.indptr = (const i64*)indptr; p.indices = indices; p.nseg = nseg;
  p.list_n = (int*)(ws + L.counters);
  p.mid_list = (i64*)(ws + L.lists); p.long_list = p.mid_list + (nseg + 1);
  p.scratch = ws + L.scratch; p.err = d_err;
  return indices_dtype == GSB_I32 ? sort_launch<int>(p, st) : sort_launch<i64>(p, st);
}
