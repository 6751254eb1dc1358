// Column slicing A[:, seeds] (all edges of the chosen columns) and small
// gather utilities.
//
// count: thread per seed, degree -> block scan -> chained tile prefix, so the
//        offsets come out of one pass.
// fill : thread per OUTPUT edge; the owning column is found by a binary search
//        in the (L2-resident) offset array, which keeps loads and stores
//        coalesced however skewed the degrees are.
#include "gsb_common.cuh"

namespace gsb {

constexpr int SLICE_THREADS = 256;

// Pick count of one column: K == 0 -> the whole column; otherwise min(deg, K)
// without replacement, K (0 for an empty column) with replacement.
__global__ void __launch_bounds__(SLICE_THREADS)
count_kernel(const i64* __restrict__ indptr, i64 num_cols, const i64* __restrict__ seeds, i64 S_max,
             const i64* __restrict__ d_S, i64 K, int replace, i64* __restrict__ sub_indptr,
             i64* __restrict__ d_total, u64* status, int* ticket, int* err, const CountExtra x) {
  __shared__ i64 s_scan[34];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  i64 S = S_max;
  if (d_S) { i64 live = *d_S; S = live < S ? (live < 0 ? 0 : live) : S; }
  const i64 tiles = S == 0 ? 1 : (S + SLICE_THREADS - 1) / SLICE_THREADS;
  if (tile >= tiles) return;
  const i64 slot = (i64)tile * SLICE_THREADS + threadIdx.x;
  i64 cnt = 0;
  bool listed = false;
  if (slot < S) {
    const i64 c = seeds ? seeds[slot] : slot;
    i64 st = 0, deg = 0;
    if ((u64)c < (u64)num_cols) {
      st = __ldg(indptr + c);
      deg = __ldg(indptr + c + 1) - st;
    }
    if ((u64)c >= (u64)num_cols || deg < 0) {  // bad seed / offsets: reported, counted as empty
      raise(err, ERRBIT_BAD_INPUT);
      deg = 0;
    }
    cnt = K == 0 ? deg : (replace ? (deg == 0 ? 0 : K) : (deg < K ? deg : K));
    if (x.start) { x.start[slot] = st; x.deg[slot] = deg > 0xFFFFFFFFll ? 0xFFFFFFFFu : (u32)deg; }
    listed = x.list && cnt > 0 && deg >= x.list_min_deg;
  }
  if (x.list) {  // columns of at least list_min_deg entries, in no particular order
    const unsigned bal = __ballot_sync(0xffffffffu, listed);
    int base = 0;
    if ((threadIdx.x & 31) == 0 && bal) base = atomicAdd(x.list_n, __popc(bal));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (listed) x.list[base + __popc(bal & ((1u << (threadIdx.x & 31)) - 1u))] = slot;
  }
  i64 total;
  const i64 loff = block_exclusive_scan(cnt, s_scan, &total);
  if (threadIdx.x < 32) {
    i64 base = chained_exclusive_prefix(status, tile, total, err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  if (slot < S) sub_indptr[slot] = s_base + loff;
  if (tile == tiles - 1 && threadIdx.x == 0) {
    sub_indptr[S] = s_base + total;
    if (d_total) *d_total = s_base + total;
  }
}

size_t count_workspace_bytes(i64 S_max) {
  return 256 + (size_t)((S_max + SLICE_THREADS - 1) / SLICE_THREADS + 1) * sizeof(u64);
}

int launch_count(const i64* indptr, i64 num_cols, const i64* seeds, i64 S_max, const i64* d_S, i64 K,
                 int replace, i64* sub_indptr, i64* d_total, void* workspace, int* d_err,
                 cudaStream_t st, const CountExtra& extra) {
  const int tiles = S_max == 0 ? 1 : ceil_div_i(S_max, SLICE_THREADS);
  GSB_CUDA_OK(cudaMemsetAsync(workspace, 0, 256 + (size_t)(tiles + 1) * sizeof(u64), st));
  LaunchScope ls(KID_COUNT, st);
  count_kernel<<<tiles, SLICE_THREADS, 0, st>>>(indptr, num_cols, seeds, S_max, d_S, K, replace, sub_indptr,
                                                d_total, (u64*)((char*)workspace + 256),
                                                (int*)workspace, d_err, extra);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

// largest i in [0, n) with ptr[i] <= x, searched by a whole warp: 32 probes per round, so a
// search over 10^6 offsets is 4 dependent loads instead of 20
__device__ __forceinline__ i64 warp_find_segment(const i64* __restrict__ ptr, i64 n, i64 x) {
  const int lane = threadIdx.x & 31;
  i64 lo = 0, hi = n;  // answer in [lo, hi)
  while (hi - lo > 1) {
    const i64 stride = (hi - lo + 31) / 32;
    const i64 probe = lo + (i64)lane * stride;
    const bool le = probe < hi && __ldg(ptr + probe) <= x;
    const int k = __popc(__ballot_sync(0xffffffffu, le));  // probes are monotone: the first k hold
    const i64 nlo = lo + (i64)(k > 0 ? k - 1 : 0) * stride;
    hi = nlo + stride < hi ? nlo + stride : hi;
    lo = nlo;
  }
  return lo;
}

// CTA per tile of 1024 output entries: two warps locate the tile's first and last column slot,
// every thread then searches only between those for each of its four entries.
constexpr int SF_PER_THREAD = 4;
constexpr int SF_TILE = SLICE_THREADS * SF_PER_THREAD;

template <typename IndexT>
__global__ void __launch_bounds__(SLICE_THREADS)
slice_fill_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices,
                  const i64* __restrict__ seeds, i64 S, const i64* __restrict__ sub_indptr, i64 E,
                  i64* __restrict__ out_rows, i64* __restrict__ out_cols,
                  i64* __restrict__ out_sel, const i64* __restrict__ col_bptr, int B,
                  i64 encoding_size) {
  __shared__ i64 s_lo, s_hi;
  const i64 tiles = (E + SF_TILE - 1) / SF_TILE;
  for (i64 tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const i64 e0 = tile * SF_TILE;
    const i64 e_last = e0 + SF_TILE - 1 < E - 1 ? e0 + SF_TILE - 1 : E - 1;
    __syncthreads();  // the previous tile's readers of s_lo / s_hi
    if (threadIdx.x < 64) {
      const i64 s = warp_find_segment(sub_indptr, S, threadIdx.x < 32 ? e0 : e_last);
      if (threadIdx.x == 0) s_lo = s;
      if (threadIdx.x == 32) s_hi = s;
    }
    __syncthreads();
    // entry e0 + k * 256 + thread: neighbouring lanes read and write neighbouring words
    const i64 t_lo = s_lo, t_hi = s_hi;
#pragma unroll
    for (int k = 0; k < SF_PER_THREAD; ++k) {
      const i64 e = e0 + k * SLICE_THREADS + threadIdx.x;
      if (e >= E) break;
      i64 lo = t_lo, hi = t_hi;  // column slot of e: largest i in [lo, hi] with sub_indptr[i] <= e
      while (lo < hi) {
        const i64 mid = (lo + hi + 1) >> 1;
        if (__ldg(sub_indptr + mid) <= e) lo = mid; else hi = mid - 1;
      }
      const i64 pos = __ldg(indptr + seeds[lo]) + (e - __ldg(sub_indptr + lo));
      i64 row = load_index<IndexT>(indices, pos);
      if (encoding_size > 0 && col_bptr) row += (i64)find_segment(col_bptr, B, lo) * encoding_size;
      out_rows[e] = row;
      out_sel[e] = pos;
      if (out_cols) out_cols[e] = lo;
    }
  }
}

__global__ void gather_i64_kernel(const i64* __restrict__ src, const i64* __restrict__ idx, i64 n,
                                  i64* __restrict__ out) {
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x)
    out[i] = src[idx[i]];
}

// Row gather for node / edge data: out row i = src row idx[i].  A row is cut
// into chunks of VecT; consecutive threads copy consecutive chunks of the same
// row, so both the reads and the writes of a row are contiguous.  `src` may be
// device memory or page-locked host memory (read in place over the bus).
template <typename VecT>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const VecT* __restrict__ src, i64 chunks_per_row, i64 src_rows,
                   const i64* __restrict__ idx, i64 n, VecT* __restrict__ out, int* err) {
  const i64 total = n * chunks_per_row;
  for (i64 g = (i64)blockIdx.x * blockDim.x + threadIdx.x; g < total;
       g += (i64)gridDim.x * blockDim.x) {
    const i64 i = g / chunks_per_row, c = g - i * chunks_per_row;
    const i64 r = __ldg(idx + i);
    if (r < 0 || r >= src_rows) { raise(err, ERRBIT_BAD_INPUT); continue; }
    out[g] = __ldg(src + r * chunks_per_row + c);
  }
}

// out[e] = segment (column) that owns position e of a CSC/CSR offset array
__global__ void expand_indptr_kernel(const i64* __restrict__ indptr, i64 nseg, i64 nnz,
                                     i64* __restrict__ out) {
  for (i64 e = (i64)blockIdx.x * blockDim.x + threadIdx.x; e < nnz;
       e += (i64)gridDim.x * blockDim.x) {
    i64 lo = 0, hi = nseg;
    while (hi - lo > 1) {
      i64 mid = (lo + hi) >> 1;
      if (__ldg(indptr + mid) <= e) lo = mid; else hi = mid;
    }
    out[e] = lo;
  }
}

// indptr[k] = number of keys < k, for k in [0, nkeys]; keys sorted ascending
__global__ void indptr_from_sorted_kernel(const i64* __restrict__ keys, i64 nnz, i64 nkeys,
                                          i64* __restrict__ indptr) {
  for (i64 k = (i64)blockIdx.x * blockDim.x + threadIdx.x; k <= nkeys;
       k += (i64)gridDim.x * blockDim.x) {
    i64 lo = 0, hi = nnz;  // first position with keys[pos] >= k
    while (lo < hi) {
      i64 mid = (lo + hi) >> 1;
      if (__ldg(keys + mid) < k) lo = mid + 1; else hi = mid;
    }
    indptr[k] = lo;
  }
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_expand_indptr(const int64_t* indptr, int64_t nseg, int64_t nnz, int64_t* out,
                                 void* cuda_stream) {
  if (nnz == 0) return GSB_OK;
  if (!indptr || !out || nseg <= 0 || nnz < 0) return GSB_ERR_INVALID;
  i64 blocks = (nnz + 255) / 256;
  if (blocks > sm_count() * 32) blocks = sm_count() * 32;
  LaunchScope ls(KID_EXPAND, (cudaStream_t)cuda_stream);
  expand_indptr_kernel<<<(int)blocks, 256, 0, (cudaStream_t)cuda_stream>>>(
      (const i64*)indptr, nseg, nnz, (i64*)out);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_indptr_from_sorted(const int64_t* keys, int64_t nnz, int64_t nkeys,
                                      int64_t* indptr, void* cuda_stream) {
  if (!indptr || nkeys < 0 || nnz < 0 || (nnz > 0 && !keys)) return GSB_ERR_INVALID;
  i64 blocks = (nkeys + 1 + 255) / 256;
  if (blocks > sm_count() * 32) blocks = sm_count() * 32;
  LaunchScope ls(KID_INDPTR_SORTED, (cudaStream_t)cuda_stream);
  indptr_from_sorted_kernel<<<(int)blocks, 256, 0, (cudaStream_t)cuda_stream>>>(
      (const i64*)keys, nnz, nkeys, (i64*)indptr);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" size_t gsb_slice_cols_workspace_bytes(int64_t S) {
  if (S < 0) return 0;
  return count_workspace_bytes(S);
}

extern "C" int gsb_slice_cols_count(const int64_t* indptr, int64_t num_cols, const int64_t* seeds,
                                    int64_t S, int64_t* sub_indptr, void* workspace,
                                    size_t workspace_bytes, int* d_err, void* cuda_stream) {
  if (!indptr || !sub_indptr || S < 0 || num_cols < 0 || (S > 0 && !seeds)) return GSB_ERR_INVALID;
  if (!workspace || workspace_bytes < gsb_slice_cols_workspace_bytes(S)) return GSB_ERR_WORKSPACE;
  return launch_count((const i64*)indptr, num_cols, (const i64*)seeds, S, nullptr, 0, 0, (i64*)sub_indptr,
                      nullptr, workspace, d_err, (cudaStream_t)cuda_stream);
}

extern "C" int gsb_slice_cols_fill(const int64_t* indptr, const void* indices, int indices_dtype,
                                   const int64_t* seeds, int64_t S, const int64_t* sub_indptr,
                                   int64_t E, int64_t* out_rows, int64_t* out_cols,
                                   int64_t* out_sel, const int64_t* col_bptr, int64_t B,
                                   int64_t encoding_size, void* cuda_stream) {
  if (E == 0) return GSB_OK;
  if (!indptr || !indices || !seeds || !sub_indptr || !out_rows || !out_sel || S <= 0 || E < 0)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  i64 blocks = (E + SF_TILE - 1) / SF_TILE;
  if (blocks > sm_count() * 64) blocks = sm_count() * 64;
  LaunchScope ls(KID_SLICE_FILL, st);
  if (indices_dtype == GSB_I32)
    slice_fill_kernel<int><<<(int)blocks, SLICE_THREADS, 0, st>>>(
        (const i64*)indptr, indices, (const i64*)seeds, S, (const i64*)sub_indptr, E,
        (i64*)out_rows, (i64*)out_cols, (i64*)out_sel, (const i64*)col_bptr, (int)B, encoding_size);
  else
    slice_fill_kernel<i64><<<(int)blocks, SLICE_THREADS, 0, st>>>(
        (const i64*)indptr, indices, (const i64*)seeds, S, (const i64*)sub_indptr, E,
        (i64*)out_rows, (i64*)out_cols, (i64*)out_sel, (const i64*)col_bptr, (int)B, encoding_size);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_gather_i64(const int64_t* src, const int64_t* idx, int64_t n, int64_t* out,
                              void* cuda_stream) {
  if (n == 0) return GSB_OK;
  if (!src || !idx || !out || n < 0) return GSB_ERR_INVALID;
  i64 blocks = (n + 255) / 256;
  if (blocks > sm_count() * 32) blocks = sm_count() * 32;
  LaunchScope ls(KID_GATHER, (cudaStream_t)cuda_stream);
  gather_i64_kernel<<<(int)blocks, 256, 0, (cudaStream_t)cuda_stream>>>(
      (const i64*)src, (const i64*)idx, n, (i64*)out);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

template <typename VecT>
static void launch_gather_rows(const void* src, i64 row_bytes, i64 src_rows, const i64* idx, i64 n,
                               void* out, int* d_err, cudaStream_t st) {
  const i64 cpr = row_bytes / (i64)sizeof(VecT);
  i64 blocks = (n * cpr + 255) / 256;
  if (blocks > sm_count() * 32) blocks = sm_count() * 32;
  gather_rows_kernel<VecT><<<(int)blocks, 256, 0, st>>>((const VecT*)src, cpr, src_rows, idx, n,
                                                        (VecT*)out, d_err);
}

extern "C" int gsb_gather_rows(const void* src, int64_t row_bytes, int64_t src_rows,
                               const int64_t* idx, int64_t n, void* out, int* d_err,
                               void* cuda_stream) {
  if (n == 0 || row_bytes == 0) return GSB_OK;
  if (!src || !idx || !out || n < 0 || row_bytes < 0 || src_rows < 0) return GSB_ERR_INVALID;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  const uintptr_t align = (uintptr_t)src | (uintptr_t)out | (uintptr_t)row_bytes;
  LaunchScope ls(KID_GATHER, st);
  if ((align & 15) == 0) launch_gather_rows<uint4>(src, row_bytes, src_rows, (const i64*)idx, n, out, d_err, st);
  else if ((align & 7) == 0) launch_gather_rows<uint2>(src, row_bytes, src_rows, (const i64*)idx, n, out, d_err, st);
  else if ((align & 3) == 0) launch_gather_rows<u32>(src, row_bytes, src_rows, (const i64*)idx, n, out, d_err, st);
  else if ((align & 1) == 0) launch_gather_rows<unsigned short>(src, row_bytes, src_rows, (const i64*)idx, n, out, d_err, st);
  else launch_gather_rows<unsigned char>(src, row_bytes, src_rows, (const i64*)idx, n, out, d_err, st);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
