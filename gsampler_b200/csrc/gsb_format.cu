// Unsorted COO -> CSC / CSR: group the entries by key (column for a CSC, row for a CSR), keeping
// the entries of a key in their original order, and report where every entry came from.
//
// The reference sorts (key, position) pairs with a device-wide radix sort
// (src/cuda/format_transform.cu:66-86, 108-142).  Here the keys are node ids of a graph, i.e. a
// dense range, so the grouping is a counting sort:
//   histogram : entries per key (one L2 reduction per entry)
//   scan      : offsets = exclusive running sum (tiles of 4096 keys, chained prefix)
//   scatter   : every entry takes the next free place of its key's segment (one L2 atomic) and
//               leaves `position:32 | value:32` there -- in whatever order the atomics land
//   sort      : every segment sorted by the packed word, i.e. by original position: the per-segment
//               sort of gsb_sort.cu (segments are columns: tens of entries, a warp each)
//   unpack    : values and positions apart
// which makes the result the stable grouping, bit for bit what a stable sort by key gives.
// Limits (checked): fewer than 2^31 entries, values in [0, 2^32).
#include "gsb_common.cuh"

namespace gsb {

constexpr int FM_THREADS = 256;
constexpr int SC_THREADS = 1024;
constexpr int SC_ITEMS = 4;
constexpr int SC_TILE = SC_THREADS * SC_ITEMS;

__global__ void __launch_bounds__(FM_THREADS) group_hist_kernel(const i64* __restrict__ keys, i64 nnz, i64 nkeys,
                                                               unsigned long long* __restrict__ count, int* err) {
  for (i64 e = (i64)blockIdx.x * FM_THREADS + threadIdx.x; e < nnz; e += (i64)gridDim.x * FM_THREADS) {
    const i64 k = __ldg(keys + e);
    if ((u64)k < (u64)nkeys) atomicAdd(count + k, 1ull);
    else raise(err, ERRBIT_BAD_INPUT);  // not a segment: the entry is left out
  }
}

// out[i] = sum of in[0 .. i), i in [0, n]; in and out may be the same array
__global__ void __launch_bounds__(SC_THREADS) scan_i64_kernel(const i64* in, i64 n, i64* out, u64* status,
                                                             int* ticket, int* err) {
  __shared__ i64 s_scan[34];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  const i64 n_tiles = (n + SC_TILE) / SC_TILE;  // covers index n as well
  if (tile >= n_tiles) return;
  const i64 i0 = (i64)tile * SC_TILE + (i64)threadIdx.x * SC_ITEMS;
  i64 v[SC_ITEMS], sum = 0;
#pragma unroll
  for (int j = 0; j < SC_ITEMS; ++j) {
    v[j] = i0 + j < n ? in[i0 + j] : 0;
    sum += v[j];
  }
  i64 total;
  const i64 ex = block_exclusive_scan(sum, s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 base = chained_exclusive_prefix(status, tile, total, err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  i64 run = s_base + ex;
#pragma unroll
  for (int j = 0; j < SC_ITEMS; ++j) {
    if (i0 + j <= n) out[i0 + j] = run;
    run += v[j];
  }
}

__global__ void __launch_bounds__(FM_THREADS) group_scatter_kernel(const i64* __restrict__ keys,
                                                                  const i64* __restrict__ vals, i64 nnz, i64 nkeys,
                                                                  unsigned long long* __restrict__ cursor,
                                                                  u64* __restrict__ packed, int* err) {
  for (i64 e = (i64)blockIdx.x * FM_THREADS + threadIdx.x; e < nnz; e += (i64)gridDim.x * FM_THREADS) {
    const i64 k = __ldg(keys + e);
    if ((u64)k >= (u64)nkeys) continue;  // reported by the histogram pass
    i64 v = __ldg(vals + e);
    if ((u64)v > 0xFFFFFFFFull) { raise(err, ERRBIT_BAD_INPUT); v = 0xFFFFFFFFll; }
    const unsigned long long at = atomicAdd(cursor + k, 1ull);
    packed[at] = ((u64)e << 32) | (u64)v;
  }
}

__global__ void __launch_bounds__(FM_THREADS) group_unpack_kernel(const u64* __restrict__ packed, i64 n,
                                                                 i64* __restrict__ vals, i64* __restrict__ pos) {
  for (i64 i = (i64)blockIdx.x * FM_THREADS + threadIdx.x; i < n; i += (i64)gridDim.x * FM_THREADS) {
    const u64 w = packed[i];
    vals[i] = (i64)(w & 0xFFFFFFFFull);
    pos[i] = (i64)(w >> 32);
  }
}

// ---------------------------------------------------------------- compaction of an id axis
// Sorted unique of node ids + the map id -> position in it (Graph::Compact, the encoding of batch
// column slicing).  The ids lie below a known bound (rows / columns of the graph, times the
// number of minibatches for encoded ids), so "sorted unique" is a presence table over that
// range: one BIT per possible id, a running sum of the set bits per 32-bit word, and
// rank(v) = prefix[v / 32] + popc(bits[v / 32] below bit v % 32).  3/8 of a byte per possible id.
// The reference sorts (src/cuda/compact.cu:10-30, torch::_unique2).
template <typename IndexT>
__global__ void __launch_bounds__(FM_THREADS) compact_mark_kernel(const IndexT* __restrict__ ids, i64 n, i64 bound,
                                                                 u32* __restrict__ bits, int* err) {
  for (i64 i = (i64)blockIdx.x * FM_THREADS + threadIdx.x; i < n; i += (i64)gridDim.x * FM_THREADS) {
    const i64 v = (i64)ids[i];
    if ((u64)v < (u64)bound) {
      const u32 bit = 1u << (v & 31);
      if (!(bits[v >> 5] & bit)) atomicOr(bits + (v >> 5), bit);  // most ids repeat: skip the atomic then
    } else {
      raise(err, ERRBIT_BAD_INPUT);
    }
  }
}

__global__ void __launch_bounds__(FM_THREADS) compact_popc_kernel(const u32* __restrict__ bits, i64 words,
                                                                 i64* __restrict__ count) {
  for (i64 w = (i64)blockIdx.x * FM_THREADS + threadIdx.x; w < words; w += (i64)gridDim.x * FM_THREADS)
    count[w] = __popc(bits[w]);
}

__device__ __forceinline__ i64 compact_rank_of(const u32* __restrict__ bits, const i64* __restrict__ prefix, i64 v) {
  return __ldg(prefix + (v >> 5)) + __popc(__ldg(bits + (v >> 5)) & ((1u << (v & 31)) - 1u));
}

// the distinct ids in ascending order: every set bit writes its id at its rank
__global__ void __launch_bounds__(FM_THREADS) compact_unique_kernel(const u32* __restrict__ bits,
                                                                   const i64* __restrict__ prefix, i64 words,
                                                                   i64* __restrict__ unique) {
  for (i64 w = (i64)blockIdx.x * FM_THREADS + threadIdx.x; w < words; w += (i64)gridDim.x * FM_THREADS) {
    u32 b = bits[w];
    i64 r = prefix[w];
    while (b) {
      const int k = __ffs(b) - 1;
      unique[r++] = (w << 5) + k;
      b &= b - 1;
    }
  }
}

template <typename IndexT>
__global__ void __launch_bounds__(FM_THREADS) compact_map_kernel(const IndexT* __restrict__ ids, i64 n, i64 bound,
                                                                const u32* __restrict__ bits,
                                                                const i64* __restrict__ prefix, i64* __restrict__ out) {
  for (i64 i = (i64)blockIdx.x * FM_THREADS + threadIdx.x; i < n; i += (i64)gridDim.x * FM_THREADS) {
    const i64 v = (i64)ids[i];
    out[i] = (u64)v < (u64)bound ? compact_rank_of(bits, prefix, v) : -1;
  }
}

struct CompactLayout {
  size_t status, bits, prefix, total;
  i64 words, scan_tiles;
};

static CompactLayout compact_layout(i64 bound) {
  CompactLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.words = (bound + 31) / 32;
  L.scan_tiles = (L.words + SC_TILE) / SC_TILE;
  size_t o = 0;
  L.status = o; o = up(o + 256 + sizeof(u64) * (size_t)(L.scan_tiles + 1));
  L.bits = o; o = up(o + sizeof(u32) * (size_t)(L.words + 1));
  L.prefix = o; o = up(o + sizeof(i64) * (size_t)(L.words + 1));
  L.total = o;
  return L;
}

// ---------------------------------------------------------------- position lookup (IndexSearch)
// out[j] = the smallest i with data[i] == keys[j], or -1.  An open-addressing table in global
// memory, twice as many slots as entries (a power of two): slot key claimed by compare-and-swap,
// slot value lowered by atomicMin, so that the result does not depend on the order of execution
// (the reference's table keeps whichever duplicate wrote last, src/cuda/index_search.cu:46-57).
// -1 is the empty key, as in the reference: it cannot be looked up.  Every probe loop ends after
// `slots` probes.
constexpr i64 IS_EMPTY = -1;
__device__ __forceinline__ u64 mix64(u64 k) {
  k ^= k >> 30; k *= 0xBF58476D1CE4E5B9ull; k ^= k >> 27; k *= 0x94D049BB133111EBull; k ^= k >> 31;
  return k;
}

__global__ void __launch_bounds__(FM_THREADS) index_insert_kernel(const i64* __restrict__ data, i64 n,
                                                                 long long* tab_k, long long* tab_v, u64 slots,
                                                                 int* err) {
  const u64 mask = slots - 1;
  for (i64 i = (i64)blockIdx.x * FM_THREADS + threadIdx.x; i < n; i += (i64)gridDim.x * FM_THREADS) {
    const i64 key = __ldg(data + i);
    if (key == IS_EMPTY) { raise(err, ERRBIT_BAD_INPUT); continue; }
    u64 pos = mix64((u64)key) & mask;
    u64 probes = 0;
    for (; probes < slots; ++probes) {
      long long cur = tab_k[pos];
      if (cur == IS_EMPTY) cur = (long long)atomicCAS((unsigned long long*)(tab_k + pos), (unsigned long long)IS_EMPTY,
                                                      (unsigned long long)key);
      if (cur == IS_EMPTY || cur == key) { atomicMin(tab_v + pos, (long long)i); break; }
      pos = (pos + 1) & mask;
    }
    if (probes == slots) raise(err, ERRBIT_TABLE_FULL);
  }
}

__global__ void __launch_bounds__(FM_THREADS) index_query_kernel(const i64* __restrict__ keys, i64 m,
                                                                const long long* __restrict__ tab_k,
                                                                const long long* __restrict__ tab_v, u64 slots,
                                                                i64* __restrict__ out) {
  const u64 mask = slots - 1;
  for (i64 j = (i64)blockIdx.x * FM_THREADS + threadIdx.x; j < m; j += (i64)gridDim.x * FM_THREADS) {
    const i64 key = __ldg(keys + j);
    i64 found = -1;
    if (key != IS_EMPTY) {
      u64 pos = mix64((u64)key) & mask;
      for (u64 probes = 0; probes < slots; ++probes) {
        const long long cur = tab_k[pos];
        if (cur == key) { found = tab_v[pos]; break; }
        if (cur == IS_EMPTY) break;
        pos = (pos + 1) & mask;
      }
    }
    out[j] = found;
  }
}

static u64 index_slots(i64 n) {
  u64 s = 64;
  while (s < 2 * (u64)n) s <<= 1;
  return s;
}

struct GroupLayout {
  size_t status, cursor, packed, sort, total;
  i64 scan_tiles;
};

static GroupLayout group_layout(i64 nnz, i64 nkeys) {
  GroupLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.scan_tiles = (nkeys + SC_TILE) / SC_TILE;
  size_t o = 0;
  L.status = o; o = up(o + 256 + sizeof(u64) * (size_t)(L.scan_tiles + 1));  // ticket, then status words
  L.cursor = o; o = up(o + sizeof(i64) * (size_t)(nkeys + 1));
  L.packed = o; o = up(o + sizeof(u64) * (size_t)(nnz + 1));
  L.sort = o; o = up(o + gsb_sort_segments_workspace_bytes(nkeys, nnz, GSB_I64));
  L.total = o;
  return L;
}

static int wide_grid_fm(i64 n) {
  i64 g = (n + FM_THREADS - 1) / FM_THREADS;
  const i64 cap = (i64)sm_count() * 16;
  if (g > cap) g = cap;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_group_by_key_workspace_bytes(int64_t nnz, int64_t nkeys) {
  if (nnz < 0 || nkeys < 0) return 0;
  return group_layout(nnz, nkeys).total;
}

extern "C" int gsb_group_by_key(const int64_t* keys, const int64_t* vals, int64_t nnz, int64_t nkeys,
                                int64_t* indptr, int64_t* out_vals, int64_t* out_pos, void* workspace,
                                size_t workspace_bytes, int* d_err, void* cuda_stream) {
  if (nnz < 0 || nkeys < 0 || !indptr || (nnz > 0 && (!keys || !vals || !out_vals || !out_pos)))
    return GSB_ERR_INVALID;
  if (nnz >= (1ll << 31) || nkeys >= (1ll << 40)) return GSB_ERR_UNSUPPORTED;
  const GroupLayout L = group_layout(nnz, nkeys);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  int* ticket = (int*)(ws + L.status);
  u64* status = (u64*)(ws + L.status + 256);
  i64* cursor = (i64*)(ws + L.cursor);
  u64* packed = (u64*)(ws + L.packed);
  GSB_CUDA_OK(cudaMemsetAsync(ws + L.status, 0, L.cursor - L.status, st));
  GSB_CUDA_OK(cudaMemsetAsync(indptr, 0, sizeof(i64) * (size_t)(nkeys + 1), st));
  LaunchScope ls(KID_INDPTR_SORTED, st);
  if (nnz > 0)
    group_hist_kernel<<<wide_grid_fm(nnz), FM_THREADS, 0, st>>>((const i64*)keys, nnz, nkeys,
                                                                 (unsigned long long*)indptr, d_err);
  scan_i64_kernel<<<(int)L.scan_tiles, SC_THREADS, 0, st>>>((const i64*)indptr, nkeys, (i64*)indptr, status,
                                                            ticket, d_err);
  if (nnz > 0) {
    GSB_CUDA_OK(cudaMemcpyAsync(cursor, indptr, sizeof(i64) * (size_t)(nkeys + 1), cudaMemcpyDeviceToDevice, st));
    group_scatter_kernel<<<wide_grid_fm(nnz), FM_THREADS, 0, st>>>((const i64*)keys, (const i64*)vals, nnz, nkeys,
                                                                    (unsigned long long*)cursor, packed, d_err);
    // entries with a key that is no segment were left out: the segments cover indptr[nkeys] <= nnz entries
    const int rc = gsb_sort_segments(indptr, packed, GSB_I64, nkeys, nnz, ws + L.sort, workspace_bytes - L.sort,
                                     d_err, cuda_stream);
    if (rc != GSB_OK) return rc;
    group_unpack_kernel<<<wide_grid_fm(nnz), FM_THREADS, 0, st>>>(packed, nnz, (i64*)out_vals, (i64*)out_pos);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" size_t gsb_compact_workspace_bytes(int64_t bound) {
  if (bound < 0) return 0;
  return compact_layout(bound).total;
}

extern "C" int gsb_compact_rank(const void* ids, int ids_dtype, int64_t n, int64_t bound, void* workspace,
                                size_t workspace_bytes, int64_t* d_count, int* d_err, void* cuda_stream) {
  if (n < 0 || bound < 0 || (n > 0 && !ids)) return GSB_ERR_INVALID;
  if (ids_dtype != GSB_I32 && ids_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (bound >= (1ll << 44)) return GSB_ERR_UNSUPPORTED;
  const CompactLayout L = compact_layout(bound);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  u32* bits = (u32*)(ws + L.bits);
  i64* prefix = (i64*)(ws + L.prefix);
  GSB_CUDA_OK(cudaMemsetAsync(ws, 0, L.prefix, st));  // ticket, status words, presence bits
  LaunchScope ls(KID_MISC, st);
  if (n > 0) {
    if (ids_dtype == GSB_I32)
      compact_mark_kernel<int><<<wide_grid_fm(n), FM_THREADS, 0, st>>>((const int*)ids, n, bound, bits, d_err);
    else
      compact_mark_kernel<i64><<<wide_grid_fm(n), FM_THREADS, 0, st>>>((const i64*)ids, n, bound, bits, d_err);
  }
  compact_popc_kernel<<<wide_grid_fm(L.words + 1), FM_THREADS, 0, st>>>(bits, L.words, prefix);
  scan_i64_kernel<<<(int)L.scan_tiles, SC_THREADS, 0, st>>>(prefix, L.words, prefix, (u64*)(ws + L.status + 256),
                                                            (int*)(ws + L.status), d_err);
  if (d_count)
    GSB_CUDA_OK(cudaMemcpyAsync(d_count, prefix + L.words, sizeof(i64), cudaMemcpyDeviceToDevice, st));
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_compact_apply(const void* workspace, int64_t bound, int64_t* unique, const void* ids,
                                 int ids_dtype, int64_t n, int64_t* out, void* cuda_stream) {
  if (!workspace || bound < 0 || n < 0 || (n > 0 && (!ids || !out))) return GSB_ERR_INVALID;
  if (n > 0 && ids_dtype != GSB_I32 && ids_dtype != GSB_I64) return GSB_ERR_INVALID;
  const CompactLayout L = compact_layout(bound);
  const u32* bits = (const u32*)((const char*)workspace + L.bits);
  const i64* prefix = (const i64*)((const char*)workspace + L.prefix);
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_MISC, st);
  if (unique && L.words > 0)
    compact_unique_kernel<<<wide_grid_fm(L.words), FM_THREADS, 0, st>>>(bits, prefix, L.words, (i64*)unique);
  if (n > 0) {
    if (ids_dtype == GSB_I32)
      compact_map_kernel<int><<<wide_grid_fm(n), FM_THREADS, 0, st>>>((const int*)ids, n, bound, bits, prefix, (i64*)out);
    else
      compact_map_kernel<i64><<<wide_grid_fm(n), FM_THREADS, 0, st>>>((const i64*)ids, n, bound, bits, prefix, (i64*)out);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" size_t gsb_index_search_workspace_bytes(int64_t n) {
  if (n < 0) return 0;
  return (size_t)index_slots(n) * 16;
}

extern "C" int gsb_index_search(const int64_t* data, int64_t n, const int64_t* keys, int64_t m, int64_t* out,
                                void* workspace, size_t workspace_bytes, int* d_err, void* cuda_stream) {
  if (n < 0 || m < 0 || (n > 0 && !data) || (m > 0 && (!keys || !out))) return GSB_ERR_INVALID;
  if (n >= (1ll << 40)) return GSB_ERR_UNSUPPORTED;
  const u64 slots = index_slots(n);
  if (!workspace || workspace_bytes < slots * 16) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  long long* tab_k = (long long*)workspace;
  long long* tab_v = tab_k + slots;
  GSB_CUDA_OK(cudaMemsetAsync(tab_k, 0xFF, slots * 8, st));  // every key -1 = empty
  GSB_CUDA_OK(cudaMemsetAsync(tab_v, 0x7F, slots * 8, st));  // every value above any position
  LaunchScope ls(KID_MISC, st);
  if (n > 0)
    index_insert_kernel<<<wide_grid_fm(n), FM_THREADS, 0, st>>>((const i64*)data, n, tab_k, tab_v, slots, d_err);
  if (m > 0)
    index_query_kernel<<<wide_grid_fm(m), FM_THREADS, 0, st>>>((const i64*)keys, m, tab_k, tab_v, slots, (i64*)out);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
