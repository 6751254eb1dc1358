// Slicing ACROSS the compressed dimension: keep the entries of a CSC (CSR)
// whose row (column) id belongs to a given set and rename each kept id to its
// position in the set -- A[rows, :] evaluated on a CSC operand -- and the same
// filter on a COO operand.
//
// Membership is a direct-address map (one 32-bit word per possible id, built
// per call in the workspace): no probing, one L2-resident load per entry.
// Both the CSC and the COO form are edge-parallel ordered compactions (tile
// scan + chained tile prefix), so the output keeps the operand's entry order
// and the cost does not depend on how the entries are spread over segments.
#include "gsb_common.cuh"

namespace gsb {

constexpr int RS_THREADS = 256;
constexpr int RS_WARPS = RS_THREADS / 32;
constexpr u32 MAP_ABSENT = 0xFFFFFFFFu;

__global__ void map_fill_kernel(u32* map, i64 n) {
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x)
    map[i] = MAP_ABSENT;
}

// map[id] = smallest position of id in ids[0..R)
__global__ void map_build_kernel(const i64* __restrict__ ids, i64 R, u32* map, i64 id_bound,
                                 int* err) {
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < R; i += (i64)gridDim.x * blockDim.x) {
    const i64 id = ids[i];
    if (id < 0 || id >= id_bound) { raise(err, ERRBIT_BAD_INPUT); continue; }
    atomicMin(map + id, (u32)i);
  }
}

// Slicing across a CSC (CSR) is EDGE-parallel: a CTA takes a tile of 1024 consecutive
// entries (four per thread), whatever segments they belong to, so a few very long segments
// cost the same as many short ones.  Entries are already in segment order, hence an ordered
// compaction over all entries (tile scan + chained tile prefix) IS the segment-major output,
// and the output offset of a segment is the number of kept entries before its first entry.
// Pass 1 (FILL = false) writes those offsets, pass 2 the kept entries.
constexpr int AC_PER_THREAD = 4;
constexpr int AC_TILE = RS_THREADS * AC_PER_THREAD;

// largest s in [lo, hi] with indptr[s] <= e
__device__ __forceinline__ i64 segment_in_range(const i64* __restrict__ indptr, i64 lo, i64 hi, i64 e) {
  while (lo < hi) {
    const i64 mid = (lo + hi + 1) >> 1;
    if (__ldg(indptr + mid) <= e) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename IndexT, bool FILL>
__global__ void __launch_bounds__(RS_THREADS)
across_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 nseg, i64 nnz_max,
              const u32* __restrict__ map, i64 id_bound, i64* __restrict__ out_indptr,
              i64* __restrict__ out_ids, i64* __restrict__ out_seg, i64* __restrict__ out_sel,
              u64* status, int* ticket, int* err) {
  __shared__ i64 s_scan[34];
  __shared__ int s_tile;
  __shared__ i64 s_base, s_lo, s_hi;
  if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  i64 nnz = nseg > 0 ? indptr[nseg] : 0;
  if (nnz > nnz_max || nnz < 0) {
    if (tile == 0 && threadIdx.x == 0) raise(err, ERRBIT_CAPACITY);
    nnz = 0;
  }
  const i64 tiles = nnz == 0 ? 1 : (nnz + AC_TILE - 1) / AC_TILE;
  if (tile >= tiles) return;
  const i64 e0 = (i64)tile * AC_TILE;
  const i64 e_last = e0 + AC_TILE - 1 < nnz - 1 ? e0 + AC_TILE - 1 : nnz - 1;
  if (threadIdx.x < 2 && nnz > 0) {
    const i64 s = find_segment(indptr, (int)nseg, threadIdx.x == 0 ? e0 : e_last);
    if (threadIdx.x == 0) s_lo = s; else s_hi = s;
  }
  // four consecutive entries per thread
  const i64 first = e0 + (i64)threadIdx.x * AC_PER_THREAD;
  u32 pos[AC_PER_THREAD];
  int kept = 0;
#pragma unroll
  for (int j = 0; j < AC_PER_THREAD; ++j) {
    const i64 e = first + j;
    pos[j] = MAP_ABSENT;
    if (e < nnz) {
      const i64 id = load_index<IndexT>(indices, e);
      if (id >= 0 && id < id_bound) pos[j] = __ldg(map + id);
    }
    kept += pos[j] != MAP_ABSENT;
  }
  i64 total;
  const i64 loff = block_exclusive_scan((i64)kept, s_scan, &total);  // also orders s_lo / s_hi
  if (threadIdx.x < 32) {
    const i64 base = chained_exclusive_prefix(status, tile, total, err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  i64 run = s_base + loff;  // kept entries before this thread's first entry
  if (first < nnz) {
    i64 seg = segment_in_range(indptr, s_lo, s_hi, first);
    i64 seg_end = __ldg(indptr + seg + 1);
#pragma unroll
    for (int j = 0; j < AC_PER_THREAD; ++j) {
      const i64 e = first + j;
      if (e >= nnz) break;
      while (e >= seg_end) { ++seg; seg_end = __ldg(indptr + seg + 1); }  // skips empty segments
      if (!FILL) {
        if (__ldg(indptr + seg) == e) {  // first entry of its segment: the segment's output offset
          i64 s = seg;
          out_indptr[s] = run;
          while (s > 0 && __ldg(indptr + s - 1) == e) out_indptr[--s] = run;  // empty ones before it
        }
      } else if (pos[j] != MAP_ABSENT) {
        out_ids[run] = (i64)pos[j];
        out_sel[run] = e;
        if (out_seg) out_seg[run] = seg;
      }
      run += pos[j] != MAP_ABSENT;
    }
  }
  if (!FILL && tile == tiles - 1 && threadIdx.x == 0) {
    const i64 grand = s_base + total;  // everything kept; also the offset of trailing empty segments
    i64 s = nseg;
    out_indptr[s] = grand;
    while (s > 0 && indptr[s - 1] == nnz) out_indptr[--s] = grand;
  }
}

// COO filter: keep edge e iff key[e] is in the set; ordered compaction.
__global__ void __launch_bounds__(RS_THREADS)
coo_filter_kernel(const i64* __restrict__ key, const i64* __restrict__ other, i64 nnz,
                  const u32* __restrict__ map, i64 id_bound, i64* __restrict__ out_key,
                  i64* __restrict__ out_other, i64* __restrict__ out_sel, i64* d_count, u64* status,
                  int* ticket, int* err) {
  __shared__ i64 s_scan[34];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  const i64 e = (i64)tile * RS_THREADS + threadIdx.x;
  u32 pos = MAP_ABSENT;
  if (e < nnz) {
    const i64 id = key[e];
    if (id >= 0 && id < id_bound) pos = __ldg(map + id);
  }
  i64 total;
  const i64 loff = block_exclusive_scan(pos != MAP_ABSENT ? 1 : 0, s_scan, &total);
  if (threadIdx.x < 32) {
    i64 base = chained_exclusive_prefix(status, tile, total, err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  if (pos != MAP_ABSENT) {
    const i64 w = s_base + loff;
    out_key[w] = (i64)pos;
    out_other[w] = other[e];
    out_sel[w] = e;
  }
  if ((e == nnz - 1) || (nnz == 0 && e == 0)) *d_count = s_base + total;
}

struct AcrossLayout {
  size_t ticket, status, map, total;
  i64 tiles;
};

static AcrossLayout across_layout(i64 units, i64 id_bound) {
  AcrossLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.tiles = (units + RS_THREADS - 1) / RS_THREADS + 1;
  size_t o = 0;
  L.ticket = o; o = up(o + 256);
  L.status = o; o = up(o + sizeof(u64) * (size_t)L.tiles);
  L.map = o; o = up(o + sizeof(u32) * (size_t)(id_bound > 0 ? id_bound : 1));
  L.total = o;
  return L;
}

static int build_map(char* ws, const AcrossLayout& L, const i64* ids, i64 R, i64 id_bound,
                     int* d_err, cudaStream_t st) {
  GSB_CUDA_OK(cudaMemsetAsync(ws, 0, L.map, st));  // ticket + status
  i64 g = (id_bound + 255) / 256; if (g > 148 * 16) g = 148 * 16; if (g < 1) g = 1;
  { LaunchScope ls(KID_SLICE_ROWS, st); map_fill_kernel<<<(int)g, 256, 0, st>>>((u32*)(ws + L.map), id_bound); }
  if (R > 0) {
    g = (R + 255) / 256; if (g > 148 * 16) g = 148 * 16;
    LaunchScope ls(KID_SLICE_ROWS, st);
    map_build_kernel<<<(int)g, 256, 0, st>>>(ids, R, (u32*)(ws + L.map), id_bound, d_err);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}


// ---------------------------------------------------------------- columns AND rows, per minibatch
// Induced sub-matrices: minibatch b keeps, of its columns cols[col_ptr[b]..),
// the entries whose row id is in its own row list rows[row_ptr[b]..).  B direct
// maps would be B * id_bound words, so membership is one open-addressing table
// per minibatch (slot = id:32 | position:32, smallest position wins), sized
// 2 * |rows_b| + 32 and placed at 2 * row_ptr[b] + 32 * b -- both follow from
// row_ptr alone, no set-up pass.
constexpr u64 RT_EMPTY = ~0ull;

__device__ __forceinline__ u64* rowtab_of(u64* table, const i64* __restrict__ row_ptr, int b,
                                          u32* slots) {
  const i64 r0 = row_ptr[b];
  *slots = (u32)(2 * (row_ptr[b + 1] - r0) + 32);
  return table + 2 * r0 + 32 * (i64)b;
}

__global__ void rowtab_insert_kernel(const i64* __restrict__ rows, const i64* __restrict__ row_ptr,
                                     int B, u64* table, int* err) {
  const i64 R = row_ptr[B];
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < R; i += (i64)gridDim.x * blockDim.x) {
    const int b = find_segment(row_ptr, B, i);
    const i64 id = rows[i];
    if (id < 0 || id >= 0xFFFFFFFFll) { raise(err, ERRBIT_BAD_INPUT); continue; }
    u32 slots;
    u64* tab = rowtab_of(table, row_ptr, b, &slots);
    const u64 packed = ((u64)(u32)id << 32) | (u32)i;
    u32 pos = __umulhi(hash32((u32)id), slots);
    u32 probes = 0;
    for (; probes < slots; ++probes) {
      u64 cur = ld_relaxed(tab + pos);
      if (cur == RT_EMPTY) {
        cur = atomicCAS(tab + pos, RT_EMPTY, packed);
        if (cur == RT_EMPTY) break;
      }
      if ((u32)(cur >> 32) == (u32)id) {
        if ((u32)cur > (u32)i) atomicMin(tab + pos, packed);
        break;
      }
      pos = pos + 1 == slots ? 0 : pos + 1;
    }
    if (probes == slots) raise(err, ERRBIT_TABLE_FULL);
  }
}

__device__ __forceinline__ u32 rowtab_find(const u64* __restrict__ tab, u32 slots, i64 id) {
  if (id < 0 || id >= 0xFFFFFFFFll) return MAP_ABSENT;
  u32 pos = __umulhi(hash32((u32)id), slots);
  for (u32 probes = 0; probes < slots; ++probes) {
    const u64 cur = __ldg(tab + pos);
    if (cur == RT_EMPTY) return MAP_ABSENT;
    if ((u32)(cur >> 32) == (u32)id) return (u32)cur;
    pos = pos + 1 == slots ? 0 : pos + 1;
  }
  return MAP_ABSENT;
}

// CTA = RS_THREADS consecutive column slots; a warp walks one column at a time.
template <typename IndexT>
__global__ void __launch_bounds__(RS_THREADS)
colrow_count_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 num_cols,
                    const i64* __restrict__ cols, const i64* __restrict__ col_ptr,
                    const i64* __restrict__ row_ptr, int B, u64* table, i64* __restrict__ out_indptr,
                    u64* status, int* ticket, int* err) {
  __shared__ i64 s_scan[34];
  __shared__ int s_cnt[RS_THREADS];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const i64 nseg = col_ptr[B];
  const i64 seg0 = (i64)tile * RS_THREADS;
  for (int k = wid; k < RS_THREADS; k += RS_WARPS) {
    const i64 seg = seg0 + k;
    int cnt = 0;
    if (seg < nseg) {
      const i64 c = cols[seg];
      if (c < 0 || c >= num_cols) {
        if (lane == 0) raise(err, ERRBIT_BAD_INPUT);
      } else {
        u32 slots;
        const u64* tab = rowtab_of(table, row_ptr, find_segment(col_ptr, B, seg), &slots);
        const i64 st = __ldg(indptr + c), en = __ldg(indptr + c + 1);
        for (i64 e = st + lane; e < en; e += 32)
          if (rowtab_find(tab, slots, load_index<IndexT>(indices, e)) != MAP_ABSENT) ++cnt;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
      }
    }
    if (lane == 0) s_cnt[k] = cnt;
  }
  __syncthreads();
  i64 total;
  const i64 loff = block_exclusive_scan((i64)s_cnt[threadIdx.x], s_scan, &total);
  if (threadIdx.x < 32) {
    i64 base = chained_exclusive_prefix(status, tile, total, err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  const i64 seg = seg0 + threadIdx.x;
  if (seg < nseg) out_indptr[seg] = s_base + loff;
  if (seg == nseg - 1 || (nseg == 0 && seg == 0)) out_indptr[nseg] = s_base + total;
}

template <typename IndexT>
__global__ void __launch_bounds__(RS_THREADS)
colrow_fill_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 num_cols,
                   const i64* __restrict__ cols, const i64* __restrict__ col_ptr,
                   const i64* __restrict__ row_ptr, int B, const u64* __restrict__ table,
                   const i64* __restrict__ out_indptr, i64* __restrict__ out_ids,
                   i64* __restrict__ out_seg, i64* __restrict__ out_sel) {
  const int lane = threadIdx.x & 31;
  const i64 nseg = col_ptr[B];
  const i64 warp0 = ((i64)blockIdx.x * RS_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * RS_THREADS) >> 5;
  for (i64 seg = warp0; seg < nseg; seg += nwarps) {
    const i64 c = cols[seg];
    if (c < 0 || c >= num_cols) continue;
    u32 slots;
    const u64* tab = rowtab_of(const_cast<u64*>(table), row_ptr, find_segment(col_ptr, B, seg), &slots);
    const i64 st = __ldg(indptr + c), en = __ldg(indptr + c + 1);
    i64 o = out_indptr[seg];
    for (i64 e0 = st; e0 < en; e0 += 32) {
      const i64 e = e0 + lane;
      u32 pos = MAP_ABSENT;
      if (e < en) pos = rowtab_find(tab, slots, load_index<IndexT>(indices, e));
      const unsigned keep = __ballot_sync(0xffffffffu, pos != MAP_ABSENT);
      if (pos != MAP_ABSENT) {
        const i64 w = o + __popc(keep & ((1u << lane) - 1u));
        out_ids[w] = (i64)pos;
        out_sel[w] = e;
        if (out_seg) out_seg[w] = seg;
      }
      o += __popc(keep);
    }
  }
}

struct ColRowLayout {
  size_t ticket, status, table, total;
  i64 tiles, slots;
};

static ColRowLayout colrow_layout(i64 S, i64 R, i64 B) {
  ColRowLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.tiles = (S + RS_THREADS - 1) / RS_THREADS + 1;
  L.slots = 2 * R + 32 * (B + 1);
  size_t o = 0;
  L.ticket = o; o = up(o + 256);
  L.status = o; o = up(o + sizeof(u64) * (size_t)L.tiles);
  L.table = o; o = up(o + sizeof(u64) * (size_t)L.slots);
  L.total = o;
  return L;
}

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_slice_across_workspace_bytes(int64_t nnz_max, int64_t id_bound) {
  if (nnz_max < 0 || id_bound < 0) return 0;
  return across_layout((nnz_max + AC_PER_THREAD - 1) / AC_PER_THREAD, id_bound).total;
}

template <bool FILL>
static int launch_across(const int64_t* indptr, const void* indices, int indices_dtype, int64_t nseg,
                         int64_t nnz_max, int64_t id_bound, int64_t* out_indptr, int64_t* out_ids,
                         int64_t* out_seg, int64_t* out_sel, char* ws, const AcrossLayout& L, int* d_err,
                         cudaStream_t st) {
  const int tiles = nnz_max == 0 ? 1 : ceil_div_i(nnz_max, AC_TILE);
  LaunchScope ls(KID_SLICE_ROWS, st);
  if (indices_dtype == GSB_I32)
    across_kernel<int, FILL><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, nseg, nnz_max, (const u32*)(ws + L.map), id_bound, (i64*)out_indptr,
        (i64*)out_ids, (i64*)out_seg, (i64*)out_sel, (u64*)(ws + L.status), (int*)(ws + L.ticket), d_err);
  else
    across_kernel<i64, FILL><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, nseg, nnz_max, (const u32*)(ws + L.map), id_bound, (i64*)out_indptr,
        (i64*)out_ids, (i64*)out_seg, (i64*)out_sel, (u64*)(ws + L.status), (int*)(ws + L.ticket), d_err);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_slice_across_count(const int64_t* indptr, const void* indices, int indices_dtype,
                                      int64_t nseg, int64_t nnz_max, const int64_t* ids, int64_t R,
                                      int64_t id_bound, int64_t* out_indptr, void* workspace,
                                      size_t workspace_bytes, int* d_err, void* cuda_stream) {
  if (!indptr || !out_indptr || nseg < 0 || nnz_max < 0 || R < 0 || id_bound < 0 || (R > 0 && !ids) ||
      (nnz_max > 0 && !indices))
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (R >= 0xFFFFFFFFll || id_bound > (1ll << 33)) return GSB_ERR_UNSUPPORTED;
  const AcrossLayout L = across_layout((nnz_max + AC_PER_THREAD - 1) / AC_PER_THREAD, id_bound);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  int rc = build_map(ws, L, (const i64*)ids, R, id_bound, d_err, st);
  if (rc != GSB_OK) return rc;
  return launch_across<false>(indptr, indices, indices_dtype, nseg, nnz_max, id_bound, out_indptr, nullptr,
                              nullptr, nullptr, ws, L, d_err, st);
}

extern "C" int gsb_slice_across_fill(const int64_t* indptr, const void* indices, int indices_dtype,
                                     int64_t nseg, int64_t nnz_max, int64_t id_bound,
                                     int64_t* out_ids, int64_t* out_seg, int64_t* out_sel,
                                     void* workspace, size_t workspace_bytes, int* d_err,
                                     void* cuda_stream) {
  if (nseg == 0 || nnz_max == 0) return GSB_OK;
  if (!indptr || !indices || !out_ids || !out_sel || !workspace || nseg < 0 || nnz_max < 0)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  const AcrossLayout L = across_layout((nnz_max + AC_PER_THREAD - 1) / AC_PER_THREAD, id_bound);
  if (workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  GSB_CUDA_OK(cudaMemsetAsync(ws, 0, L.map, st));  // ticket + status again; the map stays
  return launch_across<true>(indptr, indices, indices_dtype, nseg, nnz_max, id_bound, nullptr, out_ids,
                             out_seg, out_sel, ws, L, d_err, st);
}

extern "C" size_t gsb_coo_filter_workspace_bytes(int64_t nnz, int64_t id_bound) {
  if (nnz < 0 || id_bound < 0) return 0;
  return across_layout(nnz, id_bound).total;
}

extern "C" int gsb_coo_filter(const int64_t* key, const int64_t* other, int64_t nnz,
                              const int64_t* ids, int64_t R, int64_t id_bound, int64_t* out_key,
                              int64_t* out_other, int64_t* out_sel, int64_t* d_count,
                              void* workspace, size_t workspace_bytes, int* d_err,
                              void* cuda_stream) {
  if (nnz < 0 || R < 0 || id_bound < 0 || !d_count || (R > 0 && !ids)) return GSB_ERR_INVALID;
  if (nnz > 0 && (!key || !other || !out_key || !out_other || !out_sel)) return GSB_ERR_INVALID;
  if (R >= 0xFFFFFFFFll || id_bound > (1ll << 33)) return GSB_ERR_UNSUPPORTED;
  const AcrossLayout L = across_layout(nnz, id_bound);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  int rc = build_map(ws, L, (const i64*)ids, R, id_bound, d_err, st);
  if (rc != GSB_OK) return rc;
  const int tiles = nnz == 0 ? 1 : ceil_div_i(nnz, RS_THREADS);
  LaunchScope ls(KID_SLICE_ROWS, st);
  coo_filter_kernel<<<tiles, RS_THREADS, 0, st>>>(
      (const i64*)key, (const i64*)other, nnz, (const u32*)(ws + L.map), id_bound, (i64*)out_key,
      (i64*)out_other, (i64*)out_sel, (i64*)d_count, (u64*)(ws + L.status), (int*)(ws + L.ticket),
      d_err);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" size_t gsb_slice_cols_rows_workspace_bytes(int64_t S, int64_t R, int64_t B) {
  if (S < 0 || R < 0 || B < 0) return 0;
  return colrow_layout(S, R, B).total;
}

extern "C" int gsb_slice_cols_rows_count(const int64_t* indptr, const void* indices,
                                         int indices_dtype, int64_t num_cols, const int64_t* cols,
                                         const int64_t* col_ptr, int64_t S, const int64_t* rows,
                                         const int64_t* row_ptr, int64_t R, int64_t B,
                                         int64_t* out_indptr, void* workspace,
                                         size_t workspace_bytes, int* d_err, void* cuda_stream) {
  if (!indptr || !out_indptr || !col_ptr || !row_ptr || S < 0 || R < 0 || B < 1 || num_cols < 0 ||
      (S > 0 && (!cols || !indices)) || (R > 0 && !rows))
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (R >= 0x7FFFFFFFll || B >= (1ll << 24)) return GSB_ERR_UNSUPPORTED;
  const ColRowLayout L = colrow_layout(S, R, B);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  GSB_CUDA_OK(cudaMemsetAsync(ws, 0, L.table, st));                               // ticket + status
  GSB_CUDA_OK(cudaMemsetAsync(ws + L.table, 0xFF, sizeof(u64) * (size_t)L.slots, st));  // empty slots
  if (R > 0) {
    i64 g = (R + 255) / 256; if (g > 148 * 16) g = 148 * 16;
    LaunchScope ls(KID_SLICE_ROWS, st);
    rowtab_insert_kernel<<<(int)g, 256, 0, st>>>((const i64*)rows, (const i64*)row_ptr, (int)B,
                                                 (u64*)(ws + L.table), d_err);
  }
  const int tiles = S == 0 ? 1 : ceil_div_i(S, RS_THREADS);
  LaunchScope ls(KID_SLICE_ROWS, st);
  if (indices_dtype == GSB_I32)
    colrow_count_kernel<int><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_cols, (const i64*)cols, (const i64*)col_ptr,
        (const i64*)row_ptr, (int)B, (u64*)(ws + L.table), (i64*)out_indptr, (u64*)(ws + L.status),
        (int*)(ws + L.ticket), d_err);
  else
    colrow_count_kernel<i64><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_cols, (const i64*)cols, (const i64*)col_ptr,
        (const i64*)row_ptr, (int)B, (u64*)(ws + L.table), (i64*)out_indptr, (u64*)(ws + L.status),
        (int*)(ws + L.ticket), d_err);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_slice_cols_rows_fill(const int64_t* indptr, const void* indices,
                                        int indices_dtype, int64_t num_cols, const int64_t* cols,
                                        const int64_t* col_ptr, int64_t S, const int64_t* row_ptr,
                                        int64_t R, int64_t B, const int64_t* out_indptr,
                                        int64_t* out_ids, int64_t* out_seg, int64_t* out_sel,
                                        const void* workspace, void* cuda_stream) {
  if (S == 0) return GSB_OK;
  if (!indptr || !indices || !cols || !col_ptr || !row_ptr || !out_indptr || !out_ids || !out_sel ||
      !workspace || S < 0 || B < 1)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  const ColRowLayout L = colrow_layout(S, R, B);
  cudaStream_t st = (cudaStream_t)cuda_stream;
  i64 g = (S + RS_WARPS - 1) / RS_WARPS; if (g > 148 * 16) g = 148 * 16;
  const u64* table = (const u64*)((const char*)workspace + L.table);
  LaunchScope ls(KID_SLICE_ROWS, st);
  if (indices_dtype == GSB_I32)
    colrow_fill_kernel<int><<<(int)g, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_cols, (const i64*)cols, (const i64*)col_ptr,
        (const i64*)row_ptr, (int)B, table, (const i64*)out_indptr, (i64*)out_ids, (i64*)out_seg,
        (i64*)out_sel);
  else
    colrow_fill_kernel<i64><<<(int)g, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, num_cols, (const i64*)cols, (const i64*)col_ptr,
        (const i64*)row_ptr, (int)B, table, (const i64*)out_indptr, (i64*)out_ids, (i64*)out_seg,
        (i64*)out_sel);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
