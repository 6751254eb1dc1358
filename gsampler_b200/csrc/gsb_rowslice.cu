// Slicing ACROSS the compressed dimension: keep the entries of a CSC (CSR)
// whose row (column) id belongs to a given set and rename each kept id to its
// position in the set -- A[rows, :] evaluated on a CSC operand -- and the same
// filter on a COO operand.
//
// Membership is a direct-address map (one 32-bit word per possible id, built
// per call in the workspace): no probing, one L2-resident load per entry.
// A warp owns a segment (column): pass 1 counts the survivors per segment and
// turns the counts into offsets (chained tile prefix); pass 2 rewrites the
// survivors in order using warp ballots, so the output keeps the operand's
// entry order inside every segment.
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

// Tile = RS_WARPS segments per iteration is too coarse for the chained prefix,
// so a CTA owns RS_THREADS consecutive segments: warps stride over them to
// count, then one scan + tile prefix yields the offsets of all of them.
template <typename IndexT>
__global__ void __launch_bounds__(RS_THREADS)
across_count_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 nseg,
                    const u32* __restrict__ map, i64 id_bound, i64* __restrict__ out_indptr,
                    u64* status, int* ticket, int* err) {
  __shared__ i64 s_scan[34];
  __shared__ int s_cnt[RS_THREADS];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const i64 seg0 = (i64)tile * RS_THREADS;
  for (int k = wid; k < RS_THREADS; k += RS_WARPS) {
    const i64 seg = seg0 + k;
    int cnt = 0;
    if (seg < nseg) {
      const i64 st = __ldg(indptr + seg), en = __ldg(indptr + seg + 1);
      for (i64 e = st + lane; e < en; e += 32) {
        const i64 id = load_index<IndexT>(indices, e);
        if (id >= 0 && id < id_bound && __ldg(map + id) != MAP_ABSENT) ++cnt;
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
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
across_fill_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 nseg,
                   const u32* __restrict__ map, i64 id_bound, const i64* __restrict__ out_indptr,
                   i64* __restrict__ out_ids, i64* __restrict__ out_seg, i64* __restrict__ out_sel) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * RS_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * RS_THREADS) >> 5;
  for (i64 seg = warp0; seg < nseg; seg += nwarps) {
    const i64 st = __ldg(indptr + seg), en = __ldg(indptr + seg + 1);
    i64 o = out_indptr[seg];
    for (i64 e0 = st; e0 < en; e0 += 32) {
      const i64 e = e0 + lane;
      u32 pos = MAP_ABSENT;
      if (e < en) {
        const i64 id = load_index<IndexT>(indices, e);
        if (id >= 0 && id < id_bound) pos = __ldg(map + id);
      }
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

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_slice_across_workspace_bytes(int64_t nseg, int64_t id_bound) {
  if (nseg < 0 || id_bound < 0) return 0;
  return across_layout(nseg, id_bound).total;
}

extern "C" int gsb_slice_across_count(const int64_t* indptr, const void* indices, int indices_dtype,
                                      int64_t nseg, const int64_t* ids, int64_t R, int64_t id_bound,
                                      int64_t* out_indptr, void* workspace, size_t workspace_bytes,
                                      int* d_err, void* cuda_stream) {
  if (!indptr || !out_indptr || nseg < 0 || R < 0 || id_bound < 0 || (R > 0 && !ids))
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (R >= 0xFFFFFFFFll || id_bound > (1ll << 33)) return GSB_ERR_UNSUPPORTED;
  const AcrossLayout L = across_layout(nseg, id_bound);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  int rc = build_map(ws, L, (const i64*)ids, R, id_bound, d_err, st);
  if (rc != GSB_OK) return rc;
  const int tiles = nseg == 0 ? 1 : ceil_div_i(nseg, RS_THREADS);
  LaunchScope ls(KID_SLICE_ROWS, st);
  if (indices_dtype == GSB_I32)
    across_count_kernel<int><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, nseg, (const u32*)(ws + L.map), id_bound, (i64*)out_indptr,
        (u64*)(ws + L.status), (int*)(ws + L.ticket), d_err);
  else
    across_count_kernel<i64><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, nseg, (const u32*)(ws + L.map), id_bound, (i64*)out_indptr,
        (u64*)(ws + L.status), (int*)(ws + L.ticket), d_err);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_slice_across_fill(const int64_t* indptr, const void* indices, int indices_dtype,
                                     int64_t nseg, int64_t id_bound, const int64_t* out_indptr,
                                     int64_t* out_ids, int64_t* out_seg, int64_t* out_sel,
                                     const void* workspace, void* cuda_stream) {
  if (nseg == 0) return GSB_OK;
  if (!indptr || !indices || !out_indptr || !out_ids || !out_sel || !workspace || nseg < 0)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  const AcrossLayout L = across_layout(nseg, id_bound);
  cudaStream_t st = (cudaStream_t)cuda_stream;
  i64 g = (nseg + RS_WARPS - 1) / RS_WARPS; if (g > 148 * 16) g = 148 * 16;
  const u32* map = (const u32*)((const char*)workspace + L.map);
  LaunchScope ls(KID_SLICE_ROWS, st);
  if (indices_dtype == GSB_I32)
    across_fill_kernel<int><<<(int)g, RS_THREADS, 0, st>>>((const i64*)indptr, indices, nseg, map,
                                                           id_bound, (const i64*)out_indptr,
                                                           (i64*)out_ids, (i64*)out_seg, (i64*)out_sel);
  else
    across_fill_kernel<i64><<<(int)g, RS_THREADS, 0, st>>>((const i64*)indptr, indices, nseg, map,
                                                           id_bound, (const i64*)out_indptr,
                                                           (i64*)out_ids, (i64*)out_seg, (i64*)out_sel);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
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
