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

// bits[w] bit j = (map[32 w + j] present): the membership test of the counting pass, small enough
// (one bit per possible id) to stay in L1 where the 32-bit map only fits L2
__global__ void bits_build_kernel(const u32* __restrict__ map, i64 id_bound, u32* __restrict__ bits) {
  const i64 rounded = (id_bound + 31) & ~(i64)31;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < rounded; i += (i64)gridDim.x * blockDim.x) {
    const unsigned present = __ballot_sync(0xffffffffu, i < id_bound && map[i] != MAP_ABSENT);
    if ((threadIdx.x & 31) == 0) bits[i >> 5] = present;
  }
}

// tile_seg[t] = segment of entry t * AC_TILE (the last segment for tiles past the end).  One
// thread per tile: the 20-odd dependent loads of a binary search over the whole indptr are hidden
// by the other searches here, where inside the tile kernels they were each tile's critical path.
__global__ void tile_segment_kernel(const i64* __restrict__ indptr, i64 nseg, i64 n_tiles,
                                    i64* __restrict__ tile_seg) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tiles || nseg <= 0) return;
  const i64 e = t * AC_TILE, nnz = indptr[nseg];
  tile_seg[t] = e < nnz ? (i64)find_segment(indptr, (int)nseg, e) : nseg - 1;
}

// Pass 1: membership of every entry (bitmap test), one byte per thread saying which of its four
// entries stay, the thread's exclusive offset inside its tile (16 bits) and the tile's total.
// The tiles' exclusive prefixes come from a separate one-CTA scan (tile_scan_kernel): with over
// 10^5 tiles a chained look-back was the critical path of this pass (its prefix moves at most 32
// tiles per memory round trip).  No segment logic here: the segments' output offsets follow from
// these arrays (across_offsets_kernel), and so do the output positions of pass 2, which therefore
// needs neither a scan nor a barrier.
template <typename IndexT>
__global__ void __launch_bounds__(RS_THREADS)
across_mark_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 nseg,
                   i64 nnz_max, const u32* __restrict__ bits, i64 id_bound,
                   unsigned char* __restrict__ nib, unsigned short* __restrict__ toff,
                   u32* __restrict__ tile_total, int* err) {
  __shared__ i64 s_scan[34];
  const i64 tile = blockIdx.x;
  i64 nnz = nseg > 0 ? indptr[nseg] : 0;
  if (nnz > nnz_max || nnz < 0) {
    if (tile == 0 && threadIdx.x == 0) raise(err, ERRBIT_CAPACITY);
    nnz = 0;
  }
  const i64 tiles = nnz == 0 ? 1 : (nnz + AC_TILE - 1) / AC_TILE;
  if (tile >= tiles) return;
  const i64 first = tile * AC_TILE + (i64)threadIdx.x * AC_PER_THREAD;
  unsigned keep = 0;  // bit j: entry first + j stays
#pragma unroll
  for (int j = 0; j < AC_PER_THREAD; ++j) {
    const i64 e = first + j;
    if (e < nnz) {
      const i64 id = load_index<IndexT>(indices, e);
      if (id >= 0 && id < id_bound && ((__ldg(bits + (id >> 5)) >> (id & 31)) & 1u)) keep |= 1u << j;
    }
  }
  i64 total;
  const i64 loff = block_exclusive_scan((i64)__popc(keep), s_scan, &total);
  nib[tile * RS_THREADS + threadIdx.x] = (unsigned char)keep;
  toff[tile * RS_THREADS + threadIdx.x] = (unsigned short)loff;
  if (threadIdx.x == 0) tile_total[tile] = (u32)total;
}

// tile_base[t] = sum of tile_total[0..t), tile_base[tiles] = everything; one CTA, every thread a
// contiguous run of tiles
__global__ void __launch_bounds__(1024)
tile_scan_kernel(const i64* __restrict__ indptr, i64 nseg, i64 nnz_max,
                 const u32* __restrict__ tile_total, i64* __restrict__ tile_base) {
  __shared__ i64 s_scan[34];
  i64 nnz = nseg > 0 ? indptr[nseg] : 0;
  if (nnz > nnz_max || nnz < 0) nnz = 0;
  const i64 tiles = nnz == 0 ? 1 : (nnz + AC_TILE - 1) / AC_TILE;
  const i64 per = (tiles + 1023) / 1024;
  const i64 lo = (i64)threadIdx.x * per, hi = lo + per < tiles ? lo + per : tiles;
  i64 sum = 0;
  for (i64 t = lo; t < hi; ++t) sum += tile_total[t];
  i64 grand;
  i64 run = block_exclusive_scan(sum, s_scan, &grand);
  for (i64 t = lo; t < hi; ++t) { tile_base[t] = run; run += tile_total[t]; }
  if (threadIdx.x == 0) tile_base[tiles] = grand;
}

// kept entries before entry e (e < nnz)
__device__ __forceinline__ i64 across_kept_before(i64 e, const unsigned char* __restrict__ nib,
                                                  const unsigned short* __restrict__ toff,
                                                  const i64* __restrict__ tile_base) {
  const i64 t = e / AC_PER_THREAD;  // tile * RS_THREADS + thread
  const unsigned below = (1u << (unsigned)(e % AC_PER_THREAD)) - 1u;
  return tile_base[e / AC_TILE] + (i64)toff[t] + __popc((unsigned)nib[t] & below);
}

// out_indptr[s] = kept entries before the first entry of segment s; thread per segment
__global__ void across_offsets_kernel(const i64* __restrict__ indptr, i64 nseg, i64 nnz_max,
                                      const unsigned char* __restrict__ nib,
                                      const unsigned short* __restrict__ toff,
                                      const i64* __restrict__ tile_base, i64* __restrict__ out_indptr) {
  i64 nnz = nseg > 0 ? indptr[nseg] : 0;
  if (nnz > nnz_max || nnz < 0) nnz = 0;
  const i64 tiles = nnz == 0 ? 1 : (nnz + AC_TILE - 1) / AC_TILE;
  for (i64 s = (i64)blockIdx.x * blockDim.x + threadIdx.x; s <= nseg; s += (i64)gridDim.x * blockDim.x) {
    const i64 e = indptr[s];
    out_indptr[s] = e >= nnz || e < 0 ? tile_base[tiles] : across_kept_before(e, nib, toff, tile_base);
  }
}

// Pass 2: every thread writes the kept ones of its four entries; the segment of an entry is
// looked up only when the caller wants the COO form (out_seg).
template <typename IndexT>
__global__ void __launch_bounds__(RS_THREADS)
across_fill_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices, i64 nseg,
                   i64 nnz_max, const u32* __restrict__ map, const unsigned char* __restrict__ nib,
                   const unsigned short* __restrict__ toff, const i64* __restrict__ tile_base,
                   const i64* __restrict__ tile_seg, i64* __restrict__ out_ids,
                   i64* __restrict__ out_seg, i64* __restrict__ out_sel) {
  const i64 nnz = nseg > 0 ? indptr[nseg] : 0;
  if (nnz > nnz_max || nnz < 0) return;
  const i64 tile = blockIdx.x;
  const i64 t = tile * RS_THREADS + threadIdx.x;
  const i64 first = t * AC_PER_THREAD;
  if (first >= nnz) return;
  const unsigned keep = nib[t];
  if (!keep) return;
  i64 run = tile_base[tile] + (i64)toff[t];
  i64 seg = 0, seg_end = 0;
  if (out_seg) {
    seg = segment_in_range(indptr, tile_seg[tile], tile_seg[tile + 1], first);
    seg_end = __ldg(indptr + seg + 1);
  }
#pragma unroll
  for (int j = 0; j < AC_PER_THREAD; ++j) {
    if (!((keep >> j) & 1u)) continue;
    const i64 e = first + j;
    out_ids[run] = (i64)__ldg(map + load_index<IndexT>(indices, e));
    out_sel[run] = e;
    if (out_seg) {
      while (e >= seg_end) { ++seg; seg_end = __ldg(indptr + seg + 1); }  // skips empty segments
      out_seg[run] = seg;
    }
    ++run;
  }
}

// COO filter: keep edge e iff key[e] is in the set; ordered compaction over tiles of 1024 edges
// (four consecutive edges per thread).
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
  const i64 tiles = nnz == 0 ? 1 : (nnz + AC_TILE - 1) / AC_TILE;
  if (tile >= tiles) return;
  const i64 first = (i64)tile * AC_TILE + (i64)threadIdx.x * AC_PER_THREAD;
  u32 pos[AC_PER_THREAD];
  int kept = 0;
#pragma unroll
  for (int j = 0; j < AC_PER_THREAD; ++j) {
    pos[j] = MAP_ABSENT;
    if (first + j < nnz) {
      const i64 id = key[first + j];
      if (id >= 0 && id < id_bound) pos[j] = __ldg(map + id);
    }
    kept += pos[j] != MAP_ABSENT;
  }
  i64 total;
  const i64 loff = block_exclusive_scan((i64)kept, s_scan, &total);
  if (threadIdx.x < 32) {
    i64 base = chained_exclusive_prefix(status, tile, total, err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  i64 w = s_base + loff;
#pragma unroll
  for (int j = 0; j < AC_PER_THREAD; ++j) {
    if (pos[j] != MAP_ABSENT) {
      out_key[w] = (i64)pos[j];
      out_other[w] = other[first + j];
      out_sel[w] = first + j;
      ++w;
    }
  }
  if (tile == tiles - 1 && threadIdx.x == 0) *d_count = s_base + total;
}

struct AcrossLayout {
  size_t ticket, status, map, bits, nib, toff, tile_total, tile_base, tile_seg, total;
  i64 tiles;
};

// `entries` = most entries the operand can hold; with_mask adds what the two-pass CSC form hands
// from its first pass to its second
static AcrossLayout across_layout(i64 entries, i64 id_bound, bool with_mask) {
  AcrossLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.tiles = (entries + AC_TILE - 1) / AC_TILE + 1;
  size_t o = 0;
  L.ticket = o; o = up(o + 256);
  L.status = o; o = up(o + sizeof(u64) * (size_t)L.tiles);
  L.map = o; o = up(o + sizeof(u32) * (size_t)(id_bound > 0 ? id_bound : 1));
  L.bits = o; if (with_mask) o = up(o + sizeof(u32) * (size_t)(id_bound / 32 + 1));
  L.nib = o; if (with_mask) o = up(o + (size_t)L.tiles * RS_THREADS);
  L.toff = o; if (with_mask) o = up(o + sizeof(unsigned short) * (size_t)L.tiles * RS_THREADS);
  L.tile_total = o; if (with_mask) o = up(o + sizeof(u32) * (size_t)L.tiles);
  L.tile_base = o; if (with_mask) o = up(o + sizeof(i64) * (size_t)(L.tiles + 1));
  L.tile_seg = o; if (with_mask) o = up(o + sizeof(i64) * (size_t)(L.tiles + 1));
  L.total = o;
  return L;
}

static int build_map(char* ws, const AcrossLayout& L, const i64* ids, i64 R, i64 id_bound,
                     int* d_err, cudaStream_t st) {
  GSB_CUDA_OK(cudaMemsetAsync(ws, 0, L.map, st));  // ticket + status
  i64 g = (id_bound + 255) / 256; if (g > sm_count() * 16) g = sm_count() * 16; if (g < 1) g = 1;
  { LaunchScope ls(KID_SLICE_ROWS, st); map_fill_kernel<<<(int)g, 256, 0, st>>>((u32*)(ws + L.map), id_bound); }
  if (R > 0) {
    g = (R + 255) / 256; if (g > sm_count() * 16) g = sm_count() * 16;
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

// Fused column + row slicing works on PARTS of columns: a column of `deg` entries is cut into
// ceil(deg / part_len) parts, part_len = max(CR_PART, total entries / CR_EXTRA_PARTS), so the
// number of parts is at most S + CR_EXTRA_PARTS whatever the degrees are, and a warp never walks
// more than part_len entries: one very long column costs the same as many short ones.
//   deg    : length of every selected column (ids checked) + their sum       thread / column
//   parts  : vptr = exclusive scan of the columns' part counts               one CTA
//   count  : kept entries of every part                                      warp / part
//   offsets: voff = exclusive scan of those; out_indptr[seg] = voff[vptr[seg]]   one CTA
//   fill   : ordered emit of every part from voff[part]                      warp / part
constexpr i64 CR_PART = 1024;
constexpr i64 CR_EXTRA_PARTS = 1 << 19;

__device__ __forceinline__ i64 colrow_part_len(i64 total_entries) {
  const i64 by_budget = (total_entries + CR_EXTRA_PARTS - 1) / CR_EXTRA_PARTS;
  const i64 len = by_budget > CR_PART ? by_budget : CR_PART;
  return (len + 127) & ~(i64)127;  // whole steps of 4 x 32 entries
}

__global__ void colrow_deg_kernel(const i64* __restrict__ indptr, i64 num_cols,
                                  const i64* __restrict__ cols, const i64* __restrict__ col_ptr, int B,
                                  i64 S, i64* __restrict__ deg, unsigned long long* total, int* err) {
  __shared__ i64 s_scan[34];
  const i64 nseg = col_ptr[B] < S ? col_ptr[B] : S;
  const i64 seg = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  i64 d = 0;
  if (seg < nseg) {
    const i64 c = cols[seg];
    if (c < 0 || c >= num_cols) raise(err, ERRBIT_BAD_INPUT);
    else d = __ldg(indptr + c + 1) - __ldg(indptr + c);
    deg[seg] = d;
  }
  i64 block_total;
  block_exclusive_scan(d, s_scan, &block_total);
  if (threadIdx.x == 0 && block_total) atomicAdd(total, (unsigned long long)block_total);
}

// out[i] = sum of f(i') for i' < i, out[n] = everything; one CTA of 1024 threads, a contiguous run
// of elements per thread
template <typename F>
__device__ __forceinline__ void cta_exclusive_scan(i64 n, F value, i64* __restrict__ out, i64* s_scan) {
  const i64 per = (n + 1023) / 1024;
  const i64 lo = (i64)threadIdx.x * per < n ? (i64)threadIdx.x * per : n;
  const i64 hi = lo + per < n ? lo + per : n;
  i64 sum = 0;
  for (i64 i = lo; i < hi; ++i) sum += value(i);
  i64 grand;
  i64 run = block_exclusive_scan(sum, s_scan, &grand);
  for (i64 i = lo; i < hi; ++i) { out[i] = run; run += value(i); }
  if (threadIdx.x == 0) out[n] = grand;
}

__global__ void __launch_bounds__(1024)
colrow_parts_kernel(const i64* __restrict__ col_ptr, int B, i64 S, const i64* __restrict__ deg,
                    const unsigned long long* __restrict__ total, i64* __restrict__ vptr) {
  __shared__ i64 s_scan[34];
  const i64 nseg = col_ptr[B] < S ? col_ptr[B] : S;
  const i64 part = colrow_part_len((i64)*total);
  cta_exclusive_scan(nseg, [&](i64 s) { const i64 d = deg[s]; return d == 0 ? (i64)1 : (d + part - 1) / part; },
                     vptr, s_scan);
}

// warp per part; FILL = false counts the kept entries, FILL = true writes them from voff[part]
template <typename IndexT, bool FILL>
__global__ void __launch_bounds__(RS_THREADS)
colrow_part_kernel(const i64* __restrict__ indptr, const void* __restrict__ indices,
                   const i64* __restrict__ cols, const i64* __restrict__ col_ptr,
                   const i64* __restrict__ row_ptr, int B, i64 S, const u64* __restrict__ table,
                   const i64* __restrict__ deg, const unsigned long long* __restrict__ total,
                   const i64* __restrict__ vptr, u32* __restrict__ vcnt, const i64* __restrict__ voff,
                   i64* __restrict__ out_ids, i64* __restrict__ out_seg, i64* __restrict__ out_sel) {
  const int lane = threadIdx.x & 31;
  const i64 nseg = col_ptr[B] < S ? col_ptr[B] : S;
  if (nseg <= 0) return;
  const i64 V = vptr[nseg];
  const i64 part = colrow_part_len((i64)*total);
  const i64 warp0 = ((i64)blockIdx.x * RS_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * RS_THREADS) >> 5;
  for (i64 v = warp0; v < V; v += nwarps) {
    // the column of part v: largest seg with vptr[seg] <= v
    i64 lo = 0, hi = nseg;
    while (hi - lo > 1) { const i64 mid = (lo + hi) >> 1; if (__ldg(vptr + mid) <= v) lo = mid; else hi = mid; }
    const i64 seg = lo;
    const i64 d = deg[seg];
    int cnt = 0;
    if (d > 0) {
      const i64 c = cols[seg];
      u32 slots;
      const u64* tab = rowtab_of(const_cast<u64*>(table), row_ptr, find_segment(col_ptr, B, seg), &slots);
      const i64 col_start = __ldg(indptr + c);
      const i64 st = col_start + (v - __ldg(vptr + seg)) * part;
      const i64 en = st + part < col_start + d ? st + part : col_start + d;
      i64 o = FILL ? voff[v] : 0;
      for (i64 e0 = st; e0 < en; e0 += 128) {  // four chunks of 32 entries in flight
        i64 id[4];
        u32 pos[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const i64 e = e0 + 32 * k + lane;
          id[k] = e < en ? load_index<IndexT>(indices, e) : -1;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) pos[k] = id[k] >= 0 ? rowtab_find(tab, slots, id[k]) : MAP_ABSENT;
        if (!FILL) {
#pragma unroll
          for (int k = 0; k < 4; ++k) cnt += pos[k] != MAP_ABSENT;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const unsigned keep = __ballot_sync(0xffffffffu, pos[k] != MAP_ABSENT);
            if (pos[k] != MAP_ABSENT) {
              const i64 w = o + __popc(keep & ((1u << lane) - 1u));
              out_ids[w] = (i64)pos[k];
              out_sel[w] = e0 + 32 * k + lane;
              if (out_seg) out_seg[w] = seg;
            }
            o += __popc(keep);
          }
        }
      }
    }
    if (!FILL) {
#pragma unroll
      for (int dd = 16; dd > 0; dd >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, dd);
      if (lane == 0) vcnt[v] = (u32)cnt;
    }
  }
}

__global__ void __launch_bounds__(1024)
colrow_offsets_kernel(const i64* __restrict__ col_ptr, int B, i64 S, const i64* __restrict__ vptr,
                      const u32* __restrict__ vcnt, i64* __restrict__ voff, i64* __restrict__ out_indptr) {
  __shared__ i64 s_scan[34];
  const i64 nseg = col_ptr[B] < S ? col_ptr[B] : S;
  const i64 V = nseg > 0 ? vptr[nseg] : 0;
  cta_exclusive_scan(V, [&](i64 v) { return (i64)vcnt[v]; }, voff, s_scan);
  __syncthreads();  // voff is this CTA's own global writes
  for (i64 s = threadIdx.x; s <= nseg; s += 1024) out_indptr[s] = voff[s < nseg ? vptr[s] : V];
}

struct ColRowLayout {
  size_t total_entries, table, deg, vptr, vcnt, voff, total;
  i64 slots, parts;
};

static ColRowLayout colrow_layout(i64 S, i64 R, i64 B) {
  ColRowLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.slots = 2 * R + 32 * (B + 1);
  L.parts = S + CR_EXTRA_PARTS + 1;
  size_t o = 0;
  L.total_entries = o; o = up(o + 256);
  L.table = o; o = up(o + sizeof(u64) * (size_t)L.slots);
  L.deg = o; o = up(o + sizeof(i64) * (size_t)(S + 1));
  L.vptr = o; o = up(o + sizeof(i64) * (size_t)(S + 1));
  L.vcnt = o; o = up(o + sizeof(u32) * (size_t)L.parts);
  L.voff = o; o = up(o + sizeof(i64) * (size_t)(L.parts + 1));
  L.total = o;
  return L;
}

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_slice_across_workspace_bytes(int64_t nnz_max, int64_t id_bound) {
  if (nnz_max < 0 || id_bound < 0) return 0;
  return across_layout(nnz_max, id_bound, true).total;
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
  const AcrossLayout L = across_layout(nnz_max, id_bound, true);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  int rc = build_map(ws, L, (const i64*)ids, R, id_bound, d_err, st);
  if (rc != GSB_OK) return rc;
  {
    i64 g = (id_bound + 255) / 256; if (g > sm_count() * 16) g = sm_count() * 16; if (g < 1) g = 1;
    LaunchScope ls(KID_SLICE_ROWS, st);
    bits_build_kernel<<<(int)g, 256, 0, st>>>((const u32*)(ws + L.map), id_bound, (u32*)(ws + L.bits));
  }
  const int tiles = nnz_max == 0 ? 1 : ceil_div_i(nnz_max, AC_TILE);
  {
    LaunchScope ls(KID_SLICE_ROWS, st);
    if (indices_dtype == GSB_I32)
      across_mark_kernel<int><<<tiles, RS_THREADS, 0, st>>>(
          (const i64*)indptr, indices, nseg, nnz_max, (const u32*)(ws + L.bits), id_bound,
          (unsigned char*)(ws + L.nib), (unsigned short*)(ws + L.toff), (u32*)(ws + L.tile_total), d_err);
    else
      across_mark_kernel<i64><<<tiles, RS_THREADS, 0, st>>>(
          (const i64*)indptr, indices, nseg, nnz_max, (const u32*)(ws + L.bits), id_bound,
          (unsigned char*)(ws + L.nib), (unsigned short*)(ws + L.toff), (u32*)(ws + L.tile_total), d_err);
  }
  {
    LaunchScope ls(KID_SLICE_ROWS, st);
    tile_scan_kernel<<<1, 1024, 0, st>>>((const i64*)indptr, nseg, nnz_max, (const u32*)(ws + L.tile_total),
                                         (i64*)(ws + L.tile_base));
  }
  {
    i64 g = (nseg + 256) / 256; if (g > sm_count() * 16) g = sm_count() * 16;
    LaunchScope ls(KID_SLICE_ROWS, st);
    across_offsets_kernel<<<(int)g, 256, 0, st>>>((const i64*)indptr, nseg, nnz_max,
                                                 (const unsigned char*)(ws + L.nib),
                                                 (const unsigned short*)(ws + L.toff),
                                                 (const i64*)(ws + L.tile_base), (i64*)out_indptr);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_slice_across_fill(const int64_t* indptr, const void* indices, int indices_dtype,
                                     int64_t nseg, int64_t nnz_max, int64_t id_bound,
                                     int64_t* out_ids, int64_t* out_seg, int64_t* out_sel,
                                     void* workspace, size_t workspace_bytes, int* d_err,
                                     void* cuda_stream) {
  (void)d_err;
  if (nseg == 0 || nnz_max == 0) return GSB_OK;
  if (!indptr || !indices || !out_ids || !out_sel || !workspace || nseg < 0 || nnz_max < 0)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  const AcrossLayout L = across_layout(nnz_max, id_bound, true);
  if (workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  const int tiles = ceil_div_i(nnz_max, AC_TILE);
  if (out_seg) {
    const i64 n_tiles = (i64)tiles + 1;
    LaunchScope ls(KID_SLICE_ROWS, st);
    tile_segment_kernel<<<(int)((n_tiles + 255) / 256), 256, 0, st>>>((const i64*)indptr, nseg, n_tiles,
                                                                      (i64*)(ws + L.tile_seg));
  }
  LaunchScope ls(KID_SLICE_ROWS, st);
  if (indices_dtype == GSB_I32)
    across_fill_kernel<int><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, nseg, nnz_max, (const u32*)(ws + L.map),
        (const unsigned char*)(ws + L.nib), (const unsigned short*)(ws + L.toff),
        (const i64*)(ws + L.tile_base), (const i64*)(ws + L.tile_seg), (i64*)out_ids, (i64*)out_seg,
        (i64*)out_sel);
  else
    across_fill_kernel<i64><<<tiles, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, nseg, nnz_max, (const u32*)(ws + L.map),
        (const unsigned char*)(ws + L.nib), (const unsigned short*)(ws + L.toff),
        (const i64*)(ws + L.tile_base), (const i64*)(ws + L.tile_seg), (i64*)out_ids, (i64*)out_seg,
        (i64*)out_sel);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" size_t gsb_coo_filter_workspace_bytes(int64_t nnz, int64_t id_bound) {
  if (nnz < 0 || id_bound < 0) return 0;
  return across_layout(nnz, id_bound, false).total;
}

extern "C" int gsb_coo_filter(const int64_t* key, const int64_t* other, int64_t nnz,
                              const int64_t* ids, int64_t R, int64_t id_bound, int64_t* out_key,
                              int64_t* out_other, int64_t* out_sel, int64_t* d_count,
                              void* workspace, size_t workspace_bytes, int* d_err,
                              void* cuda_stream) {
  if (nnz < 0 || R < 0 || id_bound < 0 || !d_count || (R > 0 && !ids)) return GSB_ERR_INVALID;
  if (nnz > 0 && (!key || !other || !out_key || !out_other || !out_sel)) return GSB_ERR_INVALID;
  if (R >= 0xFFFFFFFFll || id_bound > (1ll << 33)) return GSB_ERR_UNSUPPORTED;
  const AcrossLayout L = across_layout(nnz, id_bound, false);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  int rc = build_map(ws, L, (const i64*)ids, R, id_bound, d_err, st);
  if (rc != GSB_OK) return rc;
  const int tiles = nnz == 0 ? 1 : ceil_div_i(nnz, AC_TILE);
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
  GSB_CUDA_OK(cudaMemsetAsync(ws, 0, L.table, st));                                     // entry total
  GSB_CUDA_OK(cudaMemsetAsync(ws + L.table, 0xFF, sizeof(u64) * (size_t)L.slots, st));  // empty slots
  if (R > 0) {
    i64 g = (R + 255) / 256; if (g > sm_count() * 16) g = sm_count() * 16;
    LaunchScope ls(KID_SLICE_ROWS, st);
    rowtab_insert_kernel<<<(int)g, 256, 0, st>>>((const i64*)rows, (const i64*)row_ptr, (int)B,
                                                 (u64*)(ws + L.table), d_err);
  }
  i64* deg = (i64*)(ws + L.deg);
  i64* vptr = (i64*)(ws + L.vptr);
  unsigned long long* total = (unsigned long long*)(ws + L.total_entries);
  {
    LaunchScope ls(KID_SLICE_ROWS, st);
    colrow_deg_kernel<<<S == 0 ? 1 : ceil_div_i(S, 256), 256, 0, st>>>(
        (const i64*)indptr, num_cols, (const i64*)cols, (const i64*)col_ptr, (int)B, S, deg, total, d_err);
  }
  {
    LaunchScope ls(KID_SLICE_ROWS, st);
    colrow_parts_kernel<<<1, 1024, 0, st>>>((const i64*)col_ptr, (int)B, S, deg, total, vptr);
  }
  if (S > 0) {
    i64 g = (L.parts + RS_WARPS - 1) / RS_WARPS; if (g > sm_count() * 16) g = sm_count() * 16;
    LaunchScope ls(KID_SLICE_ROWS, st);
    if (indices_dtype == GSB_I32)
      colrow_part_kernel<int, false><<<(int)g, RS_THREADS, 0, st>>>(
          (const i64*)indptr, indices, (const i64*)cols, (const i64*)col_ptr, (const i64*)row_ptr, (int)B,
          S, (const u64*)(ws + L.table), deg, total, vptr, (u32*)(ws + L.vcnt), nullptr, nullptr,
          nullptr, nullptr);
    else
      colrow_part_kernel<i64, false><<<(int)g, RS_THREADS, 0, st>>>(
          (const i64*)indptr, indices, (const i64*)cols, (const i64*)col_ptr, (const i64*)row_ptr, (int)B,
          S, (const u64*)(ws + L.table), deg, total, vptr, (u32*)(ws + L.vcnt), nullptr, nullptr,
          nullptr, nullptr);
  }
  {
    LaunchScope ls(KID_SLICE_ROWS, st);
    colrow_offsets_kernel<<<1, 1024, 0, st>>>((const i64*)col_ptr, (int)B, S, vptr,
                                              (const u32*)(ws + L.vcnt), (i64*)(ws + L.voff),
                                              (i64*)out_indptr);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_slice_cols_rows_fill(const int64_t* indptr, const void* indices,
                                        int indices_dtype, int64_t num_cols, const int64_t* cols,
                                        const int64_t* col_ptr, int64_t S, const int64_t* row_ptr,
                                        int64_t R, int64_t B, const int64_t* out_indptr,
                                        int64_t* out_ids, int64_t* out_seg, int64_t* out_sel,
                                        const void* workspace, void* cuda_stream) {
  (void)num_cols;
  if (S == 0) return GSB_OK;
  if (!indptr || !indices || !cols || !col_ptr || !row_ptr || !out_indptr || !out_ids || !out_sel ||
      !workspace || S < 0 || B < 1)
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  const ColRowLayout L = colrow_layout(S, R, B);
  cudaStream_t st = (cudaStream_t)cuda_stream;
  const char* ws = (const char*)workspace;
  i64 g = (L.parts + RS_WARPS - 1) / RS_WARPS; if (g > sm_count() * 16) g = sm_count() * 16;
  LaunchScope ls(KID_SLICE_ROWS, st);
  if (indices_dtype == GSB_I32)
    colrow_part_kernel<int, true><<<(int)g, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, (const i64*)cols, (const i64*)col_ptr, (const i64*)row_ptr, (int)B, S,
        (const u64*)(ws + L.table), (const i64*)(ws + L.deg), (const unsigned long long*)(ws + L.total_entries),
        (const i64*)(ws + L.vptr), nullptr, (const i64*)(ws + L.voff), (i64*)out_ids, (i64*)out_seg,
        (i64*)out_sel);
  else
    colrow_part_kernel<i64, true><<<(int)g, RS_THREADS, 0, st>>>(
        (const i64*)indptr, indices, (const i64*)cols, (const i64*)col_ptr, (const i64*)row_ptr, (int)B, S,
        (const u64*)(ws + L.table), (const i64*)(ws + L.deg), (const unsigned long long*)(ws + L.total_entries),
        (const i64*)(ws + L.vptr), nullptr, (const i64*)(ws + L.voff), (i64*)out_ids, (i64*)out_seg,
        (i64*)out_sel);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
