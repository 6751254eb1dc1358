// Weighted per-column sampling.
//
// Without replacement: every edge e of a column gets the key log2(u_e)/p_e
// (the logarithm of the A-Res key u^(1/p)); the K largest keys win.  A warp
// owns a column.  u_e is draw e of the column slot's counter-based stream, so a
// key can be recomputed at any time: columns of up to WP_CACHE entries compute
// their keys once into the warp's shared-memory cache, longer ones recompute
// them in every pass and need no scratch proportional to the degree.  The K-th
// largest key is found by a 4-pass radix select (8 bits per pass, per-warp
// histogram in shared memory); a last pass writes the winners in column order,
// ties on the threshold key going to the lowest positions.  No sort, no limit
// of 32 on K.
//
// With replacement: K independent draws from the column's distribution by
// streaming the running sum through the warp (no materialised CDF).
#include "gsb_common.cuh"

namespace gsb {

constexpr int WP_WARPS = 4;
constexpr int WP_THREADS = WP_WARPS * 32;
constexpr int WP_MAX_K = 1024;
constexpr int WP_CACHE = 1024;  // keys a warp caches (4 KB of shared memory per warp)

struct ProbParams {
  const i64* indptr;
  const void* indices;
  const float* probs;
  const i64* seeds;
  i64 S_max;
  const i64* d_S;
  int K;
  int replace;
  u64 seed;
  u32 stream;
  const i64* sub_indptr;
  i64* out_rows;
  i64* out_cols;
  i64* out_sel;
  i64 E_cap;
  int* err;
  int thread_path;       // columns of at most WT_MAX_DEG entries are handled by the thread kernel
  int short_rounds;      // ... which orders groups of this many tiles by column length
  const i64* slot_start;  // [S] first entry of the slot's column   } by-products of
  const u32* slot_deg;    // [S] its length                          } the count pass
  const i64* list;        // slots the warp kernel has to process (unordered)
  const int* list_n;
  i64* long_list;  // filled by the warp kernel: the columns it leaves to the CTA kernel
  int* long_n;
};

__device__ __forceinline__ u32 orderable(float f) {
  u32 b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// key of edge e (position inside the column) of column slot `slot`
__device__ __forceinline__ u32 ares_key(u32 draw, float p) {
  if (!(p > 0.f)) return 0u;  // never preferred; below every finite key
  const float u = ((float)draw + 1.0f) * 2.3283064365386963e-10f;  // (0,1]
  const float k = __log2f(u) / p;
  const u32 o = orderable(k);
  return o == 0u ? 1u : o;
}

// Short columns (K < degree <= WT_MAX_DEG) with a small K: THREAD per column.  The thread
// streams its column once, keeping the K largest keys seen so far in a shared-memory array
// (transposed: bank = thread); a new key replaces the current smallest only when it is
// strictly larger, and among equal smallest keys the one at the highest position leaves, so
// the winners are the K largest keys with ties going to the lowest positions -- the same set
// the warp kernel selects.  About 30 instructions per entry instead of a warp's several
// hundred per column.  Longer columns and larger K stay with the warp kernel.
constexpr int WT_THREADS = 128;
#ifndef GSB_WT_MAX_DEG
#define GSB_WT_MAX_DEG 128
#endif
constexpr int WT_MAX_DEG = GSB_WT_MAX_DEG;
constexpr int WT_MAX_K = 32;
#ifndef GSB_WT_BATCH
#define GSB_WT_BATCH 8
#endif
// Tiles of WT_THREADS columns ordered together (at most; fewer on small inputs).  Ordering by
// length makes the lanes of a warp agree, but neighbouring lanes then read weights from places
// far apart instead of from one contiguous stretch of the slice, and the wider the group the
// further apart: 3.7 M columns at K = 5 take 1.08 ms with groups of 1 tile, 0.95 with 2,
// 1.07 with 4, 1.26 with 8.
#ifndef GSB_WT_ROUNDS
#define GSB_WT_ROUNDS 2
#endif
constexpr int WT_ROUNDS = GSB_WT_ROUNDS;
constexpr int WT_BATCH = GSB_WT_BATCH;  // keys computed together: 8 (two Philox blocks) or 4 (one)
static_assert(WT_BATCH == 4 || WT_BATCH == 8, "whole Philox blocks");

// No minimum number of CTAs per SM is stated on purpose: left alone the compiler settles on 64
// registers (8 CTAs per SM, 1.08 ms for 3.7 M columns at K = 5); a stated minimum of 1 lets it
// take 83 (6 CTAs, 1.49 ms), one of 10 forces 48 with spills (1.43 ms).
#ifdef GSB_WT_MIN_CTAS
#define GSB_WT_BOUNDS __launch_bounds__(WT_THREADS, GSB_WT_MIN_CTAS)
#else
#define GSB_WT_BOUNDS __launch_bounds__(WT_THREADS)
#endif
template <typename IndexT>
__global__ void GSB_WT_BOUNDS sample_probs_thread_kernel(const ProbParams p) {
  extern __shared__ u32 s_top[];  // keys[K][WT_THREADS], then positions[K][WT_THREADS]
  __shared__ u32 s_hist[WT_MAX_DEG + 2];  // columns of each length in the tile, then first place of the length
  __shared__ unsigned short s_order[WT_THREADS * WT_ROUNDS];  // the group's columns by ascending length
  __shared__ i64 s_scan[34];
  const int K = p.K;
  u32* tkey = s_top + threadIdx.x;
  u32* tpos = s_top + K * WT_THREADS + threadIdx.x;
  i64 S = p.S_max;
  if (p.d_S) { i64 live = *p.d_S; S = live < S ? (live < 0 ? 0 : live) : S; }
  const int rounds = p.short_rounds;  // 1 .. WT_ROUNDS
  const i64 group = (i64)WT_THREADS * rounds;
  for (i64 g0 = (i64)blockIdx.x * group; g0 < S; g0 += (i64)gridDim.x * group) {
    // The trip count of the selection loop is the column's length, and a warp runs as long as
    // its longest column.  The CTA therefore takes a group of `rounds` x WT_THREADS consecutive
    // columns, orders them by length (a counting sort in shared memory) and goes through the
    // order in `rounds` rounds of WT_THREADS neighbours: the lanes of a warp finish together,
    // and the warps of a round get columns of similar lengths.
    for (int i = threadIdx.x; i < WT_MAX_DEG + 2; i += WT_THREADS) s_hist[i] = 0;
    __syncthreads();
    u32 len_sub[WT_ROUNDS];  // per round: length (low 8 bits; 0 = not selected from by this kernel) | place among equals
#pragma unroll
    for (int r = 0; r < WT_ROUNDS; ++r) {
      len_sub[r] = 0;
      if (r < rounds) {
        const i64 slot0 = g0 + (i64)r * WT_THREADS + threadIdx.x;
        u32 len = 0;
        if (slot0 < S) {
          const u32 dg = p.slot_deg[slot0];
          if ((i64)dg > K && dg <= (u32)WT_MAX_DEG) len = dg;
        }
        len_sub[r] = len | (atomicAdd(&s_hist[len], 1u) << 8);
      }
    }
    __syncthreads();
    {  // exclusive running sum over the lengths 0 .. WT_MAX_DEG (at most WT_THREADS + 1 values: two per thread)
      const int i0 = 2 * threadIdx.x, i1 = i0 + 1;
      const u32 h0 = i0 <= WT_MAX_DEG ? s_hist[i0] : 0u, h1 = i1 <= WT_MAX_DEG ? s_hist[i1] : 0u;
      i64 total;
      const i64 ex = block_exclusive_scan((i64)(h0 + h1), s_scan, &total);
      if (i0 <= WT_MAX_DEG) s_hist[i0] = (u32)ex;
      if (i1 <= WT_MAX_DEG) s_hist[i1] = (u32)ex + h0;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < WT_ROUNDS; ++r)
      if (r < rounds) s_order[s_hist[len_sub[r] & 0xFFu] + (len_sub[r] >> 8)] = (unsigned short)(r * WT_THREADS + threadIdx.x);
    __syncthreads();
    for (int r = 0; r < rounds; ++r) {
    const i64 slot = g0 + s_order[r * WT_THREADS + threadIdx.x];
    if (slot >= S) continue;
    const i64 in_start = p.slot_start[slot];
    const i64 deg = (i64)p.slot_deg[slot];
    if (deg == 0 || deg > WT_MAX_DEG) continue;  // nothing to do / the warp kernel's column
    const i64 out_start = p.sub_indptr[slot];
    if (out_start + (deg < K ? deg : K) > p.E_cap) { raise(p.err, ERRBIT_CAPACITY); continue; }
    if (deg <= K) {  // the whole column
      for (i64 k = 0; k < deg; ++k) {
        p.out_rows[out_start + k] = load_index<IndexT>(p.indices, in_start + k);
        p.out_sel[out_start + k] = in_start + k;
        if (p.out_cols) p.out_cols[out_start + k] = slot;
      }
      continue;
    }
    const float* pr = p.probs + in_start;
    const int d = (int)deg;
    u32 kmin = 0, pmin = 0;
    int imin = 0;
    // eight keys at a time: the two Philox blocks and the eight log2/divide chains are independent
    // of each other, so they overlap; the top-K update below stays in entry order.  The weights
    // of the next eight entries are requested before this batch's keys are computed, so that
    // their latency hides behind the arithmetic.
    float w[WT_BATCH];
#pragma unroll
    for (int j = 0; j < WT_BATCH; ++j) w[j] = j < d ? __ldg(pr + j) : 0.f;
    for (int e0 = 0; e0 < d; e0 += WT_BATCH) {
      float wn[WT_BATCH];
#pragma unroll
      for (int j = 0; j < WT_BATCH; ++j) wn[j] = e0 + WT_BATCH + j < d ? __ldg(pr + e0 + WT_BATCH + j) : 0.f;
      const Philox4 b0 = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
      Philox4 b1 = b0;
      if (WT_BATCH > 4 && e0 + 4 < d) b1 = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2) + 1u);
      u32 keys[WT_BATCH];
#pragma unroll
      for (int j = 0; j < WT_BATCH; ++j)
        keys[j] = e0 + j < d ? ares_key(pick_word(j < 4 ? b0 : b1, j & 3), w[j]) : 0u;
#pragma unroll
      for (int j = 0; j < WT_BATCH; ++j) w[j] = wn[j];
#pragma unroll
      for (int j = 0; j < WT_BATCH; ++j) {
      const int e = e0 + j;
      if (e >= d) break;
      const u32 key = keys[j];
      if (e < K) {
        tkey[e * WT_THREADS] = key;
        tpos[e * WT_THREADS] = (u32)e;
        if (e == 0 || key <= kmin) { kmin = key; pmin = (u32)e; imin = e; }  // <=: later position leaves first
      } else if (key > kmin) {
        tkey[imin * WT_THREADS] = key;
        tpos[imin * WT_THREADS] = (u32)e;
        // new smallest: least key, the highest position among equals
        kmin = tkey[0]; pmin = tpos[0]; imin = 0;
        for (int t = 1; t < K; ++t) {
          const u32 kt = tkey[t * WT_THREADS], pt = tpos[t * WT_THREADS];
          if (kt < kmin || (kt == kmin && pt > pmin)) { kmin = kt; pmin = pt; imin = t; }
        }
      }
      }
    }
    // winners in column order: repeatedly take the smallest remaining position (the ordered
    // positions go where the keys were) ...
    u32 last = 0;
    for (int k = 0; k < K; ++k) {
      u32 best = 0xFFFFFFFFu;
      for (int j = 0; j < K; ++j) {
        const u32 pj = tpos[j * WT_THREADS];
        if (pj < best && (k == 0 || pj > last)) best = pj;
      }
      last = best;
      tkey[k * WT_THREADS] = best;
    }
    // ... then the gathers of the winners' row ids, four in flight at a time
    for (int k0 = 0; k0 < K; k0 += 4) {
      i64 e[4], r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        e[j] = in_start + (k0 + j < K ? tkey[(k0 + j) * WT_THREADS] : 0u);
        r[j] = k0 + j < K ? load_index<IndexT>(p.indices, e[j]) : 0;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (k0 + j < K) {
          p.out_rows[out_start + k0 + j] = r[j];
          p.out_sel[out_start + k0 + j] = e[j];
          if (p.out_cols) p.out_cols[out_start + k0 + j] = slot;
        }
      }
    }
    }
    __syncthreads();  // the next group rewrites the order
  }
}

// In-place bitonic sort, descending, of a[0..n) in shared memory (n a power of two) by the CTA.
template <typename T>
__device__ __forceinline__ void cta_sort_desc(T* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int o = i ^ j;
        if (o > i) {
          const T x = a[i], y = a[o];
          if (((i & k) == 0) ? (x < y) : (x > y)) { a[i] = y; a[o] = x; }
        }
      }
      __syncthreads();
    }
  }
}

// Very long columns (more than WB_MIN_DEG entries): one CTA per column, same radix select and
// ordered emit as the warp kernel but with the histogram shared by 256 threads and block scans
// for the tie ranks and output offsets.  Keeps a hub column from being the tail of the launch.
// That is five passes over the column (keys are recomputed, not stored).  For K <= 256 two passes
// usually do: pass A leaves every thread's largest key, and the K-th largest of those 256 values
// is a lower bound L of the K-th largest key overall (K different entries reach it); pass B
// collects the entries with key >= L -- about K of them -- into shared memory, where a sort by
// (key descending, position ascending) gives exactly the winners of the radix select, ties
// included.  More than WB_CAND candidates (many equal keys, e.g. zero weights) -> the five-pass form.
// With the two-pass form a CTA is the faster owner of every column the warp kernel cannot cache
// in shared memory (sum of the two kernels on 3.7 M columns: 0.95 ms with the border at 4096
// entries, 0.72 at 2048, 0.59 at 1024, 0.72 at 512), eight CTAs per SM.
constexpr int WB_THREADS = 256;
#ifndef GSB_WB_MIN_DEG
#define GSB_WB_MIN_DEG 1024
#endif
#ifndef GSB_WB_CTAS_PER_SM
#define GSB_WB_CTAS_PER_SM 8
#endif
constexpr int WB_MIN_DEG = GSB_WB_MIN_DEG;
constexpr int WB_CAND = 2048;

template <typename IndexT>
__global__ void __launch_bounds__(WB_THREADS) sample_probs_block_kernel(const ProbParams p) {
  __shared__ u32 s_hist[256];
  __shared__ i64 s_scan[34];
  __shared__ u32 s_digit, s_above;
  __shared__ u32 s_top[WB_THREADS];
  __shared__ u64 s_cand[WB_CAND];
  __shared__ int s_ncand, s_nhit;
  __shared__ int s_hits[WB_THREADS];  // threads whose largest key reaches the bound
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  i64 S = p.S_max;
  if (p.d_S) { i64 live = *p.d_S; S = live < S ? (live < 0 ? 0 : live) : S; }
  const int K = p.K;
  const i64 n_listed = *p.long_n;
  for (i64 w = blockIdx.x; w < n_listed; w += gridDim.x) {
    const i64 slot = p.long_list[w];
    if (slot >= S) continue;
    const i64 in_start = p.slot_start[slot];
    const i64 deg = (i64)p.slot_deg[slot];
    const i64 out_start = p.sub_indptr[slot];
    if (out_start + K > p.E_cap) { if (threadIdx.x == 0) raise(p.err, ERRBIT_CAPACITY); continue; }
    const float* pr = p.probs + in_start;
    bool done = false;
    if (K <= WB_THREADS) {
      u32 mine = 0;  // pass A: this thread's largest key
      for (i64 e0 = (i64)threadIdx.x * 4; e0 < deg; e0 += WB_THREADS * 4) {
        const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (e0 + j < deg) {
            const u32 key = ares_key(pick_word(blk, j), __ldg(pr + e0 + j));
            mine = key > mine ? key : mine;
          }
        }
      }
      __syncthreads();  // the previous column's readers of s_top / s_cand
      s_top[threadIdx.x] = mine;
      if (threadIdx.x == 0) { s_ncand = 0; s_nhit = 0; }
      __syncthreads();
      cta_sort_desc(s_top, WB_THREADS);
      const u32 bound = s_top[K - 1];
      if (bound > 0u) {  // pass B: the entries that can still win (0 = weights <= 0 are in play)
        // Only a thread whose own largest key reaches the bound has such entries (about K of the
        // WB_THREADS threads): the strides of those threads are rescanned, by all threads together
        // -- one Philox block of four entries per thread and step -- instead of the whole column.
        if (mine >= bound) s_hits[atomicAdd(&s_nhit, 1)] = threadIdx.x;
        __syncthreads();
        const i64 per_thread = (deg + WB_THREADS * 4 - 1) / (WB_THREADS * 4);  // Philox blocks of one thread's stride
        const i64 todo = (i64)s_nhit * per_thread;
        for (i64 q = threadIdx.x; q < todo; q += WB_THREADS) {
          const i64 e0 = (i64)s_hits[q / per_thread] * 4 + (q % per_thread) * (WB_THREADS * 4);
          if (e0 >= deg) continue;
          const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (e0 + j < deg) {
              const u32 key = ares_key(pick_word(blk, j), __ldg(pr + e0 + j));
              if (key >= bound) {
                const int at = atomicAdd(&s_ncand, 1);
                if (at < WB_CAND) s_cand[at] = ((u64)key << 32) | (u64)(~(u32)(e0 + j));  // ~pos: low position first
              }
            }
          }
        }
      }
      __syncthreads();
      const int ncand = s_ncand;
      if (bound > 0u && ncand <= WB_CAND) {  // ncand >= K: K threads' maxima reach the bound
        int n2 = 2;
        while (n2 < ncand) n2 <<= 1;
        for (int i = ncand + threadIdx.x; i < n2; i += WB_THREADS) s_cand[i] = 0ull;
        __syncthreads();
        cta_sort_desc(s_cand, n2);
        // the first K are the winners; emit them in column order (sort ~pos descending)
        int k2 = 2;
        while (k2 < K) k2 <<= 1;
        const u32 inv = threadIdx.x < K ? (u32)s_cand[threadIdx.x] : 0u;
        __syncthreads();
        s_top[threadIdx.x] = inv;
        __syncthreads();
        cta_sort_desc(s_top, k2);
        if (threadIdx.x < K) {
          const i64 e = in_start + (i64)(~s_top[threadIdx.x]);
          p.out_rows[out_start + threadIdx.x] = load_index<IndexT>(p.indices, e);
          p.out_sel[out_start + threadIdx.x] = e;
          if (p.out_cols) p.out_cols[out_start + threadIdx.x] = slot;
        }
        done = true;
      }
    }
    __syncthreads();
    if (done) continue;
    u32 prefix = 0, prefix_mask = 0;
    u32 remaining = (u32)K;
    for (int shift = 24; shift >= 0; shift -= 8) {
      s_hist[threadIdx.x] = 0;
      __syncthreads();
      for (i64 e0 = (i64)threadIdx.x * 4; e0 < deg; e0 += WB_THREADS * 4) {
        const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (e0 + j < deg) {
            const u32 key = ares_key(pick_word(blk, j), __ldg(pr + e0 + j));
            if ((key & prefix_mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
          }
        }
      }
      __syncthreads();
      if (wid == 0) {  // walk the buckets from the top: lane owns 8 buckets
        u32 mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mine += s_hist[255 - (lane * 8 + j)];
        u32 inc = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          u32 t = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += t;
        }
        const u32 exc = inc - mine;
        const unsigned hit = __ballot_sync(0xffffffffu, inc >= remaining);
        const int owner = __ffs(hit) - 1;
        if (lane == owner) {
          u32 run = exc;
          for (int j = 0; j < 8; ++j) {
            const u32 h = s_hist[255 - (lane * 8 + j)];
            if (run + h >= remaining) { s_digit = 255u - (u32)(lane * 8 + j); s_above = run; break; }
            run += h;
          }
        }
      }
      __syncthreads();
      remaining -= s_above;
      prefix |= s_digit << shift;
      prefix_mask |= 255u << shift;
      __syncthreads();
    }
    const u32 thr = prefix;
    i64 ties_left = remaining;  // keys equal to the threshold still to take, lowest positions first
    i64 written = 0;
    for (i64 base = 0; base < deg; base += WB_THREADS * 4) {
      const i64 e0 = base + (i64)threadIdx.x * 4;
      u32 keys[4];
      int ntie = 0;
      if (e0 < deg) {
        const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          keys[j] = e0 + j < deg ? ares_key(pick_word(blk, j), __ldg(pr + e0 + j)) : 0u;
          if (e0 + j < deg && keys[j] == thr) ++ntie;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) keys[j] = 0u;
      }
      i64 chunk_ties;
      i64 tie_rank = block_exclusive_scan((i64)ntie, s_scan, &chunk_ties);
      __syncthreads();
      bool take[4];
      int ntake = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        take[j] = false;
        if (e0 + j < deg) {
          if (keys[j] > thr) take[j] = true;
          else if (keys[j] == thr) { take[j] = tie_rank < ties_left; ++tie_rank; }
        }
        ntake += take[j] ? 1 : 0;
      }
      i64 chunk_take;
      i64 o = out_start + written + block_exclusive_scan((i64)ntake, s_scan, &chunk_take);
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (take[j]) {
          p.out_rows[o] = load_index<IndexT>(p.indices, in_start + e0 + j);
          p.out_sel[o] = in_start + e0 + j;
          if (p.out_cols) p.out_cols[o] = slot;
          ++o;
        }
      }
      written += chunk_take;
      ties_left -= chunk_ties < ties_left ? chunk_ties : ties_left;
    }
    __syncthreads();
  }
}

template <typename IndexT>
__global__ void __launch_bounds__(WP_THREADS) sample_probs_kernel(const ProbParams p) {
  extern __shared__ u32 s_dyn[];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  u32* hist = s_dyn + wid * 256;
  float* targets = reinterpret_cast<float*>(s_dyn + WP_WARPS * 256) + wid * p.K;
  u32* kcache = s_dyn + WP_WARPS * 256 + WP_WARPS * p.K + wid * WP_CACHE;
  i64 S = p.S_max;
  if (p.d_S) { i64 live = *p.d_S; S = live < S ? (live < 0 ? 0 : live) : S; }
  const int K = p.K;
  const i64 n_listed = *p.list_n;
  for (i64 w = (i64)blockIdx.x * WP_WARPS + wid; w < n_listed; w += (i64)gridDim.x * WP_WARPS) {
    const i64 slot = p.list[w];
    if (slot >= S) continue;
    const i64 in_start = p.slot_start[slot];
    const i64 deg = (i64)p.slot_deg[slot];
    if (!p.replace && deg > WB_MIN_DEG && deg > K) {  // the block kernel's column
      if (lane == 0) p.long_list[atomicAdd(p.long_n, 1)] = slot;
      continue;
    }
    const i64 out_start = p.sub_indptr[slot];
    const i64 cnt = p.sub_indptr[slot + 1] - out_start;
    if (cnt == 0) continue;
    if (out_start + cnt > p.E_cap) { if (lane == 0) raise(p.err, ERRBIT_CAPACITY); continue; }
    const float* pr = p.probs + in_start;
    if (!p.replace && deg <= K) {
      for (i64 k = lane; k < deg; k += 32) {
        p.out_rows[out_start + k] = load_index<IndexT>(p.indices, in_start + k);
        p.out_sel[out_start + k] = in_start + k;
        if (p.out_cols) p.out_cols[out_start + k] = slot;
      }
      continue;
    }
    if (!p.replace) {
      // ---- radix select of the K-th largest key
      const bool cached = deg <= WP_CACHE;
      if (cached) {
        for (i64 e0 = (i64)lane * 4; e0 < deg; e0 += 128) {
          const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (e0 + j < deg) kcache[e0 + j] = ares_key(pick_word(blk, j), __ldg(pr + e0 + j));
        }
        __syncwarp();
      }
      // Short column, small K: K rounds of "largest remaining key" (ties to the lowest
      // position) instead of the radix select -- a few hundred instead of about a thousand
      // warp instructions for a typical column.  Same winners, written in column order.
      const int nchunk = (int)((deg + 31) >> 5);
      if (cached && K * (nchunk * 6 + 40) < 4 * (nchunk * 8 + 120)) {
        u32 taken = 0;  // bit i: entry lane + 32 i of this column is a winner
        for (int r = 0; r < K; ++r) {
          u32 bk = 0;
          int bp = -1;
          for (int i = 0; i < nchunk; ++i) {
            const int e = lane + (i << 5);
            if (e < (int)deg && !((taken >> i) & 1u)) {
              const u32 k = kcache[e];
              if (bp < 0 || k > bk) { bk = k; bp = e; }
            }
          }
          // warp argmax of (key, lowest position); lanes with nothing left offer 0
          u64 best = bp < 0 ? 0ull : (((u64)bk + 1ull) << 32) | (u64)(0xFFFFFFFFu - (u32)bp);
#pragma unroll
          for (int d = 16; d > 0; d >>= 1) {
            const u64 o = __shfl_xor_sync(0xffffffffu, best, d);
            best = o > best ? o : best;
          }
          const int win = (int)(0xFFFFFFFFu - (u32)best);
          if ((win & 31) == lane) taken |= 1u << (win >> 5);
        }
        i64 o = out_start;
        for (int i = 0; i < nchunk; ++i) {
          const bool take = (taken >> i) & 1u;
          const unsigned bal = __ballot_sync(0xffffffffu, take);
          if (take) {
            const i64 e = in_start + lane + (i << 5);
            const i64 w = o + __popc(bal & ((1u << lane) - 1u));
            p.out_rows[w] = load_index<IndexT>(p.indices, e);
            p.out_sel[w] = e;
            if (p.out_cols) p.out_cols[w] = slot;
          }
          o += __popc(bal);
        }
        continue;
      }
      u32 prefix = 0, prefix_mask = 0;
      u32 remaining = (u32)K;  // rank (1 = largest) still to locate inside the prefix class
      for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = lane; i < 256; i += 32) hist[i] = 0;
        __syncwarp();
        if (cached) {
          for (int e = lane; e < (int)deg; e += 32) {
            const u32 key = kcache[e];
            if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
          }
        } else {
          for (i64 e0 = (i64)lane * 4; e0 < deg; e0 += 128) {
            const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (e0 + j < deg) {
                const u32 key = ares_key(pick_word(blk, j), __ldg(pr + e0 + j));
                if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
              }
            }
          }
        }
        __syncwarp();
        // walk the buckets from the top: lane owns 8 buckets
        u32 mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mine += hist[255 - (lane * 8 + j)];
        u32 inc = mine;  // inclusive scan over lanes (lane 0 = top buckets)
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          u32 t = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += t;
        }
        const u32 exc = inc - mine;
        const unsigned hit = __ballot_sync(0xffffffffu, inc >= remaining);
        const int owner = __ffs(hit) - 1;
        u32 digit = 0, above = 0;
        if (lane == owner) {
          u32 run = exc;
          for (int j = 0; j < 8; ++j) {
            const u32 h = hist[255 - (lane * 8 + j)];
            if (run + h >= remaining) { digit = 255u - (u32)(lane * 8 + j); above = run; break; }
            run += h;
          }
        }
        digit = __shfl_sync(0xffffffffu, digit, owner);
        above = __shfl_sync(0xffffffffu, above, owner);
        remaining -= above;
        prefix |= digit << shift;
        prefix_mask |= 255u << shift;
        __syncwarp();
      }
      // prefix = threshold key; `remaining` = how many keys equal to it are taken
      const u32 thr = prefix;
      u32 ties_left = remaining;
      i64 written = 0;
      for (i64 base = 0; base < deg; base += 128) {
        const i64 e0 = base + (i64)lane * 4;
        u32 keys[4];
        int ntie = 0;
        if (e0 < deg && cached) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            keys[j] = e0 + j < deg ? kcache[e0 + j] : 0u;
            if (e0 + j < deg && keys[j] == thr) ++ntie;
          }
        } else if (e0 < deg) {
          const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)(e0 >> 2));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            keys[j] = e0 + j < deg ? ares_key(pick_word(blk, j), __ldg(pr + e0 + j)) : 0u;
            if (e0 + j < deg && keys[j] == thr) ++ntie;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) keys[j] = 0u;
        }
        // rank of this lane's ties among the warp's ties of this chunk
        u32 tinc = (u32)ntie;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          u32 t = __shfl_up_sync(0xffffffffu, tinc, d);
          if (lane >= d) tinc += t;
        }
        u32 tie_rank = tinc - (u32)ntie;
        const u32 chunk_ties = __shfl_sync(0xffffffffu, tinc, 31);
        bool take[4];
        int ntake = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          take[j] = false;
          if (e0 + j < deg) {
            if (keys[j] > thr) take[j] = true;
            else if (keys[j] == thr) { take[j] = tie_rank < ties_left; ++tie_rank; }
          }
          ntake += take[j] ? 1 : 0;
        }
        u32 sinc = (u32)ntake;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          u32 t = __shfl_up_sync(0xffffffffu, sinc, d);
          if (lane >= d) sinc += t;
        }
        i64 o = out_start + written + (sinc - (u32)ntake);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (take[j]) {
            p.out_rows[o] = load_index<IndexT>(p.indices, in_start + e0 + j);
            p.out_sel[o] = in_start + e0 + j;
            if (p.out_cols) p.out_cols[o] = slot;
            ++o;
          }
        }
        written += __shfl_sync(0xffffffffu, sinc, 31);
        ties_left -= chunk_ties < ties_left ? chunk_ties : ties_left;
      }
      continue;
    }
    // ---- with replacement: K draws by streaming the running sum
    float tot = 0.f;
    for (i64 e = lane; e < deg; e += 32) tot += fmaxf(__ldg(pr + e), 0.f);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, d);
    for (int k = lane; k < K; k += 32) {
      const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)k >> 2);
      const float u = ((float)pick_word(blk, k) + 1.0f) * 2.3283064365386963e-10f;
      targets[k] = u * tot;
      p.out_sel[out_start + k] = -1;
    }
    __syncwarp();
    float run = 0.f;
    for (i64 base = 0; base < deg; base += 32) {
      const i64 e = base + lane;
      const float v = e < deg ? fmaxf(__ldg(pr + e), 0.f) : 0.f;
      float inc = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        float t = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += t;
      }
      const float hi = run + __shfl_sync(0xffffffffu, inc, 31);
      const bool last_chunk = base + 32 >= deg;
      for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        const float t = k < K ? targets[k] : -1.f;
        const bool mine = k < K && t > run && (t <= hi || last_chunk) && p.out_sel[out_start + k] < 0;
        unsigned pending = __ballot_sync(0xffffffffu, mine);
        while (pending) {
          const int src = __ffs(pending) - 1;
          pending &= pending - 1;
          const float tt = __shfl_sync(0xffffffffu, t, src);
          const unsigned ge = __ballot_sync(0xffffffffu, e < deg && run + inc >= tt);
          i64 pick = ge ? base + (__ffs(ge) - 1) : deg - 1;
          if (lane == 0) {
            const int kk = k0 + src;
            p.out_sel[out_start + kk] = in_start + pick;
            p.out_rows[out_start + kk] = load_index<IndexT>(p.indices, in_start + pick);
            if (p.out_cols) p.out_cols[out_start + kk] = slot;
          }
        }
        __syncwarp();
      }
      run = hi;
    }
    // draws that fell past the accumulated total (rounding) or columns whose
    // weights are all zero: fall back to the last / a uniform position
    for (int k = lane; k < K; k += 32) {
      if (p.out_sel[out_start + k] < 0) {
        const Philox4 blk = stream_block(p.seed, p.stream, (u64)slot, (u32)k >> 2);
        const i64 pick = tot > 0.f ? deg - 1 : (i64)__umulhi(pick_word(blk, k), (u32)deg);
        p.out_sel[out_start + k] = in_start + pick;
        p.out_rows[out_start + k] = load_index<IndexT>(p.indices, in_start + pick);
        if (p.out_cols) p.out_cols[out_start + k] = slot;
      }
    }
    __syncwarp();
  }
}

}  // namespace gsb

using namespace gsb;

struct ProbLayout {
  size_t count, start, deg, list, long_list, list_n, total;
};

static ProbLayout prob_layout(i64 S_max) {
  ProbLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  size_t o = 0;
  L.count = o; o = up(o + count_workspace_bytes(S_max));
  L.start = o; o = up(o + sizeof(i64) * (size_t)(S_max + 1));
  L.deg = o; o = up(o + sizeof(u32) * (size_t)(S_max + 1));
  L.list = o; o = up(o + sizeof(i64) * (size_t)(S_max + 1));
  L.long_list = o; o = up(o + sizeof(i64) * (size_t)(S_max + 1));
  L.list_n = o; o = up(o + 256);
  L.total = o;
  return L;
}

extern "C" size_t gsb_sample_cols_probs_workspace_bytes(int64_t S_max, int64_t K) {
  if (S_max < 0 || K < 1) return 0;
  return prob_layout(S_max).total;
}

extern "C" int gsb_sample_cols_probs(const int64_t* indptr, const void* indices, int indices_dtype,
                                     int64_t num_cols, const float* probs, const int64_t* seeds,
                                     int64_t S_max,
                                     const int64_t* d_S, int64_t K, int replace, uint64_t seed,
                                     uint32_t stream, int64_t* sub_indptr, int64_t* out_rows,
                                     int64_t* out_cols, int64_t* out_sel, int64_t E_cap,
                                     int64_t* d_num_edges, void* workspace, size_t workspace_bytes,
                                     int* d_err, void* cuda_stream) {
  if (!indptr || !indices || !probs || !sub_indptr || S_max < 0 || E_cap < 0 || K < 1 || num_cols < 0)
    return GSB_ERR_INVALID;
  if (E_cap > 0 && (!out_rows || !out_sel)) return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (K > WP_MAX_K) return GSB_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < gsb_sample_cols_probs_workspace_bytes(S_max, K))
    return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  const ProbLayout L = prob_layout(S_max);
  char* ws = (char*)workspace;
  const bool thread_path = !replace && K <= WT_MAX_K;
  CountExtra extra;
  extra.start = (i64*)(ws + L.start); extra.deg = (u32*)(ws + L.deg);
  extra.list = (i64*)(ws + L.list); extra.list_n = (int*)(ws + L.list_n);
  extra.list_min_deg = thread_path ? WT_MAX_DEG + 1 : 0;  // what is left for the warp kernel
  GSB_CUDA_OK(cudaMemsetAsync(ws + L.list_n, 0, 256, st));
  int rc = launch_count((const i64*)indptr, num_cols, (const i64*)seeds, S_max, (const i64*)d_S, K,
                        replace ? 1 : 0, (i64*)sub_indptr, (i64*)d_num_edges, ws + L.count, d_err, st,
                        extra);
  if (rc != GSB_OK) return rc;
  if (S_max == 0) return GSB_OK;
  ProbParams p;
  p.indptr = (const i64*)indptr; p.indices = indices; p.probs = probs; p.seeds = (const i64*)seeds;
  p.S_max = S_max; p.d_S = (const i64*)d_S; p.K = (int)K; p.replace = replace ? 1 : 0;
  p.seed = seed; p.stream = stream; p.sub_indptr = (const i64*)sub_indptr;
  p.out_rows = (i64*)out_rows; p.out_cols = (i64*)out_cols; p.out_sel = (i64*)out_sel;
  p.E_cap = E_cap; p.err = d_err;
  p.thread_path = thread_path ? 1 : 0;
  p.short_rounds = 1;
  p.slot_start = extra.start; p.slot_deg = extra.deg; p.list = extra.list; p.list_n = extra.list_n;
  p.long_list = (i64*)(ws + L.long_list); p.long_n = (int*)(ws + L.list_n) + 16;
  if (p.thread_path) {
    i64 tb = (S_max + WT_THREADS - 1) / WT_THREADS;
    const size_t tsmem = sizeof(u32) * 2 * (size_t)K * WT_THREADS;
    int resident = 0;  // CTAs an SM holds at this K: whole waves only
    if (indices_dtype == GSB_I32)
      GSB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, sample_probs_thread_kernel<int>, WT_THREADS, tsmem));
    else
      GSB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, sample_probs_thread_kernel<i64>, WT_THREADS, tsmem));
    if (resident < 1) resident = 1;
    // as many tiles per group as still leave every resident CTA a group
    i64 rounds = tb / ((i64)sm_count() * resident);
    rounds = rounds < 1 ? 1 : (rounds > WT_ROUNDS ? WT_ROUNDS : rounds);
    p.short_rounds = (int)rounds;
    tb = (tb + rounds - 1) / rounds;
    if (tb > (i64)sm_count() * resident) tb = (i64)sm_count() * resident;
    LaunchScope ls(KID_SAMPLE_PROBS_SHORT, st);
    if (indices_dtype == GSB_I32)
      sample_probs_thread_kernel<int><<<(int)tb, WT_THREADS, tsmem, st>>>(p);
    else
      sample_probs_thread_kernel<i64><<<(int)tb, WT_THREADS, tsmem, st>>>(p);
  }
  i64 blocks = (S_max + WP_WARPS - 1) / WP_WARPS;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  const size_t smem = sizeof(u32) * WP_WARPS * 256 + sizeof(float) * WP_WARPS * (size_t)K +
                      sizeof(u32) * WP_WARPS * WP_CACHE;
  {
    LaunchScope ls(KID_SAMPLE_PROBS, st);
    if (indices_dtype == GSB_I32)
      sample_probs_kernel<int><<<(int)blocks, WP_THREADS, smem, st>>>(p);
    else
      sample_probs_kernel<i64><<<(int)blocks, WP_THREADS, smem, st>>>(p);
  }
  if (!replace) {
    LaunchScope ls2(KID_SAMPLE_PROBS_LONG, st);
    if (indices_dtype == GSB_I32)
      sample_probs_block_kernel<int><<<sm_count() * GSB_WB_CTAS_PER_SM, WB_THREADS, 0, st>>>(p);
    else
      sample_probs_block_kernel<i64><<<sm_count() * GSB_WB_CTAS_PER_SM, WB_THREADS, 0, st>>>(p);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
