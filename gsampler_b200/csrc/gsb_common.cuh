// Shared device helpers for the sm_100a sampling kernels: the counter-based
// random stream, warp/block scans, the single-pass chained prefix ("look-back")
// used to turn per-tile counts into global output offsets, and the packed
// 64-bit hash slots of the relabel tables.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gsb200.h"

namespace gsb {

typedef long long i64;
typedef unsigned long long u64;
typedef unsigned int u32;

// Bits of the device error word (gsb200.h documents them for callers).
enum : int {
  ERRBIT_LOOKBACK_TIMEOUT = 1,   // a tile waited too long for its predecessor
  ERRBIT_TABLE_FULL = 2,         // a hash probe visited every slot
  ERRBIT_KEY_MISSING = 4,        // lookup of a key that was never inserted
  ERRBIT_CAPACITY = 8,           // an output would exceed the caller's capacity
  ERRBIT_BAD_INPUT = 16          // id out of range / non-monotone offsets seen on device
};

__device__ __forceinline__ void raise(int* err, int bit) {
  if (err) atomicOr(err, bit);
}

// ---------------------------------------------------------------- Philox4x32-10
struct Philox4 {
  u32 x, y, z, w;
};

__device__ __forceinline__ Philox4 philox4x32_10(u32 c0, u32 c1, u32 c2, u32 c3, u32 k0, u32 k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    u32 hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    u32 hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    u32 n0 = hi1 ^ c1 ^ k0;
    u32 n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}

// Block `blk` (draws 4*blk .. 4*blk+3) of the stream owned by `slot`.
__device__ __forceinline__ Philox4 stream_block(u64 seed, u32 stream, u64 slot, u32 blk) {
  return philox4x32_10((u32)slot, (u32)(slot >> 32), blk, stream, (u32)seed, (u32)(seed >> 32));
}

__device__ __forceinline__ u32 pick_word(const Philox4& p, u32 n) {
  u32 a = (n & 1) ? p.y : p.x;
  u32 b = (n & 1) ? p.w : p.z;
  return (n & 2) ? b : a;
}

// Sequential reader of one stream (walks, rejection loops).
struct StreamReader {
  u64 seed, slot;
  u32 stream, n;
  Philox4 cur;
  __device__ __forceinline__ void init(u64 seed_, u32 stream_, u64 slot_) {
    seed = seed_; stream = stream_; slot = slot_; n = 0;
  }
  __device__ __forceinline__ u32 next() {
    if ((n & 3) == 0) cur = stream_block(seed, stream, slot, n >> 2);
    u32 v = pick_word(cur, n);
    ++n;
    return v;
  }
};

// ---------------------------------------------------------------- scans
__device__ __forceinline__ i64 warp_inclusive_scan(i64 v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    i64 t = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += t;
  }
  return v;
}

__device__ __forceinline__ i64 warp_sum(i64 v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// Exclusive scan over the block (blockDim.x a multiple of 32, <= 1024).
// `warp_tot` is caller-provided shared scratch of 33 i64.  Returns the
// exclusive prefix of `v`; *total receives the block sum (all threads).
__device__ __forceinline__ i64 block_exclusive_scan(i64 v, i64* warp_tot, i64* total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  i64 inc = warp_inclusive_scan(v);
  if (lane == 31) warp_tot[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    i64 t = lane < nw ? warp_tot[lane] : 0;
    i64 ti = warp_inclusive_scan(t);
    if (lane < nw) warp_tot[lane] = ti - t;
    if (lane == 31) warp_tot[32] = ti;
  }
  __syncthreads();
  i64 r = warp_tot[wid] + inc - v;
  *total = warp_tot[32];
  return r;
}

// ---------------------------------------------------------------- chained prefix
// status word: [63:62] 0 = not ready, 1 = tile aggregate, 2 = inclusive prefix;
// [61:0] value.  The array must be zero before the launch.
constexpr u64 LB_AGG = 1ull << 62;
constexpr u64 LB_PREFIX = 2ull << 62;
constexpr u64 LB_MASK = (1ull << 62) - 1;
constexpr int LB_SPIN_LIMIT = 1 << 22;

__device__ __forceinline__ u64 ld_relaxed(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed(u64* p, u64 v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Called by all 32 lanes of ONE warp of the block.  Publishes `aggregate` for
// `tile`, then walks back over predecessor tiles (32 at a time) until one with
// an inclusive prefix is found.  Returns the exclusive prefix of the tile in
// every lane.  Every wait is bounded; on timeout the error bit is raised and
// the missing predecessors count as zero so that the kernel still terminates.
__device__ __forceinline__ i64 chained_exclusive_prefix(u64* status, int tile, i64 aggregate,
                                                        int* err) {
  const int lane = threadIdx.x & 31;
  if (tile == 0) {
    if (lane == 0) st_relaxed(status, LB_PREFIX | (u64)aggregate);
    return 0;
  }
  if (lane == 0) st_relaxed(status + tile, LB_AGG | (u64)aggregate);
  i64 exclusive = 0;
  int base = tile - 1;
  for (;;) {
    int idx = base - lane;
    u64 w = LB_PREFIX;  // tiles before tile 0 behave as "prefix 0"
    if (idx >= 0) {
      int spins = 0;
      w = ld_relaxed(status + idx);
      while ((w >> 62) == 0 && ++spins < LB_SPIN_LIMIT) {
        __nanosleep(32);
        w = ld_relaxed(status + idx);
      }
      if ((w >> 62) == 0) {
        raise(err, ERRBIT_LOOKBACK_TIMEOUT);
        w = LB_PREFIX;
      }
    }
    unsigned pm = __ballot_sync(0xffffffffu, (w >> 62) == 2);
    int first = pm ? (__ffs(pm) - 1) : 31;
    i64 v = (lane <= first) ? (i64)(w & LB_MASK) : 0;
    exclusive += warp_sum(v);
    if (pm) break;
    base -= 32;
  }
  if (lane == 0) st_relaxed(status + tile, LB_PREFIX | (u64)(exclusive + aggregate));
  return exclusive;
}

// ---------------------------------------------------------------- L2 residency hints
// Per-instruction cache policy only (no device-wide setting is touched).  A small array that
// every CTA gathers from at random (the column offsets) is loaded with an evict-last policy so
// that the streams flowing past it -- gathered row ids, output stores -- do not push it out of
// L2; those streams are marked evict-first and bypass L1.
__device__ __forceinline__ u64 l2_policy_keep() {
  u64 pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ u64 l2_policy_stream() {
  u64 pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ i64 ld_i64_keep(const i64* p, u64 pol) {
  i64 v;
  asm volatile("ld.global.nc.L1::evict_last.L2::cache_hint.b64 %0, [%1], %2;" : "=l"(v) : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ i64 ld_i64_stream(const i64* p, u64 pol) {
  i64 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b64 %0, [%1], %2;" : "=l"(v) : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ int ld_i32_stream(const int* p, u64 pol) {
  int v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ void st_i64_stream(i64* p, i64 v, u64 pol) {
  asm volatile("st.global.L1::no_allocate.L2::cache_hint.b64 [%0], %1, %2;" ::"l"(p), "l"(v), "l"(pol) : "memory");
}

// ---------------------------------------------------------------- misc
__device__ __forceinline__ u32 hash32(u32 k) {
  k ^= k >> 16; k *= 0x85ebca6bu; k ^= k >> 13; k *= 0xc2b2ae35u; k ^= k >> 16;
  return k;
}

// largest b with ptr[b] <= x, for a non-decreasing ptr[0..n] (n+1 entries)
__device__ __forceinline__ int find_segment(const i64* __restrict__ ptr, int n, i64 x) {
  int lo = 0, hi = n;  // answer in [lo, hi)
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (ptr[mid] <= x) lo = mid; else hi = mid;
  }
  return lo;
}

template <typename T>
__device__ __forceinline__ i64 load_index(const void* base, i64 pos);
template <>
__device__ __forceinline__ i64 load_index<int>(const void* base, i64 pos) {
  return (i64)__ldg((const int*)base + pos);
}
template <>
__device__ __forceinline__ i64 load_index<i64>(const void* base, i64 pos) {
  return __ldg((const i64*)base + pos);
}
// the same gather marked as a stream (see the L2 hints above)
template <typename T>
__device__ __forceinline__ i64 load_index_stream(const void* base, i64 pos, u64 pol);
template <>
__device__ __forceinline__ i64 load_index_stream<int>(const void* base, i64 pos, u64 pol) {
  return (i64)ld_i32_stream((const int*)base + pos, pol);
}
template <>
__device__ __forceinline__ i64 load_index_stream<i64>(const void* base, i64 pos, u64 pol) {
  return ld_i64_stream((const i64*)base + pos, pol);
}

// gsb_batch_relabel with two extras for the layered sampler (gsb_relabel.cu)
int relabel_launch(const int64_t* seeds, const int64_t* seeds_ptr, int64_t B, int64_t S_max,
                   const int64_t* coo_row, const int64_t* coo_col, const int64_t* edge_ptr,
                   const int64_t* sub_indptr, int64_t* edge_ptr_out, int64_t E_max, int64_t id_bound,
                   int64_t* unique, int64_t U_cap, int64_t* unique_ptr, int64_t* out_row,
                   int64_t* out_col, int64_t* counts_out, int col_prefilled, void* workspace,
                   size_t workspace_bytes, int* d_err, void* cuda_stream);

// gsb_sample_cols with the extras of the layered sampler (gsb_sample.cu): `out_block_col`
// receives every edge's column slot counted from its minibatch's first slot (seeds_ptr, B);
// S_geom (>= S_max) is the slot count the workspace was sized for
int sample_launch(const int64_t* indptr, const void* indices, int indices_dtype, int64_t num_cols,
                  const int64_t* seeds, int64_t S_max, const int64_t* d_S, int64_t K, int replace,
                  uint64_t seed, uint32_t stream, int64_t* sub_indptr, int64_t* out_rows,
                  int64_t* out_cols, int64_t* out_sel, int64_t E_cap, int64_t* d_num_edges,
                  const int64_t* seeds_ptr, int64_t B, int64_t* out_block_col, int64_t S_geom,
                  void* workspace, size_t workspace_bytes, int* d_err, void* cuda_stream);

inline int ceil_div_i(i64 a, i64 b) { return (int)((a + b - 1) / b); }

// Number of SMs of the current device (queried once per device and cached); grid caps are
// stated in CTAs per SM times this.
int sm_count();

// Launch accounting: every kernel launch of the library sits inside a
// LaunchScope, which counts it and, when timing is enabled
// (gsb_timing_enable), brackets it with CUDA events on the launching stream.
enum KernelId {
  KID_SAMPLE = 0, KID_SAMPLE_PROBS, KID_COUNT, KID_SLICE_FILL, KID_GATHER, KID_EXPAND,
  KID_INDPTR_SORTED, KID_RL_SETUP, KID_RL_PCOUNT, KID_RL_PSCAN, KID_RL_SCATTER, KID_RL_DEDUPE,
  KID_RL_COUNT, KID_RL_TILES, KID_RL_SCAN, KID_RL_EDGES, KID_SLICE_ROWS, KID_EDGE_SUM,
  KID_EDGE_OP, KID_LIST_SAMPLE, KID_WALK, KID_SORT, KID_SAMPLE_PROBS_SHORT, KID_SAMPLE_PROBS_LONG, KID_MISC, KID_NUM
};
struct LaunchScope {
  LaunchScope(int id, cudaStream_t st);
  ~LaunchScope();
  int id;
  cudaStream_t st;
  int slot;
};
void set_timing_tag(int tag);

// Offsets of a slice/sample in one pass (defined in gsb_slice.cu): sub_indptr =
// exclusive scan of the per-column pick counts, optional device total.
size_t count_workspace_bytes(i64 S_max);
// optional by-products of the count pass: first entry / length of every column slot, and a
// list (unordered) of the slots whose column has at least list_min_deg entries and a non-zero
// pick count; *list_n must be zero before the launch
struct CountExtra {
  i64* start = nullptr;
  u32* deg = nullptr;
  i64* list = nullptr;
  int* list_n = nullptr;
  i64 list_min_deg = 0;
};
int launch_count(const i64* indptr, i64 num_cols, const i64* seeds, i64 S_max, const i64* d_S, i64 K,
                 int replace, i64* sub_indptr, i64* d_total, void* workspace, int* d_err,
                 cudaStream_t st, const CountExtra& extra = CountExtra());

#define GSB_CUDA_OK(expr)                          \
  do {                                             \
    cudaError_t _e = (expr);                       \
    if (_e != cudaSuccess) return GSB_ERR_CUDA;    \
  } while (0)

}  // namespace gsb
