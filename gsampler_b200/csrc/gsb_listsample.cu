// Collective (layer-wise) selection: choose K of the R candidates of every
// segment, uniformly or with probability weights, without replacement; plus
// the with-replacement draws for a single segment.
//
// Weighted selection without replacement = the K largest A-Res keys
// log2(u_i)/p_i (u_i = draw 0 of element i's counter-based stream).  Instead
// of sorting all R keys, the K-th largest key of every segment is located by a
// 4-round radix select over 32-bit orderable keys (per-segment 256-bin
// histograms, one launch per round), and one scan-and-emit pass writes the
// winners in ascending index order; ties on the threshold key go to the lowest
// indices.  Everything is sized by R, nothing by K: 6 launches per call.
// Uniform selection without replacement is one reservoir pass (Algorithm R with
// an atomic max per slot), picks in slot order.
#include "gsb_common.cuh"

namespace gsb {

constexpr int LS_THREADS = 256;

struct SegState {
  u32 prefix, mask, remaining, take_all;
};

struct ListParams {
  const float* probs;  // nullable -> uniform
  const i64* range;    // [B+1]
  int B;
  i64 R;               // range[B] upper bound (host value)
  i64 K;
  u64 seed; u32 stream;
  u32* keys;           // [R]
  u32* hist;           // [B*256]
  SegState* state;     // [B]
  u32* eq_total;       // [B] keys equal to the final threshold
  i64* seg_base;       // [B] winners before the segment's first item: above << 31 | equal
  i64* out_idx;        // [<= B*K]
  i64* out_range;      // [B+1]
  u64* status; int* ticket;
  int* done;           // CTAs that finished the current round
  int* err;
};

__device__ __forceinline__ u32 list_key(const ListParams& p, i64 i) {
  const Philox4 blk = stream_block(p.seed, p.stream, (u64)i, 0);
  if (!p.probs) return blk.x;
  const float pr = __ldg(p.probs + i);
  if (!(pr > 0.f)) return 0u;
  const float u = ((float)blk.x + 1.0f) * 2.3283064365386963e-10f;
  const float k = __log2f(u) / pr;
  u32 b = __float_as_uint(k);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return b == 0u ? 1u : b;
}

// one block: out_range = scan of min(K, len); reset the per-segment state
__global__ void list_setup_kernel(const ListParams p) {
  __shared__ i64 s_scan[34];
  __shared__ i64 s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < p.B; b0 += blockDim.x) {
    const int b = b0 + threadIdx.x;
    i64 take = 0;
    if (b < p.B) {
      i64 len = p.range[b + 1] - p.range[b];
      if (len < 0) { raise(p.err, ERRBIT_BAD_INPUT); len = 0; }
      take = len < p.K ? len : p.K;
      if (p.state) p.state[b] = SegState{0u, 0u, (u32)take, len <= p.K ? 1u : 0u};  // null: uniform path
    }
    i64 tot;
    const i64 ex = block_exclusive_scan(take, s_scan, &tot);
    if (b < p.B) p.out_range[b] = s_carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) s_carry += tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    p.out_range[p.B] = s_carry;
    if (p.range[p.B] > p.R) raise(p.err, ERRBIT_CAPACITY);
    // the segments must cover the items from 0: the weighted rounds would count an item below
    // range[0] into the first segment while the uniform pass skips it
    if (p.range[0] != 0) raise(p.err, ERRBIT_BAD_INPUT);
  }
}

constexpr int LS_TILE = LS_THREADS * 4;  // items per CTA step: four consecutive keys per thread

__device__ __forceinline__ void list_flush(const ListParams& p, u32* s_h, int b) {
  __syncthreads();
  if (b >= 0 && s_h[threadIdx.x]) atomicAdd(p.hist + b * 256 + threadIdx.x, s_h[threadIdx.x]);
  s_h[threadIdx.x] = 0;
  __syncthreads();
}

// One radix-select round for all segments: histogram of the current digit over the keys that
// still match their segment's prefix, then -- in the CTA that finishes last -- the choice of the
// digit that holds the wanted rank.  Every CTA owns one contiguous run of items and keeps its
// histogram in shared memory for as long as the run stays inside one segment (always, for a
// single list), so a round costs one flush of at most 256 counters per CTA, not one per tile.
// The first round also computes and stores the keys; the last one leaves, per segment, how many
// keys equal the threshold and the global counts of winners before the segment's first item
// (what the emit pass subtracts).  "Last CTA" is decided by a counter after a __threadfence():
// no CTA waits for another.
__global__ void __launch_bounds__(LS_THREADS) list_round_kernel(const ListParams p, int shift, int first) {
  __shared__ u32 s_h[256];
  __shared__ i64 s_scan[34];
  __shared__ i64 s_carry;
  __shared__ int s_last;
  const i64 n = p.range[p.B] < p.R ? p.range[p.B] : p.R;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const i64 per = (((n + gridDim.x - 1) / gridDim.x) + LS_TILE - 1) / LS_TILE * LS_TILE;
  const i64 c0 = (i64)blockIdx.x * per, c1 = c0 + per < n ? c0 + per : n;
  s_h[threadIdx.x] = 0;
  int cur_b = -1;  // the segment whose counts sit in s_h
  const bool spread = first && p.probs;  // weighted keys crowd into a few top digits
  for (i64 base = c0; base < c1; base += LS_TILE) {
    const i64 last_i = base + LS_TILE - 1 < c1 - 1 ? base + LS_TILE - 1 : c1 - 1;
    const int b_lo = find_segment(p.range, p.B, base), b_hi = find_segment(p.range, p.B, last_i);
    const bool one_segment = b_lo == b_hi;  // uniform over the CTA
    if (one_segment && b_lo != cur_b) { list_flush(p, s_h, cur_b); cur_b = b_lo; }
    const i64 i0 = base + (i64)threadIdx.x * 4;
    u32 k[4] = {0u, 0u, 0u, 0u};
    if (first) {
#pragma unroll
      for (int j = 0; j < 4; ++j) if (i0 + j < c1) k[j] = list_key(p, i0 + j);
      if (i0 + 3 < c1) *reinterpret_cast<uint4*>(p.keys + i0) = make_uint4(k[0], k[1], k[2], k[3]);
      else for (int j = 0; j < 4; ++j) if (i0 + j < c1) p.keys[i0 + j] = k[j];
    } else if (i0 + 3 < c1) {
      const uint4 v = *reinterpret_cast<const uint4*>(p.keys + i0);
      k[0] = v.x; k[1] = v.y; k[2] = v.z; k[3] = v.w;
    } else {
      for (int j = 0; j < 4; ++j) if (i0 + j < c1) k[j] = p.keys[i0 + j];
    }
    SegState s = p.state[b_lo];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int b = b_lo;
      bool in = i0 + j < c1;
      if (in && !one_segment) { b = find_segment(p.range, p.B, i0 + j); s = p.state[b]; }
      in = in && !s.take_all && (k[j] & s.mask) == s.prefix;
      const u32 d = (k[j] >> shift) & 255u;
      if (!one_segment) {
        if (in) atomicAdd(p.hist + b * 256 + d, 1u);
      } else if (spread) {  // one shared-memory add per distinct digit of the warp
        const unsigned same = __match_any_sync(0xffffffffu, in ? d : 256u + (u32)lane);
        if (in && lane == __ffs(same) - 1) atomicAdd(&s_h[d], (u32)__popc(same));
      } else if (in) {
        atomicAdd(&s_h[d], 1u);
      }
    }
  }
  list_flush(p, s_h, cur_b);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.done, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // warp per segment: locate the bucket that holds the `remaining`-th largest key
  for (int b = wid; b < p.B; b += LS_THREADS / 32) {
    SegState s = p.state[b];
    volatile u32* h = p.hist + b * 256;
    u32 cnt[8], mine = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { cnt[j] = h[255 - (lane * 8 + j)]; h[255 - (lane * 8 + j)] = 0; mine += cnt[j]; }
    if (s.take_all) continue;  // warp-uniform
    u32 inc = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      u32 t = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += t;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, inc >= s.remaining);
    const int owner = hit ? __ffs(hit) - 1 : 31;
    if (lane == owner) {
      u32 run = inc - mine;
      int d = 0, j = 0;
      for (; j < 8; ++j) {
        d = 255 - (lane * 8 + j);
        if (run + cnt[j] >= s.remaining || d == 0) break;
        run += cnt[j];
      }
      s.remaining -= run;
      s.prefix |= (u32)d << shift;
      s.mask |= 255u << shift;
      p.state[b] = s;
      if (shift == 0) p.eq_total[b] = cnt[j < 8 ? j : 7];
    }
  }
  if (threadIdx.x == 0) { *p.done = 0; s_carry = 0; }
  if (shift != 0) return;
  __syncthreads();
  // winners (above the threshold | equal to it) before each segment's first item, packed
  for (int b0 = 0; b0 < p.B; b0 += LS_THREADS) {
    const int b = b0 + threadIdx.x;
    i64 packed = 0;
    if (b < p.B) {
      const SegState s = p.state[b];
      i64 len = p.range[b + 1] - p.range[b];
      if (len < 0) len = 0;
      if (s.take_all) packed = len << 31;
      else packed = (((len < p.K ? len : p.K) - (i64)s.remaining) << 31) | (i64)p.eq_total[b];
    }
    i64 tot;
    const i64 ex = block_exclusive_scan(packed, s_scan, &tot);
    if (b < p.B) p.seg_base[b] = s_carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) s_carry += tot;
    __syncthreads();
  }
}

// Ordered emit: a chained scan over tiles of 1024 keys counts the winners before every item
// (keys above the segment's threshold, and keys equal to it); a winner's output position is its
// segment's offset plus its rank inside the segment, ties on the threshold going to the lowest
// indices.  Only winners are written.
__global__ void __launch_bounds__(LS_THREADS) list_emit_kernel(const ListParams p) {
  __shared__ i64 s_scan[34];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(p.ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  const i64 n = p.range[p.B] < p.R ? p.range[p.B] : p.R;
  const i64 tiles = (n + LS_TILE - 1) / LS_TILE;
  if (tile >= tiles) return;
  const i64 base = (i64)tile * LS_TILE;
  const i64 i0 = base + (i64)threadIdx.x * 4;
  const i64 last_i = base + LS_TILE - 1 < n - 1 ? base + LS_TILE - 1 : n - 1;
  const int b_lo = find_segment(p.range, p.B, base), b_hi = find_segment(p.range, p.B, last_i);
  const bool one_segment = b_lo == b_hi;
  u32 k[4] = {0u, 0u, 0u, 0u};
  if (i0 + 3 < n) {
    const uint4 v = *reinterpret_cast<const uint4*>(p.keys + i0);
    k[0] = v.x; k[1] = v.y; k[2] = v.z; k[3] = v.w;
  } else {
    for (int j = 0; j < 4; ++j) if (i0 + j < n) k[j] = p.keys[i0 + j];
  }
  int seg[4];
  bool gt[4], eq[4];
  i64 packed = 0;
  SegState s = p.state[b_lo];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    seg[j] = b_lo; gt[j] = false; eq[j] = false;
    if (i0 + j < n) {
      if (!one_segment) { seg[j] = find_segment(p.range, p.B, i0 + j); s = p.state[seg[j]]; }
      gt[j] = s.take_all || k[j] > s.prefix;
      eq[j] = !s.take_all && k[j] == s.prefix;
      packed += gt[j] ? (1ll << 31) : (eq[j] ? 1 : 0);
    }
  }
  i64 total;
  const i64 loff = block_exclusive_scan(packed, s_scan, &total);
  if (threadIdx.x < 32) {
    i64 b = chained_exclusive_prefix(p.status, tile, total, p.err);
    if (threadIdx.x == 0) s_base = b;
  }
  __syncthreads();
  i64 run = s_base + loff;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (gt[j] || eq[j]) {
      if (!one_segment || j == 0) s = p.state[seg[j]];
      const i64 rel = run - p.seg_base[seg[j]];  // winners of this segment before this item
      const u32 gt_before = (u32)(rel >> 31), eq_before = (u32)(rel & 0x7FFFFFFF);
      if (gt[j] || eq_before < s.remaining) {
        const u32 eq_taken = s.take_all ? 0u : (eq_before < s.remaining ? eq_before : s.remaining);
        p.out_idx[p.out_range[seg[j]] + gt_before + eq_taken] = i0 + j;
      }
      run += gt[j] ? (1ll << 31) : 1;
    }
  }
}

// Uniform selection without replacement: reservoir sampling (Algorithm R) evaluated in
// parallel, the reference's scheme (list_sampling.cu:47-64).  Candidate j of a segment (j counted
// from the segment's start) owns slot j if j < K; otherwise it draws num = floor(u * (j + 1)) and
// claims slot num when num < K.  Sequentially a slot ends with the last candidate that drew it,
// i.e. the largest index: an atomic max, whatever the order of execution.  `out_idx` must be zero
// before the launch; picks come out in slot order.
__global__ void __launch_bounds__(LS_THREADS) list_reservoir_kernel(const ListParams p) {
  const bool whole = p.range == nullptr;  // one list [0, R), stated by the caller: no offsets to read or write
  const i64 n = whole ? p.R : (p.range[p.B] < p.R ? p.range[p.B] : p.R);
  if (!whole && p.B == 1 && blockIdx.x == 0 && threadIdx.x == 0) {  // a single list has no set-up launch
    i64 len = p.range[1] - p.range[0];
    if (len < 0) { raise(p.err, ERRBIT_BAD_INPUT); len = 0; }
    if (p.range[1] > p.R) raise(p.err, ERRBIT_CAPACITY);
    p.out_range[0] = 0;
    p.out_range[1] = len < p.K ? len : p.K;
  }
  for (i64 i = (i64)blockIdx.x * LS_THREADS + threadIdx.x; i < n; i += (i64)gridDim.x * LS_THREADS) {
    const int b = p.B == 1 ? 0 : find_segment(p.range, p.B, i);
    const i64 r0 = whole ? 0 : p.range[b], j = i - r0, len = whole ? p.R : p.range[b + 1] - r0;
    if (j < 0) continue;  // an item before the first segment
    long long* out = reinterpret_cast<long long*>(p.out_idx) + (p.B == 1 ? 0 : p.out_range[b]);
    if (len <= p.K) { out[j] = i; continue; }
    if (j < p.K) { atomicMax(out + j, (long long)i); continue; }
    const u32 d = stream_block(p.seed, p.stream, (u64)i, 0).x;
    const u64 num = ((u64)d * (u64)(j + 1)) >> 32;
    if (num < (u64)p.K) atomicMax(out + num, (long long)i);
  }
}

// K draws with replacement from one segment [0, n): uniform, or by inverse CDF
__global__ void list_replace_uniform_kernel(i64 n, i64 K, u64 seed, u32 stream, i64* out) {
  for (i64 k = (i64)blockIdx.x * blockDim.x + threadIdx.x; k < K; k += (i64)gridDim.x * blockDim.x) {
    const Philox4 blk = stream_block(seed, stream, 0, (u32)(k >> 2));
    out[k] = (i64)(((u64)pick_word(blk, (u32)k) * (u64)n) >> 32);
  }
}

// inclusive prefix sums of probs (double accumulators) by one block
__global__ void list_cdf_kernel(const float* __restrict__ probs, i64 n, double* __restrict__ cdf) {
  __shared__ double s_part[1024];
  const i64 per = (n + blockDim.x - 1) / blockDim.x;
  const i64 lo = (i64)threadIdx.x * per, hi = lo + per < n ? lo + per : n;
  double acc = 0;
  for (i64 i = lo; i < hi; ++i) acc += fmaxf(probs[i], 0.f);
  s_part[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double run = 0;
    for (int t = 0; t < (int)blockDim.x; ++t) { const double v = s_part[t]; s_part[t] = run; run += v; }
  }
  __syncthreads();
  acc = s_part[threadIdx.x];
  for (i64 i = lo; i < hi; ++i) { acc += fmaxf(probs[i], 0.f); cdf[i] = acc; }
}

__global__ void list_replace_cdf_kernel(const double* __restrict__ cdf, i64 n, i64 K, u64 seed,
                                        u32 stream, i64* out) {
  const double total = cdf[n - 1];
  for (i64 k = (i64)blockIdx.x * blockDim.x + threadIdx.x; k < K; k += (i64)gridDim.x * blockDim.x) {
    const Philox4 blk = stream_block(seed, stream, 0, (u32)(k >> 2));
    const double target = ((double)pick_word(blk, (u32)k) + 1.0) * (1.0 / 4294967296.0) * total;
    i64 lo = 0, hi = n - 1;  // first position with cdf >= target
    while (lo < hi) {
      const i64 mid = (lo + hi) >> 1;
      if (cdf[mid] < target) lo = mid + 1; else hi = mid;
    }
    out[k] = lo;
  }
}

struct ListLayout {
  size_t ticket, status, keys, hist, state, eq_total, seg_base, total;
  i64 tiles;
};

static ListLayout list_layout(i64 R, i64 B) {
  ListLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.tiles = R / (LS_THREADS * 4) + 2;
  size_t o = 0;
  L.ticket = o; o = up(o + 256);
  L.status = o; o = up(o + sizeof(u64) * (size_t)L.tiles);
  L.hist = o; o = up(o + sizeof(u32) * 256 * (size_t)(B > 0 ? B : 1));
  L.keys = o; o = up(o + sizeof(u32) * (size_t)(R + 1));
  L.state = o; o = up(o + sizeof(SegState) * (size_t)(B > 0 ? B : 1));
  L.eq_total = o; o = up(o + sizeof(u32) * (size_t)(B > 0 ? B : 1));
  L.seg_base = o; o = up(o + sizeof(i64) * (size_t)(B > 0 ? B : 1));
  // the with-replacement path reuses the region as a double CDF
  size_t cdf = up(sizeof(double) * (size_t)(R + 1));
  L.total = o > cdf ? o : cdf;
  return L;
}

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_list_sample_workspace_bytes(int64_t R, int64_t B) {
  if (R < 0 || B < 0) return 0;
  return list_layout(R, B).total;
}

extern "C" int gsb_list_sample(const float* probs, const int64_t* range, int64_t B, int64_t R,
                               int64_t K, uint64_t seed, uint32_t stream, int64_t* out_idx,
                               int64_t* out_range, void* workspace, size_t workspace_bytes,
                               int* d_err, void* cuda_stream) {
  const bool whole = !range && !probs && B == 1;  // uniform choice from the one list [0, R)
  if ((!whole && (!range || !out_range)) || B < 1 || R < 0 || K < 0 || (R > 0 && K > 0 && !out_idx))
    return GSB_ERR_INVALID;
  if (R >= (1ll << 31) || B >= (1ll << 22)) return GSB_ERR_UNSUPPORTED;
  const ListLayout L = list_layout(R, B);
  if (probs && (!workspace || workspace_bytes < L.total)) return GSB_ERR_WORKSPACE;  // uniform: no scratch
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  ListParams p;
  p.probs = probs; p.range = (const i64*)range; p.B = (int)B; p.R = R; p.K = K; p.seed = seed;
  p.stream = stream; p.keys = (u32*)(ws + L.keys); p.hist = (u32*)(ws + L.hist);
  p.state = (SegState*)(ws + L.state); p.eq_total = (u32*)(ws + L.eq_total);
  p.seg_base = (i64*)(ws + L.seg_base); p.out_idx = (i64*)out_idx; p.out_range = (i64*)out_range;
  p.status = (u64*)(ws + L.status); p.ticket = (int*)(ws + L.ticket); p.done = p.ticket + 16;
  p.err = d_err;
  if (!probs) {  // uniform: one reservoir pass, no keys, nothing in the workspace (it may be absent)
    p.keys = nullptr; p.hist = nullptr; p.state = nullptr; p.eq_total = nullptr; p.seg_base = nullptr;
    p.status = nullptr; p.ticket = nullptr; p.done = nullptr;
    const i64 cap = R < B * K ? R : B * K;  // most picks there can be
    if (cap > 0) GSB_CUDA_OK(cudaMemsetAsync(out_idx, 0, sizeof(i64) * (size_t)cap, st));
    if (!whole && (B > 1 || R == 0 || K == 0)) { LaunchScope ls(KID_LIST_SAMPLE, st); list_setup_kernel<<<1, 1024, 0, st>>>(p); }
    if (R > 0 && K > 0) {
      i64 gr = (R + LS_THREADS - 1) / LS_THREADS; if (gr > sm_count() * 16) gr = sm_count() * 16;
      LaunchScope ls(KID_LIST_SAMPLE, st);
      list_reservoir_kernel<<<(int)gr, LS_THREADS, 0, st>>>(p);
    }
    GSB_CUDA_OK(cudaGetLastError());
    return GSB_OK;
  }
  GSB_CUDA_OK(cudaMemsetAsync(ws, 0, L.keys, st));  // ticket, status, histograms
  i64 g = (R + LS_TILE - 1) / LS_TILE; if (g > sm_count() * 4) g = sm_count() * 4; if (g < 1) g = 1;
  { LaunchScope ls(KID_LIST_SAMPLE, st); list_setup_kernel<<<1, 1024, 0, st>>>(p); }
  if (R > 0 && K > 0) {
    for (int shift = 24; shift >= 0; shift -= 8) {
      LaunchScope ls(KID_LIST_SAMPLE, st);
      list_round_kernel<<<(int)g, LS_THREADS, 0, st>>>(p, shift, shift == 24 ? 1 : 0);
    }
    { LaunchScope ls(KID_LIST_SAMPLE, st); list_emit_kernel<<<(int)L.tiles, LS_THREADS, 0, st>>>(p); }
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_list_sample_replace(const float* probs, int64_t n, int64_t K, uint64_t seed,
                                       uint32_t stream, int64_t* out_idx, void* workspace,
                                       size_t workspace_bytes, void* cuda_stream) {
  if (K == 0) return GSB_OK;
  if (n < 1 || K < 0 || !out_idx) return GSB_ERR_INVALID;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  i64 g = (K + 255) / 256; if (g > sm_count() * 8) g = sm_count() * 8;
  if (!probs) {
    LaunchScope ls(KID_LIST_SAMPLE, st);
    list_replace_uniform_kernel<<<(int)g, 256, 0, st>>>(n, K, seed, stream, (i64*)out_idx);
  } else {
    if (!workspace || workspace_bytes < list_layout(n, 1).total) return GSB_ERR_WORKSPACE;
    { LaunchScope ls(KID_LIST_SAMPLE, st); list_cdf_kernel<<<1, 1024, 0, st>>>(probs, n, (double*)workspace); }
    { LaunchScope ls(KID_LIST_SAMPLE, st);
      list_replace_cdf_kernel<<<(int)g, 256, 0, st>>>((const double*)workspace, n, K, seed, stream, (i64*)out_idx); }
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
