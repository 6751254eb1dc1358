// Per-minibatch first-occurrence unique + relabel (block construction).
//
// Items of a minibatch = its seeds followed by its sampled row ids; the item
// with the smallest index among those carrying an id is the id's first
// occurrence, and `unique` lists the first occurrences in item order.
//
// Finding the smallest index per id is a hashing problem whose cost on this
// GPU is the number of random L2 transactions and atomics (whole-minibatch
// tables in global memory -- open addressing or direct addressing -- measured
// 0.6 ms for 23 M items and, worse, slowed down the kernels of the other
// streams).  So the items are first PARTITIONED by hash into buckets of at
// most a few thousand items, and every bucket is deduplicated by one CTA in a
// SHARED-memory table:
//   setup   : item / bucket geometry of every minibatch           (one block)
//   scatter : (id, index) pairs grouped by bucket.  A bucket owns a region of
//             fixed capacity, so nothing is counted first: every 8192-item
//             tile reserves a run per bucket with one global atomic; what
//             finds its region full goes to an overflow list kept
//             in lanes, so that a bucket rereads only its lane     (streaming)
//   dedupe  : CTA per bucket: shared table id -> smallest index, then
//             min_idx[item] for every REPEATED item of the bucket; a bucket
//             whose ids do not fit the shared table falls back to a table in
//             global memory that the CTA owns                     (streaming
//             read + for a repeat one scattered 4-byte store and one bit set
//             in a bit array with one bit per item)
//   prefix  : first occurrences (clear bits) before every 32-item word of that
//             bit array (popcounts + chained prefix; 1/32 of a word per item)
//   emit    : one pass over the items: node lists, their offsets, and for
//             the items that are edges the relabelled row (position of the
//             id's first item, from the two small arrays above, which stay
//             in L2) and column                                    (streaming)
// Only the prefix pass has CTAs that wait for one another (a bounded chained
// prefix over a few hundred CTAs).  An earlier version kept a 4-byte rank per
// item: count + scan + rank + emit measured 0.40 ms per step on the benchmark
// against 0.30 for mark + prefix + emit.
#include "gsb_common.cuh"

namespace gsb {

constexpr int RL_THREADS = 256;
#ifndef GSB_RL_ITEMS
#define GSB_RL_ITEMS 4
#endif
constexpr int RL_ITEMS = GSB_RL_ITEMS;
constexpr int RL_TILE = RL_THREADS * RL_ITEMS;
constexpr u64 SLOT_EMPTY = ~0ull;
constexpr u32 IDX_UNSET = 0xFFFFFFFFu;
#ifndef GSB_PT_TILE
#define GSB_PT_TILE 8192
#endif
#ifndef GSB_PT_BATCH
#define GSB_PT_BATCH 8
#endif
constexpr int PT_TILE = GSB_PT_TILE;   // items per CTA tile of pcount / scatter
constexpr int PT_THREADS = 512;
constexpr int PT_BATCH = GSB_PT_BATCH; // loads in flight per thread
constexpr int OVF_LANES = 512;         // the overflow list is kept in this many lanes (see relabel_scatter_kernel)
constexpr int PT_MAX_BUCKETS = 1024;   // buckets per minibatch that the scatter pass's shared histogram holds
// grid caps in CTAs per SM: tile kernels (pcount, scatter), the bucket kernel (dedupe) and emit.  One
// CTA per tile / bucket up to 64 per SM lets the hardware scheduler even out the tail (layer 3 of
// cfg2: 2800 tiles, 6400 buckets; caps of 8 and 12 left CTAs with 2 or 3 tiles each): -1.2 % per step.
#ifndef GSB_RL_WIDE
#define GSB_RL_WIDE 64
#endif
#ifndef GSB_RL_BK
#define GSB_RL_BK 64
#endif
#ifndef GSB_BUCKET_ITEMS
#define GSB_BUCKET_ITEMS 3584
#endif
#ifndef GSB_DD_TAB
#define GSB_DD_TAB 8192
#endif
#ifndef GSB_DD_MIN_CTAS
#define GSB_DD_MIN_CTAS 3
#endif
#ifndef GSB_SCATTER_MIN_CTAS
#define GSB_SCATTER_MIN_CTAS 2
#endif
constexpr int PT_BUCKET_ITEMS = GSB_BUCKET_ITEMS;  // a minibatch gets ceil(items / this) buckets
constexpr i64 BK_CAP = 4096;                       // entries of a bucket's region in `part`
constexpr int DD_THREADS = 512;
constexpr int DD_BATCH = 8;            // items a dedupe thread keeps in registers
constexpr int DD_TAB = GSB_DD_TAB;           // shared-table slots of the dedupe CTA
constexpr u32 KEY_EMPTY = 0xFFFFFFFFu;

struct RelabelHeader {
  i64 n_items;
  i64 n_edges;
  i64 n_seeds;
  i64 n_tiles;
  i64 n_buckets;
  i64 n_unique;  // first occurrences of the call (written by the prefix pass)
};

struct RelabelParams {
  const i64* seeds;
  const i64* seeds_ptr;
  const i64* coo_row;
  const i64* coo_col;
  const i64* edge_ptr;
  const i64* sub_indptr;  // non-null: setup derives edge_ptr[b] = sub_indptr[seeds_ptr[b]] first
  i64* edge_ptr_out;
  i64* counts_out;        // nullable {S, (unused), U} of the call, written by the rank pass
  int B;
  i64 S_max, E_max;
  u64 id_limit;       // ids must be below this (at most 2^32 - 1)
  i64* unique;
  i64 U_cap;
  i64* unique_ptr;
  i64* out_row;
  i64* out_col;
  RelabelHeader* hdr;
  i64* item_ptr;      // [B+1] start of minibatch b in the interleaved item order
  u32* min_idx;       // [items] for a repeat: offset of the first item carrying its id
  u32* repeat_bits;   // [items / 32] bit g % 32 of word g / 32: item g repeats an earlier item (zeroed)
  u32* word_prefix;   // [items / 32] first occurrences before the word
  u64* pf_status;     // chained-prefix words of the prefix pass (zeroed)
  int* pf_ticket;     // its CTA ticket (zeroed)
  i64* bucket_ptr;    // [B+1] first bucket of minibatch b
  u32* bucket_fill;   // [buckets] items of the bucket (zeroed; may exceed BK_CAP: the rest is on the overflow list)
  u64* part;          // [buckets * BK_CAP] id:32 | index:32, bucket k owns entries k * BK_CAP ...
  u64* ovf_item;      // [OVF_LANES * ovf_lane_cap] items that found their bucket's region full
  u32* ovf_bucket;    // ... and the bucket each belongs to
  u32* ovf_count;     // [OVF_LANES] entries pushed to each lane (zeroed; above ovf_lane_cap: the lane is full)
  u32 ovf_lane_cap;
  u64* overflow;      // global tables of buckets whose distinct ids overflow the shared table
  u64* gt_cursor;     // bump pointer into `overflow` (zeroed)
  u32* seed_repeat;   // [B] set when a seed of the minibatch repeats an earlier seed (or is invalid)
  int col_prefilled;  // out_col already holds "slot - first slot of the minibatch" (the sampler wrote it)
  i64 buckets_cap;
  int* err;
};

// One block: item_ptr / bucket_ptr = running sums over the minibatches.
__global__ void relabel_setup_kernel(const RelabelParams p) {
  __shared__ i64 s_scan[34];
  __shared__ i64 s_carry_items, s_carry_bk;
  if (threadIdx.x == 0) { s_carry_items = 0; s_carry_bk = 0; }
  __syncthreads();
  for (int b0 = 0; b0 < p.B; b0 += blockDim.x) {
    const int b = b0 + threadIdx.x;
    i64 items = 0, nbk = 0;
    if (b < p.B) {
      i64 ns = p.seeds_ptr[b + 1] - p.seeds_ptr[b];
      i64 ne;
      if (p.sub_indptr) {
        const i64 e_lo = p.sub_indptr[p.seeds_ptr[b]], e_hi = p.sub_indptr[p.seeds_ptr[b + 1]];
        p.edge_ptr_out[b] = e_lo;
        if (b == p.B - 1) p.edge_ptr_out[p.B] = e_hi;
        ne = e_hi - e_lo;
      } else {
        ne = p.edge_ptr[b + 1] - p.edge_ptr[b];
      }
      if (ns < 0 || ne < 0) { raise(p.err, ERRBIT_BAD_INPUT); ns = ns < 0 ? 0 : ns; ne = ne < 0 ? 0 : ne; }
      items = ns + ne;
      const i64 need = (items + PT_BUCKET_ITEMS - 1) / PT_BUCKET_ITEMS;
      nbk = need < 1 ? 1 : need;
    }
    i64 tot_items, tot_bk;
    i64 ei = block_exclusive_scan(items, s_scan, &tot_items);
    __syncthreads();
    i64 eb = block_exclusive_scan(nbk, s_scan, &tot_bk);
    if (b < p.B) {
      p.item_ptr[b] = s_carry_items + ei;
      p.bucket_ptr[b] = s_carry_bk + eb;
    }
    __syncthreads();
    if (threadIdx.x == 0) { s_carry_items += tot_items; s_carry_bk += tot_bk; }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    i64 n_items = s_carry_items;
    i64 n_seeds = p.seeds_ptr[p.B];
    i64 n_edges = p.sub_indptr ? p.sub_indptr[n_seeds < 0 ? 0 : n_seeds] : p.edge_ptr[p.B];
    if (n_items > p.S_max + p.E_max || n_seeds > p.S_max || n_edges > p.E_max || n_seeds < 0 ||
        n_edges < 0 || s_carry_bk > p.buckets_cap) {
      raise(p.err, ERRBIT_CAPACITY);
      n_items = 0; n_seeds = 0; n_edges = 0;  // later kernels become no-ops
    }
    p.item_ptr[p.B] = n_items;
    p.bucket_ptr[p.B] = s_carry_bk;
    p.hdr->n_items = n_items;
    p.hdr->n_edges = n_items == 0 ? 0 : n_edges;
    p.hdr->n_seeds = n_items == 0 ? 0 : n_seeds;
    p.hdr->n_tiles = (n_items + RL_TILE - 1) / RL_TILE;
    p.hdr->n_buckets = n_items == 0 ? 0 : s_carry_bk;
    p.hdr->n_unique = 0;
  }
}

// ---------------------------------------------------------------- global-memory table of one bucket
// Slot = id:32 | smallest index:32 (atomicMin on the whole word: the id half is
// equal for all contenders).  Used by a dedupe CTA for a bucket whose ids do
// not fit its shared table.  The hash differs from the one that chose the
// bucket (all ids of a bucket share that one's leading bits).
__device__ __forceinline__ u32 rehash(u32 key) { return hash32(key * 0x9E3779B1u + 0x7F4A7C15u); }

__device__ __forceinline__ bool gtab_insert(u64* tab, u32 slots, u32 key, u32 idx) {
  const u64 packed = ((u64)key << 32) | idx;
  u32 pos = __umulhi(rehash(key), slots);
  for (u32 probes = 0; probes < slots; ++probes) {
    u64 cur = ld_relaxed(tab + pos);
    if (cur == SLOT_EMPTY) {
      cur = atomicCAS(tab + pos, SLOT_EMPTY, packed);
      if (cur == SLOT_EMPTY) return true;
    }
    if ((u32)(cur >> 32) == key) {
      if ((u32)cur > idx) atomicMin(tab + pos, packed);
      return true;
    }
    pos = pos + 1 == slots ? 0 : pos + 1;
  }
  return false;
}

__device__ __forceinline__ u32 gtab_find(const u64* tab, u32 slots, u32 key) {
  u32 pos = __umulhi(rehash(key), slots);
  for (u32 probes = 0; probes < slots; ++probes) {
    const u64 cur = ld_relaxed(tab + pos);
    if (cur == SLOT_EMPTY) return IDX_UNSET;
    if ((u32)(cur >> 32) == key) return (u32)cur;
    pos = pos + 1 == slots ? 0 : pos + 1;
  }
  return IDX_UNSET;
}

// ---------------------------------------------------------------- a minibatch seen from a kernel
// Offsets inside a minibatch fit 32 bits, so the per-item arithmetic is 32-bit;
// the 64-bit bases are loaded once per minibatch and tile.
struct Segment {
  i64 ibase;           // first item of the minibatch
  i64 iend;            // one past its last item
  const i64* seeds_b;  // its seeds
  const i64* rows_b;   // its row ids, biased by -ns so that seeds and rows index by item offset
  u32 ns;              // number of seeds
  i64 bk0;             // first bucket
  int nbk;
};

__device__ __forceinline__ Segment load_segment(const RelabelParams& p, int b) {
  Segment s;
  s.ibase = p.item_ptr[b];
  s.iend = p.item_ptr[b + 1];
  const i64 s0 = p.seeds_ptr[b];
  const i64 ns = p.seeds_ptr[b + 1] - s0;
  s.seeds_b = p.seeds + s0;
  s.rows_b = p.coo_row + p.edge_ptr[b] - ns;
  s.ns = (u32)ns;
  s.bk0 = p.bucket_ptr[b];
  s.nbk = (int)(p.bucket_ptr[b + 1] - s.bk0);
  return s;
}

__device__ __forceinline__ i64 segment_id(const Segment& s, u32 off) {
  return __ldg((off < s.ns ? s.seeds_b : s.rows_b) + off);
}

// Bucket of an id: its hash scaled to [0, nbk) -- any bucket count works, so a
// minibatch gets exactly ceil(items / PT_BUCKET_ITEMS) buckets of near-equal
// size.  The leading hash bits decide; the shared table inside a bucket uses
// the trailing ones.
__device__ __forceinline__ u32 bucket_of(u32 key, int nbk) {
  return __umulhi(hash32(key), (u32)nbk);
}

// The ids of up to PT_BATCH items of a segment, PT_THREADS apart, loaded before
// any is used (PT_BATCH loads in flight per thread); -1 past `lim`.
#define GSB_LOAD_ID_BATCH(off0, lim)                                 \
  i64 id[PT_BATCH];                                                  \
  _Pragma("unroll") for (int u = 0; u < PT_BATCH; ++u) {             \
    const u32 off = (off0) + (u32)(u * PT_THREADS);                  \
    id[u] = -1;                                                      \
    if (off < (lim)) id[u] = segment_id(sg, off);                    \
  }

// An item that is not a first occurrence: min_idx[g] = offset of the first item carrying its id
// inside the minibatch (IDX_UNSET for an invalid id), and its bit in the array that the prefix
// and emit passes read.  First occurrences are never written: their bit stays clear.
__device__ __forceinline__ void mark_repeat(const RelabelParams& p, i64 g, u32 first_off) {
  p.min_idx[g] = first_off;
  atomicOr(p.repeat_bits + (g >> 5), 1u << (g & 31));
}

// Writes (id, index) of every item into its bucket's region of `part`.  A bucket owns a region of
// BK_CAP entries at a fixed place (bucket k: part[k * BK_CAP ...)), so no counting pass and no
// scan come first: per tile and minibatch a shared histogram, ONE global atomic per non-empty
// bucket reserves the tile's run inside the bucket's region, then every item takes the next free
// entry of its bucket's run.  A minibatch of n items has ceil(n / PT_BUCKET_ITEMS) buckets, so a
// bucket holds PT_BUCKET_ITEMS items on average and its size scatters by a few tens around that;
// items that do not fit the region any more (an id repeated thousands of times) go to the
// overflow list, tagged with their bucket, which the bucket's dedupe CTA reads after its region.
// The list is kept in OVF_LANES lanes of equal capacity so that a bucket does not have to look
// at all of it: bucket k pushes to lane k % OVF_LANES, and to the next lane (and so on, around)
// when that one is full.  The ids are read twice (the
// second read hits L1/L2); the 8-byte stores of a run meet in L2 before they reach DRAM.
__global__ void __launch_bounds__(PT_THREADS, GSB_SCATTER_MIN_CTAS) relabel_scatter_kernel(const RelabelParams p) {
  __shared__ u32 s_hist[PT_MAX_BUCKETS];  // items of the bucket in this tile
  __shared__ u32 s_next[PT_MAX_BUCKETS];  // next free entry of the bucket's run (may pass BK_CAP)
  const i64 n = p.hdr->n_items;
  for (i64 lo = (i64)blockIdx.x * PT_TILE; lo < n; lo += (i64)gridDim.x * PT_TILE) {
    const i64 hi = lo + PT_TILE < n ? lo + PT_TILE : n;
    int b = find_segment(p.item_ptr, p.B, lo);
    i64 at = lo;
    while (at < hi) {
      while (p.item_ptr[b + 1] <= at) ++b;
      const Segment sg = load_segment(p, b);
      const i64 seg_hi = hi < sg.iend ? hi : sg.iend;
      const u32 lim = (u32)(seg_hi - sg.ibase);
      const u32 first = (u32)(at - sg.ibase) + threadIdx.x;
      // entry `dst` of bucket k's items: inside the bucket's region, or on the overflow list
      auto place = [&](i64 id, u32 off, u32 k, u32 dst) {
        const u64 item = ((u64)(u32)id << 32) | off;
        if (dst < (u32)BK_CAP) {
          p.part[(sg.bk0 + k) * BK_CAP + dst] = item;
        } else {
          u32 lane = (u32)((sg.bk0 + k) % OVF_LANES);
          int tries = 0;
          for (; tries < OVF_LANES; ++tries) {
            const u32 q = atomicAdd(p.ovf_count + lane, 1u);
            if (q < p.ovf_lane_cap) {
              const size_t at = (size_t)lane * p.ovf_lane_cap + q;
              p.ovf_item[at] = item;
              p.ovf_bucket[at] = (u32)(sg.bk0 + k);
              break;
            }
            lane = (lane + 1) % OVF_LANES;
          }
          if (tries == OVF_LANES) raise(p.err, ERRBIT_CAPACITY);  // cannot happen: the lanes hold every item
        }
      };
      auto reject = [&](u32 off) {
        raise(p.err, ERRBIT_BAD_INPUT);  // negative, or not below the stated bound
        mark_repeat(p, sg.ibase + off, IDX_UNSET);  // in no node list; relabels to -1
        if (off < sg.ns) p.seed_repeat[b] = 1u;  // its edges' columns relabel to -1: no shortcut
      };
      if (sg.nbk > PT_MAX_BUCKETS) {
        // a minibatch of more than PT_MAX_BUCKETS * PT_BUCKET_ITEMS items (one relabel call over
        // a whole layer): more buckets than the shared histogram holds, so every item takes its
        // entry with a global atomic of its own (thousands of addresses, all in L2)
        for (u32 off0 = first; off0 < lim; off0 += PT_BATCH * PT_THREADS) {
          GSB_LOAD_ID_BATCH(off0, lim)
#pragma unroll
          for (int u = 0; u < PT_BATCH; ++u) {
            const u32 off = off0 + (u32)(u * PT_THREADS);
            if ((u64)id[u] < p.id_limit) {
              const u32 k = bucket_of((u32)id[u], sg.nbk);
              place(id[u], off, k, atomicAdd(p.bucket_fill + sg.bk0 + k, 1u));
            } else if (off < lim) {
              reject(off);
            }
          }
        }
        at = seg_hi;
        continue;
      }
      for (int k = threadIdx.x; k < sg.nbk; k += PT_THREADS) s_hist[k] = 0;
      __syncthreads();
      for (u32 off0 = first; off0 < lim; off0 += PT_BATCH * PT_THREADS) {
        GSB_LOAD_ID_BATCH(off0, lim)
#pragma unroll
        for (int u = 0; u < PT_BATCH; ++u)
          if ((u64)id[u] < p.id_limit) atomicAdd(&s_hist[bucket_of((u32)id[u], sg.nbk)], 1u);
      }
      __syncthreads();
      for (int k = threadIdx.x; k < sg.nbk; k += PT_THREADS) {
        const u32 h = s_hist[k];
        if (h) s_next[k] = atomicAdd(p.bucket_fill + sg.bk0 + k, h);
      }
      __syncthreads();
      for (u32 off0 = first; off0 < lim; off0 += PT_BATCH * PT_THREADS) {
        GSB_LOAD_ID_BATCH(off0, lim)
#pragma unroll
        for (int u = 0; u < PT_BATCH; ++u) {
          const u32 off = off0 + (u32)(u * PT_THREADS);
          if ((u64)id[u] < p.id_limit) {
            const u32 k = bucket_of((u32)id[u], sg.nbk);
            place(id[u], off, k, atomicAdd(&s_next[k], 1u));
          } else if (off < lim) {
            reject(off);
          }
        }
      }
      __syncthreads();
      at = seg_hi;
    }
  }
}

// Shared table of a dedupe CTA: claim the slot of `key` (linear probing) and
// lower its index; returns the slot, or `tab` when the table is full.
__device__ __forceinline__ u32 stab_insert(u32* s_key, u32* s_min, u32 tab, u32 key, u32 idx) {
  const u32 mask = tab - 1;
  u32 pos = hash32(key) & mask;
  for (u32 probes = 0; probes < tab; ++probes) {
    u32 cur = s_key[pos];
    if (cur == KEY_EMPTY) cur = atomicCAS(&s_key[pos], KEY_EMPTY, key);
    if (cur == KEY_EMPTY || cur == key) { atomicMin(&s_min[pos], idx); return pos; }
    pos = (pos + 1) & mask;
  }
  return tab;
}

// CTA per bucket: shared table id -> smallest index, then min_idx + the repeat bit for every
// repeated item of the bucket.  Only the distinct ids have to fit the table, so a hub id repeated
// thousands of times costs nothing extra.  A bucket whose items all lie in its own region (the
// normal case: at most BK_CAP = DD_BATCH * DD_THREADS of them) stays in registers between the two
// phases together with the table slot each item found; a bucket with items on the overflow list
// streams its region and then its lane of the list (every entry of the lane is looked at, the
// bucket's own are used).
template <typename Fn>
__device__ __forceinline__ void for_each_bucket_item(const RelabelParams& p, i64 k, u32 in_region, bool spilled,
                                                     Fn fn) {
  const u64* items = p.part + k * BK_CAP;
  for (u32 i = threadIdx.x; i < in_region; i += DD_THREADS) fn(__ldg(items + i));
  if (!spilled) return;
  // the bucket's lane, and the lanes after it for as long as each was filled to the brim (only
  // then can an entry of this bucket have moved on to the next)
  u32 lane = (u32)(k % OVF_LANES);
  for (int t = 0; t < OVF_LANES; ++t) {
    const u32 pushed = p.ovf_count[lane];
    const u32 n = pushed < p.ovf_lane_cap ? pushed : p.ovf_lane_cap;
    const size_t base = (size_t)lane * p.ovf_lane_cap;
    for (u32 j = threadIdx.x; j < n; j += DD_THREADS)
      if (__ldg(p.ovf_bucket + base + j) == (u32)k) fn(__ldg(p.ovf_item + base + j));
    if (pushed < p.ovf_lane_cap) break;
    lane = (lane + 1) % OVF_LANES;
  }
}

__global__ void __launch_bounds__(DD_THREADS, GSB_DD_MIN_CTAS) relabel_dedupe_kernel(const RelabelParams p) {
  extern __shared__ __align__(16) unsigned char dd_smem[];
  u32* s_key = reinterpret_cast<u32*>(dd_smem);
  u32* s_min = s_key + DD_TAB;
  __shared__ int s_over;
  __shared__ u64 s_gt_off;
  const i64 nb = p.hdr->n_buckets;
  for (i64 k = blockIdx.x; k < nb; k += gridDim.x) {
    const u32 cnt = p.bucket_fill[k];
    if (cnt == 0) continue;  // uniform over the CTA
    const bool spilled = cnt > (u32)BK_CAP;
    const u32 in_region = spilled ? (u32)BK_CAP : cnt;
    const int b = find_segment(p.bucket_ptr, p.B, k);
    const i64 gbase = p.item_ptr[b];
    const u32 ns = (u32)(p.seeds_ptr[b + 1] - p.seeds_ptr[b]);  // items below ns are the minibatch's seeds
    const u64* items = p.part + k * BK_CAP;
    auto repeat = [&](u64 it, u32 m) {
      if (m != (u32)it) {
        mark_repeat(p, gbase + (u32)it, m);
        if ((u32)it < ns) p.seed_repeat[b] = 1u;
      }
    };
    // table size: a power of two >= 1.5 * cnt (at most DD_TAB)
    u32 tab = 1024;
    while (tab < DD_TAB && 2 * tab < 3 * cnt) tab <<= 1;
    {
      uint4* k4 = reinterpret_cast<uint4*>(s_key);
      uint4* m4 = reinterpret_cast<uint4*>(s_min);
      const uint4 ones = make_uint4(KEY_EMPTY, KEY_EMPTY, KEY_EMPTY, KEY_EMPTY);
      for (u32 i = threadIdx.x; i < tab / 4; i += DD_THREADS) { k4[i] = ones; m4[i] = ones; }
    }
    if (threadIdx.x == 0) s_over = 0;
    __syncthreads();
    if (!spilled) {
      u64 it[DD_BATCH];
      u32 slot[DD_BATCH];
#pragma unroll
      for (int u = 0; u < DD_BATCH; ++u) {
        const u32 i = u * DD_THREADS + threadIdx.x;
        it[u] = i < cnt ? __ldg(items + i) : ~0ull;
      }
#pragma unroll
      for (int u = 0; u < DD_BATCH; ++u) {
        slot[u] = 0;
        if (it[u] == ~0ull) continue;
        slot[u] = stab_insert(s_key, s_min, tab, (u32)(it[u] >> 32), (u32)it[u]);
        if (slot[u] == tab) s_over = 1;
      }
      __syncthreads();
      if (!s_over) {
#pragma unroll
        for (int u = 0; u < DD_BATCH; ++u)
          if (it[u] != ~0ull) repeat(it[u], s_min[slot[u]]);
        __syncthreads();
        continue;
      }
    } else {
      for_each_bucket_item(p, k, in_region, spilled, [&](u64 it) {
        if (stab_insert(s_key, s_min, tab, (u32)(it >> 32), (u32)it) == tab) s_over = 1;
      });
      __syncthreads();
      if (!s_over) {
        const u32 mask = tab - 1;
        for_each_bucket_item(p, k, in_region, spilled, [&](u64 it) {
          const u32 key = (u32)(it >> 32);
          u32 pos = hash32(key) & mask;
          for (u32 probes = 0; s_key[pos] != key && probes < tab; ++probes) pos = (pos + 1) & mask;
          repeat(it, s_min[pos]);
        });
        __syncthreads();
        continue;
      }
    }
    // more distinct ids than the shared table holds: a table in global memory, owned by this
    // CTA (2 slots per item of the bucket, taken off a bump pointer)
    const u32 slots = 2 * cnt + 32;
    if (threadIdx.x == 0) s_gt_off = atomicAdd(p.gt_cursor, (u64)slots);
    __syncthreads();
    u64* gt = p.overflow + s_gt_off;
    for (u32 i = threadIdx.x; i < slots; i += DD_THREADS) gt[i] = SLOT_EMPTY;
    __syncthreads();
    for_each_bucket_item(p, k, in_region, spilled, [&](u64 it) {
      if (!gtab_insert(gt, slots, (u32)(it >> 32), (u32)it)) raise(p.err, ERRBIT_TABLE_FULL);
    });
    __syncthreads();
    for_each_bucket_item(p, k, in_region, spilled, [&](u64 it) {
      const u32 m = gtab_find(gt, slots, (u32)(it >> 32));
      if (m == IDX_UNSET) raise(p.err, ERRBIT_KEY_MISSING);
      else repeat(it, m);
    });
    __syncthreads();
  }
}

// ---------------------------------------------------------------- mark / prefix / emit
// The dedupe pass leaves one bit per item, 32 items per word: set = the item repeats an earlier
// one (min_idx then says which).  The position of a first occurrence in `unique` is the number of
// first occurrences before it, so:
//   prefix : word_prefix[w] = first occurrences (clear bits) in all words before w (popcounts,
//            block scan, chained prefix across CTAs) -- the position of ANY item g is then
//            word_prefix[g / 32] + popc(clear bits of word g / 32 below bit g % 32): two loads
//            from arrays of one bit and one 32nd of a word per item, which stay in L2;
//   emit   : one pass over the items writes `unique` (first occurrences, in order), the offsets of
//            the node lists and, for the items that are edges, the relabelled row (and column).
// Items are laid out so that warp w of a 1024-item tile owns 128 consecutive items and lane l
// handles items w*128 + j*32 + l (j = 0..3): every load / store instruction of a warp touches 32
// consecutive items, which are exactly one word of the bit array.
struct ItemCursor {
  int b;
  i64 ibase, iend;
};

__device__ __forceinline__ void cursor_seek(const RelabelParams& p, ItemCursor& c, i64 g) {
  if (g < c.iend) return;
  while (g >= p.item_ptr[c.b + 1]) ++c.b;
  c.ibase = p.item_ptr[c.b];
  c.iend = p.item_ptr[c.b + 1];
}

__device__ __forceinline__ ItemCursor cursor_at(const RelabelParams& p, i64 g) {
  ItemCursor c;
  c.b = find_segment(p.item_ptr, p.B, g);
  c.ibase = p.item_ptr[c.b];
  c.iend = p.item_ptr[c.b + 1];
  return c;
}

#ifndef GSB_PF_THREADS
#define GSB_PF_THREADS 1024
#endif
constexpr int PF_THREADS = GSB_PF_THREADS;
constexpr int PF_WORDS = PF_THREADS * 4;  // words per CTA: 32 768 items

// word_prefix over the whole bit array; the CTA that owns the last word also stores the number
// of first occurrences of the call and checks it against the capacity of `unique`.
__global__ void __launch_bounds__(PF_THREADS) relabel_prefix_kernel(const RelabelParams p) {
  __shared__ i64 s_scan[34];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(p.pf_ticket, 1);
  __syncthreads();
  const int cta = s_tile;
  const i64 n_words = (p.hdr->n_items + 31) >> 5;
  const i64 n_ctas = n_words == 0 ? 1 : (n_words + PF_WORDS - 1) / PF_WORDS;
  if (cta >= n_ctas) return;
  const i64 w0 = (i64)cta * PF_WORDS + (i64)threadIdx.x * 4;
  uint4 v = make_uint4(~0u, ~0u, ~0u, ~0u);
  if (w0 < n_words) v = *reinterpret_cast<const uint4*>(p.repeat_bits + w0);  // padded to a multiple of 4 words
  const i64 n = p.hdr->n_items;
  // first occurrences of a word: its clear bits among the items that exist
  auto firsts = [n](u32 bits, i64 w) -> u32 {
    const i64 left = n - (w << 5);
    const u32 valid = left >= 32 ? ~0u : (left <= 0 ? 0u : ((1u << left) - 1u));
    return (u32)__popc(~bits & valid);
  };
  const u32 c0 = firsts(v.x, w0), c1 = firsts(v.y, w0 + 1), c2 = firsts(v.z, w0 + 2), c3 = firsts(v.w, w0 + 3);
  i64 total;
  const i64 ex = block_exclusive_scan((i64)(c0 + c1 + c2 + c3), s_scan, &total);
  if (threadIdx.x < 32) {
    const i64 base = chained_exclusive_prefix(p.pf_status, cta, total, p.err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  const u32 run = (u32)(s_base + ex);
  if (w0 < n_words)
    *reinterpret_cast<uint4*>(p.word_prefix + w0) = make_uint4(run, run + c0, run + c0 + c1, run + c0 + c1 + c2);
  if (cta == n_ctas - 1 && threadIdx.x == 0) {
    const i64 grand = s_base + total;
    p.hdr->n_unique = grand;
    if (grand > p.U_cap || grand >= 0x7FFFFFFFll) raise(p.err, ERRBIT_CAPACITY);
  }
}

// number of first occurrences before item g (= position in `unique` of a first occurrence g)
__device__ __forceinline__ u32 position_of(const RelabelParams& p, i64 g) {
  const i64 w = g >> 5;
  return __ldg(p.word_prefix + w) + __popc(~__ldg(p.repeat_bits + w) & ((1u << (g & 31)) - 1u));
}

// Everything a thread needs to know about the minibatch of its current item.
struct EmitCursor {
  int b;
  i64 ibase, iend;  // items of the minibatch
  i64 s0;           // its first seed slot
  i64 e0;           // its first edge
  u32 ns;           // number of seeds
  u32 ubase;        // its first position in `unique`
  bool repeat;      // a seed repeats an earlier one (or is invalid): columns need the table
};

__device__ __forceinline__ void emit_cursor_load(const RelabelParams& p, EmitCursor& c) {
  c.ibase = p.item_ptr[c.b];
  c.iend = p.item_ptr[c.b + 1];
  c.s0 = p.seeds_ptr[c.b];
  c.ns = (u32)(p.seeds_ptr[c.b + 1] - c.s0);
  c.e0 = p.edge_ptr[c.b];
  c.ubase = position_of(p, c.ibase);
  c.repeat = p.seed_repeat[c.b] != 0u;
}

#ifndef GSB_EMIT_MIN_CTAS
#define GSB_EMIT_MIN_CTAS 8   // measured per step (three layers): 4 CTAs/SM 0.218 ms, 5 0.196, 6 0.191, 8 0.179
#endif
__global__ void __launch_bounds__(RL_THREADS, GSB_EMIT_MIN_CTAS) relabel_emit_kernel(const RelabelParams p) {
  const i64 n = p.hdr->n_items;
  const i64 tiles = p.hdr->n_tiles;
  const i64 tile = blockIdx.x;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (tile >= tiles) {
    if (tile == 0 && threadIdx.x == 0) {  // no items at all: every node list is empty
      for (int b = 0; b <= p.B; ++b) p.unique_ptr[b] = 0;
      if (p.counts_out) { p.counts_out[0] = p.seeds_ptr[p.B]; p.counts_out[2] = 0; }
    }
    return;
  }
  const bool fits = p.hdr->n_unique <= p.U_cap;
  const i64 g_warp = tile * RL_TILE + (i64)wid * (32 * RL_ITEMS);
  if (g_warp < n) {
    // this warp's own four words of the bit array and their prefixes (one load each, broadcast)
    const i64 w_warp = g_warp >> 5;
    const u32 my_bits = lane < RL_ITEMS ? __ldg(p.repeat_bits + w_warp + lane) : ~0u;
    const u32 my_pref = lane < RL_ITEMS ? __ldg(p.word_prefix + w_warp + lane) : 0u;
    // min_idx is defined for repeats only
    u32 m[RL_ITEMS];
#pragma unroll
    for (int j = 0; j < RL_ITEMS; ++j) {
      const i64 g = g_warp + j * 32 + lane;
      const u32 bits = __shfl_sync(0xffffffffu, my_bits, j);
      m[j] = (g < n && ((bits >> lane) & 1u)) ? __ldg(p.min_idx + g) : IDX_UNSET;
    }
    EmitCursor c;
    c.b = find_segment(p.item_ptr, p.B, g_warp);
    emit_cursor_load(p, c);
    const u32 lt_mask = (1u << lane) - 1u;
    // The common case by far: all 128 items of the warp are edges of one minibatch whose columns
    // are already in place.  Straight-line code, so that the four independent chains of gathers
    // (min_idx -> bit word + prefix of the first item) and the id loads are all in flight before
    // the first store.
    if (p.out_row && p.col_prefilled && !c.repeat && g_warp - c.ibase >= (i64)c.ns &&
        g_warp + 32 * RL_ITEMS <= c.iend) {
      const i64 e_warp = c.e0 + (g_warp - c.ibase - (i64)c.ns) + lane;
      u32 pos[RL_ITEMS];
      bool first[RL_ITEMS];
#pragma unroll
      for (int j = 0; j < RL_ITEMS; ++j) {
        const u32 bits = __shfl_sync(0xffffffffu, my_bits, j);
        const u32 pref = __shfl_sync(0xffffffffu, my_pref, j);
        first[j] = ((bits >> lane) & 1u) == 0u;
        pos[j] = pref + __popc(~bits & lt_mask);
        if (!first[j] && m[j] != IDX_UNSET) pos[j] = position_of(p, c.ibase + m[j]);
      }
      i64 idv[RL_ITEMS];
#pragma unroll
      for (int j = 0; j < RL_ITEMS; ++j) idv[j] = (first[j] && fits) ? __ldg(p.coo_row + e_warp + j * 32) : 0;
#pragma unroll
      for (int j = 0; j < RL_ITEMS; ++j) {
        if (first[j] && fits) p.unique[pos[j]] = idv[j];
        p.out_row[e_warp + j * 32] = (first[j] || m[j] != IDX_UNSET) ? (i64)pos[j] - (i64)c.ubase : -1;
      }
    } else
#pragma unroll
    for (int j = 0; j < RL_ITEMS; ++j) {
      const i64 g = g_warp + j * 32 + lane;
      const u32 bits = __shfl_sync(0xffffffffu, my_bits, j);
      const u32 pref = __shfl_sync(0xffffffffu, my_pref, j);
      if (g >= n) continue;
      if (g >= c.iend) {
        while (g >= p.item_ptr[c.b + 1]) ++c.b;
        emit_cursor_load(p, c);
      }
      const u32 off = (u32)(g - c.ibase);
      const u32 here = pref + __popc(~bits & lt_mask);  // first occurrences before this item
      if (off == 0) {
        // first item of its minibatch: the running count is the minibatch's offset; empty
        // minibatches directly before it share the same value
        int b = c.b;
        p.unique_ptr[b] = here;
        while (b > 0 && p.item_ptr[b - 1] == g) p.unique_ptr[--b] = here;
      }
      const bool first = ((bits >> lane) & 1u) == 0u;
      const bool valid_id = first || m[j] != IDX_UNSET;
      u32 pos = here;
      if (!first && valid_id) pos = position_of(p, c.ibase + m[j]);
      const bool is_edge = off >= c.ns;
      if (first && fits) {
        // the id is read only here: one item in three is a repeat
        const i64 id = is_edge ? __ldg(p.coo_row + c.e0 + (off - c.ns)) : __ldg(p.seeds + c.s0 + off);
        p.unique[pos] = id;
      }
      if (is_edge && p.out_row) {
        const i64 e = c.e0 + (off - c.ns);
        p.out_row[e] = valid_id ? (i64)pos - (i64)c.ubase : -1;
        // The COLUMN of an edge needs no table when the seeds of its minibatch are distinct
        // (always, from the second layer on: they are a node list): seed i is then the i-th entry
        // of the minibatch's list, so the relabelled column is the column slot counted from the
        // minibatch's first slot -- which the layered sampler has already written.
        if (c.repeat || !p.col_prefilled) {
          const u64 lc = (u64)(__ldg(p.coo_col + e) - c.s0);  // seed slot inside the minibatch
          if (lc >= c.ns) {
            raise(p.err, ERRBIT_BAD_INPUT);  // a column slot outside the edge's own minibatch
            p.out_col[e] = -1;
          } else if (!c.repeat) {
            p.out_col[e] = (i64)lc;
          } else {
            // the seed's own item: a first occurrence, or a repeat of an earlier seed
            const i64 gs = c.ibase + (i64)lc;
            const bool seed_first = ((__ldg(p.repeat_bits + (gs >> 5)) >> (gs & 31)) & 1u) == 0u;
            const u32 mc = seed_first ? (u32)lc : __ldg(p.min_idx + gs);
            p.out_col[e] = mc != IDX_UNSET ? (i64)position_of(p, c.ibase + mc) - (i64)c.ubase : -1;
          }
        }
      }
    }
  }
  if (tile == tiles - 1 && threadIdx.x == 0) {
    const i64 grand = p.hdr->n_unique;
    int b = p.B;
    p.unique_ptr[b] = grand;
    while (b > 0 && p.item_ptr[b - 1] == n) p.unique_ptr[--b] = grand;
    if (p.counts_out) { p.counts_out[0] = p.seeds_ptr[p.B]; p.counts_out[2] = grand; }
  }
}

// offsets inside the zeroed block
constexpr size_t ZB_GT_CURSOR = 0, ZB_OVF_COUNT = 256, ZB_BUCKET_FILL = 256 + sizeof(u32) * OVF_LANES;
static_assert(ZB_BUCKET_FILL % 256 == 0, "bucket fill levels start on a 256-byte boundary");

struct RelabelLayout {
  size_t hdr, item_ptr, bucket_ptr, bucket_fill, seed_repeat, pf_status, repeat_bits,
      min_idx, word_prefix, part, ovf_item, ovf_bucket, overflow, total;
  i64 tiles, buckets_cap, pf_ctas, ovf_lane_cap;
};

static RelabelLayout relabel_layout(i64 S_max, i64 E_max, i64 B) {
  RelabelLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const i64 items = S_max + E_max;
  L.tiles = (items + RL_TILE - 1) / RL_TILE + 1;
  // a minibatch of n items has ceil(n / PT_BUCKET_ITEMS) buckets, at least one
  L.buckets_cap = B + (items + PT_BUCKET_ITEMS - 1) / PT_BUCKET_ITEMS + 1;
  size_t o = 0;
  L.hdr = o; o = up(o + sizeof(RelabelHeader));
  L.item_ptr = o; o = up(o + sizeof(i64) * (size_t)(B + 1));
  L.bucket_ptr = o; o = up(o + sizeof(i64) * (size_t)(B + 1));
  // zeroed block: table bump pointer (first 256 bytes), overflow-lane fill levels, bucket fill
  // levels, repeated-seed flags, prefix-pass ticket / status, repeat bits
  L.bucket_fill = o; o = up(o + ZB_BUCKET_FILL + sizeof(u32) * (size_t)(L.buckets_cap + 1));
  L.seed_repeat = o; o = up(o + sizeof(u32) * (size_t)(B + 1));
  const i64 words = (items + 31) / 32 + 8;
  L.pf_ctas = (words + PF_WORDS - 1) / PF_WORDS + 1;
  L.pf_status = o; o = up(o + 256 + sizeof(u64) * (size_t)(L.pf_ctas + 1));   // ticket, then status words
  L.repeat_bits = o; o = up(o + sizeof(u32) * (size_t)(words + 8));
  L.min_idx = o; o = up(o + sizeof(u32) * (size_t)(items + 4));
  L.word_prefix = o; o = up(o + sizeof(u32) * (size_t)(words + 8));
  L.part = o; o = up(o + sizeof(u64) * (size_t)(L.buckets_cap + 1) * (size_t)BK_CAP);
  // together the lanes hold every item, whichever lanes they crowd into
  L.ovf_lane_cap = (items + OVF_LANES - 1) / OVF_LANES + 64;
  L.ovf_item = o; o = up(o + sizeof(u64) * (size_t)(L.ovf_lane_cap * OVF_LANES));
  L.ovf_bucket = o; o = up(o + sizeof(u32) * (size_t)(L.ovf_lane_cap * OVF_LANES));
  // overflow tables: 2 slots per item + 32 per bucket; touched only by buckets that need them
  L.overflow = o; o = up(o + sizeof(u64) * (size_t)(2 * items + 32 * (L.buckets_cap + 1)));
  L.total = o;
  return L;
}

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_batch_relabel_workspace_bytes(int64_t S_max, int64_t E_max, int64_t B) {
  if (S_max < 0 || E_max < 0 || B < 0) return 0;
  return relabel_layout(S_max, E_max, B).total;
}

extern "C" int gsb_batch_relabel(const int64_t* seeds, const int64_t* seeds_ptr, int64_t B,
                                 int64_t S_max, const int64_t* coo_row, const int64_t* coo_col,
                                 const int64_t* edge_ptr, int64_t E_max, int64_t id_bound,
                                 int64_t* unique, int64_t U_cap, int64_t* unique_ptr,
                                 int64_t* out_row, int64_t* out_col, void* workspace,
                                 size_t workspace_bytes, int* d_err, void* cuda_stream) {
  return gsb::relabel_launch(seeds, seeds_ptr, B, S_max, coo_row, coo_col, edge_ptr, nullptr, nullptr,
                             E_max, id_bound, unique, U_cap, unique_ptr, out_row, out_col, nullptr, 0,
                             workspace, workspace_bytes, d_err, cuda_stream);
}

// `sub_indptr` non-null: edge_ptr is derived on the device (edge_ptr_out[b] =
// sub_indptr[seeds_ptr[b]]) instead of read; `counts_out` non-null: receives
// {seeds_ptr[B], -, unique_ptr[B]}.  Both spare the layered sampler a launch.
// `col_prefilled`: out_col[e] already holds coo_col[e] - seeds_ptr[minibatch of e].
int gsb::relabel_launch(const int64_t* seeds, const int64_t* seeds_ptr, int64_t B, int64_t S_max,
                        const int64_t* coo_row, const int64_t* coo_col, const int64_t* edge_ptr,
                        const int64_t* sub_indptr, int64_t* edge_ptr_out, int64_t E_max,
                        int64_t id_bound, int64_t* unique, int64_t U_cap, int64_t* unique_ptr,
                        int64_t* out_row, int64_t* out_col, int64_t* counts_out, int col_prefilled,
                        void* workspace, size_t workspace_bytes, int* d_err, void* cuda_stream) {
  if (sub_indptr) edge_ptr = edge_ptr_out;
  if (B < 1 || S_max < 0 || E_max < 0 || !seeds_ptr || !edge_ptr || !unique_ptr || U_cap < 0)
    return GSB_ERR_INVALID;
  if ((S_max > 0 && !seeds) || (E_max > 0 && !coo_row) || (U_cap > 0 && !unique)) return GSB_ERR_INVALID;
  if ((out_row == nullptr) != (out_col == nullptr)) return GSB_ERR_INVALID;
  if (out_row && E_max > 0 && !coo_col) return GSB_ERR_INVALID;
  if (id_bound > 0xFFFFFFFFll || S_max + E_max >= (1ll << 31) || B >= (1ll << 30))
    return GSB_ERR_UNSUPPORTED;
  const RelabelLayout L = relabel_layout(S_max, E_max, B);
  if (!workspace || workspace_bytes < L.total) return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  char* ws = (char*)workspace;
  RelabelParams p;
  p.seeds = (const i64*)seeds; p.seeds_ptr = (const i64*)seeds_ptr; p.coo_row = (const i64*)coo_row;
  p.coo_col = (const i64*)coo_col; p.edge_ptr = (const i64*)edge_ptr; p.B = (int)B;
  p.sub_indptr = (const i64*)sub_indptr; p.edge_ptr_out = (i64*)edge_ptr_out; p.counts_out = (i64*)counts_out;
  p.S_max = S_max; p.E_max = E_max; p.unique = (i64*)unique; p.U_cap = U_cap;
  p.id_limit = id_bound > 0 && id_bound < 0xFFFFFFFFll ? (u64)id_bound : 0xFFFFFFFFull;
  p.unique_ptr = (i64*)unique_ptr; p.out_row = (i64*)out_row; p.out_col = (i64*)out_col;
  p.hdr = (RelabelHeader*)(ws + L.hdr); p.item_ptr = (i64*)(ws + L.item_ptr);
  p.min_idx = (u32*)(ws + L.min_idx); p.err = d_err;
  p.repeat_bits = (u32*)(ws + L.repeat_bits); p.word_prefix = (u32*)(ws + L.word_prefix);
  p.pf_ticket = (int*)(ws + L.pf_status); p.pf_status = (u64*)(ws + L.pf_status + 256);
  p.bucket_ptr = (i64*)(ws + L.bucket_ptr);
  p.gt_cursor = (u64*)(ws + L.bucket_fill + ZB_GT_CURSOR); p.ovf_count = (u32*)(ws + L.bucket_fill + ZB_OVF_COUNT);
  p.bucket_fill = (u32*)(ws + L.bucket_fill + ZB_BUCKET_FILL); p.ovf_lane_cap = (u32)L.ovf_lane_cap;
  p.ovf_item = (u64*)(ws + L.ovf_item); p.ovf_bucket = (u32*)(ws + L.ovf_bucket);
  p.part = (u64*)(ws + L.part); p.overflow = (u64*)(ws + L.overflow); p.buckets_cap = L.buckets_cap;
  p.seed_repeat = (u32*)(ws + L.seed_repeat); p.col_prefilled = col_prefilled ? 1 : 0;

  { LaunchScope ls(KID_RL_SETUP, st); relabel_setup_kernel<<<1, 1024, 0, st>>>(p); }
  // table bump pointer, overflow-lane and bucket fill levels, the repeated-seed flags, the prefix pass's ticket /
  // status words and the repeat bits are adjacent: one clear
  GSB_CUDA_OK(cudaMemsetAsync(ws + L.bucket_fill, 0, L.min_idx - L.bucket_fill, st));
  const i64 items_max = S_max + E_max;
  const int wide = sm_count() * GSB_RL_WIDE;
  int g_tiles = (int)((items_max + PT_TILE - 1) / PT_TILE); if (g_tiles < 1) g_tiles = 1;
  if (g_tiles > wide) g_tiles = wide;
  { LaunchScope ls(KID_RL_SCATTER, st); relabel_scatter_kernel<<<g_tiles, PT_THREADS, 0, st>>>(p); }
  const int g_bk = (int)(L.buckets_cap < sm_count() * GSB_RL_BK ? L.buckets_cap : sm_count() * GSB_RL_BK);
  const int dd_smem = 2 * DD_TAB * (int)sizeof(u32);
  GSB_CUDA_OK(cudaFuncSetAttribute(relabel_dedupe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dd_smem));
  { LaunchScope ls(KID_RL_DEDUPE, st); relabel_dedupe_kernel<<<g_bk, DD_THREADS, dd_smem, st>>>(p); }
  { LaunchScope ls(KID_RL_TILES, st); relabel_prefix_kernel<<<(int)L.pf_ctas, PF_THREADS, 0, st>>>(p); }
  { LaunchScope ls(KID_RL_EDGES, st); relabel_emit_kernel<<<(int)L.tiles, RL_THREADS, 0, st>>>(p); }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
