// Per-minibatch first-occurrence unique + relabel (block construction).
//
// Every minibatch gets its own open-addressing table; the tables sit back to
// back in the workspace and are sized from the minibatch's item count (items =
// its seeds followed by its sampled row ids).  A slot is ONE 64-bit word:
// key in the high half, the smallest item index carrying that key in the low
// half (atomicMin on the whole word; the key half is equal for all contenders,
// so the minimum is the minimum index).  The item whose own index equals that
// minimum is the first occurrence of its id.
//
// Passes (each a plain data-parallel kernel; no CTA ever waits for another):
//   insert : claim / lower the slot of every item                (random RMW)
//   lookup : min_idx[item] = payload of the item's slot, and the number of
//            first occurrences of every 1024-item tile           (random read)
//   tiles  : exclusive scan of the per-tile counts               (one block)
//   rank   : first occurrences get their position in `unique` (tile base +
//            warp ballots), written to unique[] and rank[item]   (streaming)
//   emit   : every edge reads rank[first item of its row id] and of its
//            column's seed -> relabelled COO                     (streaming +
//            one gather for ids that were seen before)
// When the caller states a bound on the ids and B * bound 32-bit words are not
// more memory than the hash tables would be, the tables are direct-address
// arrays instead (word = smallest item index of that id): no probing, no key
// compare, and the insert is a fire-and-forget atomic min.
// The tables are written only by `insert`; nothing is finalised in place.  The
// measured limiter of the stage is the number of random L2/DRAM transactions,
// which this arrangement keeps at about two per item (one RMW, one read).
#include "gsb_common.cuh"

namespace gsb {

constexpr int RL_THREADS = 256;
constexpr int RL_ITEMS = 4;
constexpr int RL_TILE = RL_THREADS * RL_ITEMS;
constexpr u64 SLOT_EMPTY = ~0ull;
constexpr u32 IDX_UNSET = 0xFFFFFFFFu;

struct RelabelHeader {
  i64 n_items;
  i64 n_slots;
  i64 n_edges;
  i64 n_seeds;
  i64 n_tiles;
};

struct RelabelParams {
  const i64* seeds;
  const i64* seeds_ptr;
  const i64* coo_row;
  const i64* coo_col;
  const i64* edge_ptr;
  int B;
  i64 S_max, E_max;
  i64* unique;
  i64 U_cap;
  i64* unique_ptr;
  i64* out_row;
  i64* out_col;
  RelabelHeader* hdr;
  i64* item_ptr;     // [B+1] start of minibatch b in the interleaved item order
  i64* table_ptr;    // [B+1] start of minibatch b's table
  u32* tile_count;   // [tiles+1] first occurrences per tile, then their exclusive scan
  u64* table;
  u32* min_idx;      // [items] smallest item index carrying the item's id
  u32* rank;         // [items] position in `unique`, valid for first occurrences
  i64 slots_cap;
  i64 tiles_cap;
  i64 direct_bound;  // > 0: direct-address tables of this many 32-bit words per minibatch
  int* err;
};

__host__ __device__ inline i64 table_slots_for(i64 items) { return items * 2 + 32; }

// One block: item_ptr / table_ptr = running sums over the minibatches.
__global__ void relabel_setup_kernel(const RelabelParams p) {
  __shared__ i64 s_scan[34];
  __shared__ i64 s_carry_items, s_carry_slots;
  if (threadIdx.x == 0) { s_carry_items = 0; s_carry_slots = 0; }
  __syncthreads();
  for (int b0 = 0; b0 < p.B; b0 += blockDim.x) {
    const int b = b0 + threadIdx.x;
    i64 items = 0, slots = 0;
    if (b < p.B) {
      i64 ns = p.seeds_ptr[b + 1] - p.seeds_ptr[b];
      i64 ne = p.edge_ptr[b + 1] - p.edge_ptr[b];
      if (ns < 0 || ne < 0) { raise(p.err, ERRBIT_BAD_INPUT); ns = ns < 0 ? 0 : ns; ne = ne < 0 ? 0 : ne; }
      items = ns + ne;
      slots = table_slots_for(items);
    }
    i64 tot_items, tot_slots;
    i64 ei = block_exclusive_scan(items, s_scan, &tot_items);
    __syncthreads();
    i64 es = block_exclusive_scan(slots, s_scan, &tot_slots);
    if (b < p.B) {
      p.item_ptr[b] = s_carry_items + ei;
      p.table_ptr[b] = s_carry_slots + es;
    }
    __syncthreads();
    if (threadIdx.x == 0) { s_carry_items += tot_items; s_carry_slots += tot_slots; }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    i64 n_items = s_carry_items, n_slots = s_carry_slots;
    if (p.direct_bound > 0) n_slots = (p.direct_bound * p.B + 1) / 2;  // 64-bit words to clear
    i64 n_seeds = p.seeds_ptr[p.B], n_edges = p.edge_ptr[p.B];
    if (n_items > p.S_max + p.E_max || n_slots > p.slots_cap || n_seeds > p.S_max ||
        n_edges > p.E_max || n_seeds < 0 || n_edges < 0) {
      raise(p.err, ERRBIT_CAPACITY);
      n_items = 0; n_slots = 0; n_seeds = 0; n_edges = 0;  // later kernels become no-ops
    }
    p.item_ptr[p.B] = n_items;
    p.table_ptr[p.B] = n_slots;
    p.hdr->n_items = n_items;
    p.hdr->n_slots = n_slots;
    p.hdr->n_edges = n_items == 0 ? 0 : n_edges;
    p.hdr->n_seeds = n_items == 0 ? 0 : n_seeds;
    p.hdr->n_tiles = (n_items + RL_TILE - 1) / RL_TILE;
  }
}

// tables <- empty, per-tile counters <- 0
__global__ void relabel_clear_kernel(const RelabelParams p) {
  const i64 tid = (i64)blockIdx.x * blockDim.x + threadIdx.x, nth = (i64)gridDim.x * blockDim.x;
  const i64 n = p.hdr->n_slots;
  ulonglong2* t2 = reinterpret_cast<ulonglong2*>(p.table);  // 256-byte aligned base
  for (i64 i = tid; i < (n >> 1); i += nth) t2[i] = make_ulonglong2(SLOT_EMPTY, SLOT_EMPTY);
  if ((n & 1) && tid == 0) p.table[n - 1] = SLOT_EMPTY;
  const i64 nt = p.hdr->n_tiles + 1;
  for (i64 i = tid; i < nt; i += nth) p.tile_count[i] = 0;
}

struct Item {
  int b;
  u32 key;
  u32 idx;      // index inside the minibatch's item list
  i64 src;      // seed slot (seeds) or edge index (rows) in the caller's arrays
  bool is_seed;
  bool ok;
};

// `b_hint` = minibatch of an item at or before g: the binary search runs once
// per warp, the walk below is a no-op except at minibatch boundaries.
__device__ __forceinline__ Item fetch_item(const RelabelParams& p, i64 g, int b_hint) {
  Item it;
  it.b = b_hint;
  while (g >= p.item_ptr[it.b + 1]) ++it.b;
  const i64 off = g - p.item_ptr[it.b];
  const i64 s0 = p.seeds_ptr[it.b];
  const i64 ns = p.seeds_ptr[it.b + 1] - s0;
  it.is_seed = off < ns;
  it.src = it.is_seed ? s0 + off : p.edge_ptr[it.b] + (off - ns);
  const i64 key = it.is_seed ? p.seeds[it.src] : p.coo_row[it.src];
  it.ok = key >= 0 && key < 0xFFFFFFFFll;
  it.key = (u32)key;
  it.idx = (u32)off;
  return it;
}

// Read before claiming: duplicates of a popular id mostly find a smaller index
// already in place and leave without an atomic, which keeps hot slots from
// serialising in L2 (claim-first measured 2x slower on a power-law graph).
// Items are visited in order so that the smallest index tends to arrive first.
__global__ void __launch_bounds__(RL_THREADS) relabel_insert_kernel(const RelabelParams p) {
  const i64 n = p.hdr->n_items;
  for (i64 g = (i64)blockIdx.x * RL_THREADS + threadIdx.x; g < n; g += (i64)gridDim.x * RL_THREADS) {
    const int b_hint = find_segment(p.item_ptr, p.B, g - (threadIdx.x & 31));  // warp-uniform
    const Item it = fetch_item(p, g, b_hint);
    if (!it.ok) { raise(p.err, ERRBIT_BAD_INPUT); continue; }
    if (p.direct_bound > 0) {
      if ((i64)it.key >= p.direct_bound) { raise(p.err, ERRBIT_BAD_INPUT); continue; }
      u32* w = reinterpret_cast<u32*>(p.table) + (i64)it.b * p.direct_bound + it.key;
      u32 cur;  // read first: later duplicates of a popular id leave without an atomic
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(cur) : "l"(w) : "memory");
      if (cur > it.idx) atomicMin(w, it.idx);
      continue;
    }
    const i64 base = p.table_ptr[it.b];
    const u32 slots = (u32)(p.table_ptr[it.b + 1] - base);
    u64* tab = p.table + base;
    const u64 packed = ((u64)it.key << 32) | it.idx;
    u32 pos = __umulhi(hash32(it.key), slots);
    u32 probes = 0;
    for (; probes < slots; ++probes) {
      u64 cur = ld_relaxed(tab + pos);
      if (cur == SLOT_EMPTY) {
        cur = atomicCAS(tab + pos, SLOT_EMPTY, packed);
        if (cur == SLOT_EMPTY) break;
      }
      if ((u32)(cur >> 32) == it.key) {
        if ((u32)cur > it.idx) atomicMin(tab + pos, packed);
        break;
      }
      pos = pos + 1 == slots ? 0 : pos + 1;
    }
    if (probes == slots) raise(p.err, ERRBIT_TABLE_FULL);
  }
}

// payload (smallest item index) of `key`, or IDX_UNSET if the key is absent.
// The tables are read-only once the insert pass is over.
__device__ __forceinline__ u32 lookup_min_index(const u64* __restrict__ tab, u32 slots, u32 key) {
  u32 pos = __umulhi(hash32(key), slots);
  for (u32 probes = 0; probes < slots; ++probes) {
    const u64 cur = __ldg(tab + pos);
    if (cur == SLOT_EMPTY) return IDX_UNSET;
    if ((u32)(cur >> 32) == key) return (u32)cur;
    pos = pos + 1 == slots ? 0 : pos + 1;
  }
  return IDX_UNSET;
}

// Thread per item (consecutive threads, consecutive items).  A CTA's 256
// items lie inside one 1024-item tile, whose counter collects the number of
// first occurrences (one atomic per warp).
__global__ void __launch_bounds__(RL_THREADS) relabel_lookup_kernel(const RelabelParams p) {
  const i64 n = p.hdr->n_items;
  const int lane = threadIdx.x & 31;
  for (i64 g0 = (i64)blockIdx.x * RL_THREADS; g0 < n; g0 += (i64)gridDim.x * RL_THREADS) {
    const i64 g = g0 + threadIdx.x;
    bool first = false;
    if (g < n) {
      const int b_hint = find_segment(p.item_ptr, p.B, g - lane);
      const Item it = fetch_item(p, g, b_hint);
      u32 m = IDX_UNSET;
      if (it.ok && p.direct_bound > 0) {
        if ((i64)it.key < p.direct_bound)
          m = __ldg(reinterpret_cast<const u32*>(p.table) + (i64)it.b * p.direct_bound + it.key);
        first = m == it.idx;
      } else if (it.ok) {
        const i64 base = p.table_ptr[it.b];
        m = lookup_min_index(p.table + base, (u32)(p.table_ptr[it.b + 1] - base), it.key);
        if (m == IDX_UNSET) raise(p.err, ERRBIT_KEY_MISSING);
        first = m == it.idx;
      }
      p.min_idx[g] = m;
    }
    const unsigned mask = __ballot_sync(0xffffffffu, first);
    if (lane == 0 && mask) atomicAdd(p.tile_count + g0 / RL_TILE, (u32)__popc(mask));
  }
}

// One block: tile_count <- exclusive scan (the entry after the last tile
// receives the total).
__global__ void relabel_tiles_kernel(const RelabelParams p) {
  __shared__ i64 s_scan[34];
  const i64 nt = p.hdr->n_tiles;
  const i64 per = (nt + blockDim.x - 1) / blockDim.x;
  const i64 lo = (i64)threadIdx.x * per, hi = lo + per < nt ? lo + per : nt;
  i64 acc = 0;
  for (i64 i = lo; i < hi; ++i) acc += p.tile_count[i];
  i64 total;
  i64 run = block_exclusive_scan(acc, s_scan, &total);
  for (i64 i = lo; i < hi; ++i) { const u32 c = p.tile_count[i]; p.tile_count[i] = (u32)run; run += c; }
  if (threadIdx.x == 0) {
    p.tile_count[nt] = (u32)total;
    if (total > p.U_cap || total >= 0x7FFFFFFFll) raise(p.err, ERRBIT_CAPACITY);
  }
}

// Tile layout: warp w owns 128 consecutive items, lane l handles items
// w*128 + j*32 + l (j = 0..3), so every load/store instruction of a warp
// touches 32 consecutive items and ranks follow from warp ballots.
__global__ void __launch_bounds__(RL_THREADS) relabel_rank_kernel(const RelabelParams p) {
  __shared__ int s_warp[RL_THREADS / 32];
  const i64 n = p.hdr->n_items;
  const i64 tiles = p.hdr->n_tiles;
  const i64 tile = blockIdx.x;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (tile >= tiles) {
    if (tile == 0 && threadIdx.x == 0)  // no items at all: every node list is empty
      for (int b = 0; b <= p.B; ++b) p.unique_ptr[b] = 0;
    return;
  }
  const unsigned lt_mask = (1u << lane) - 1u;
  const i64 g_warp = tile * RL_TILE + (i64)wid * (32 * RL_ITEMS);
  const int b_warp = g_warp < n ? find_segment(p.item_ptr, p.B, g_warp) : 0;
  Item it[RL_ITEMS];
  bool live[RL_ITEMS], first[RL_ITEMS];
  int before[RL_ITEMS];
  int warp_firsts = 0;
#pragma unroll
  for (int j = 0; j < RL_ITEMS; ++j) {
    const i64 g = g_warp + j * 32 + lane;
    live[j] = g < n;
    first[j] = false;
    if (live[j]) {
      it[j] = fetch_item(p, g, b_warp);
      first[j] = it[j].ok && __ldg(p.min_idx + g) == it[j].idx;
    }
    const unsigned m = __ballot_sync(0xffffffffu, first[j]);
    before[j] = warp_firsts + __popc(m & lt_mask);
    warp_firsts += __popc(m);
  }
  if (lane == 0) s_warp[wid] = warp_firsts;
  __syncthreads();
  i64 wbase = p.tile_count[tile];
  for (int w = 0; w < wid; ++w) wbase += s_warp[w];
  const bool fits = (i64)p.tile_count[tiles] <= p.U_cap;
#pragma unroll
  for (int j = 0; j < RL_ITEMS; ++j) {
    if (!live[j]) continue;
    const i64 g = g_warp + j * 32 + lane;
    const i64 run = wbase + before[j];
    if (it[j].idx == 0) {
      // first item of its minibatch: the running count is the minibatch's
      // offset; empty minibatches directly before it share the same value
      int b = it[j].b;
      p.unique_ptr[b] = run;
      while (b > 0 && p.item_ptr[b - 1] == g) p.unique_ptr[--b] = run;
    }
    if (first[j]) {
      if (fits) p.unique[run] = (i64)it[j].key;
      p.rank[g] = (u32)run;
    }
  }
  if (tile == tiles - 1 && threadIdx.x == 0) {
    const i64 grand = p.tile_count[tiles];
    int b = p.B;
    p.unique_ptr[b] = grand;
    while (b > 0 && p.item_ptr[b - 1] == n) p.unique_ptr[--b] = grand;
  }
}

// Thread per edge.  Position of an id = rank[first item carrying it]; for an
// id seen for the first time on this very edge that is the edge's own item, so
// two thirds of the gathers of a GraphSAGE layer are in fact coalesced.
__global__ void __launch_bounds__(RL_THREADS) relabel_emit_kernel(const RelabelParams p) {
  const i64 n = p.hdr->n_edges;
  const int lane = threadIdx.x & 31;
  for (i64 e = (i64)blockIdx.x * RL_THREADS + threadIdx.x; e < n; e += (i64)gridDim.x * RL_THREADS) {
    int b = find_segment(p.edge_ptr, p.B, e - lane);  // warp-uniform start
    while (e >= p.edge_ptr[b + 1]) ++b;
    const i64 ibase = p.item_ptr[b];
    const i64 s0 = p.seeds_ptr[b], ns = p.seeds_ptr[b + 1] - s0;
    const i64 ubase = p.unique_ptr[b];
    const u32 m = __ldg(p.min_idx + ibase + ns + (e - p.edge_ptr[b]));
    const i64 c = __ldg(p.coo_col + e);
    i64 r = -1, cc = -1;
    if (m != IDX_UNSET) r = (i64)__ldg(p.rank + ibase + m) - ubase;
    if (c >= s0 && c < s0 + ns) {
      const u32 mc = __ldg(p.min_idx + ibase + (c - s0));
      if (mc != IDX_UNSET) cc = (i64)__ldg(p.rank + ibase + mc) - ubase;
    } else {
      raise(p.err, ERRBIT_BAD_INPUT);  // a column slot outside the edge's own minibatch
    }
    p.out_row[e] = r;
    p.out_col[e] = cc;
  }
}

struct RelabelLayout {
  size_t hdr, item_ptr, table_ptr, tile_count, min_idx, rank, table, total;
  i64 slots_cap, tiles;
};

// Direct-address tables are used when they need no more memory than hashing.
static bool use_direct(i64 S_max, i64 E_max, i64 B, i64 id_bound) {
  if (id_bound <= 0 || id_bound >= 0xFFFFFFFFll) return false;
  const i64 hash_words = (S_max + E_max) * 2 + 32 * (B + 1);          // 64-bit words
  return (id_bound * B + 1) / 2 <= hash_words;
}

static RelabelLayout relabel_layout(i64 S_max, i64 E_max, i64 B) {
  RelabelLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.tiles = (S_max + E_max + RL_TILE - 1) / RL_TILE + 1;
  L.slots_cap = (S_max + E_max) * 2 + 32 * (B + 1);
  size_t o = 0;
  L.hdr = o; o = up(o + sizeof(RelabelHeader));
  L.item_ptr = o; o = up(o + sizeof(i64) * (size_t)(B + 1));
  L.table_ptr = o; o = up(o + sizeof(i64) * (size_t)(B + 1));
  L.tile_count = o; o = up(o + sizeof(u32) * (size_t)(L.tiles + 1));
  L.min_idx = o; o = up(o + sizeof(u32) * (size_t)(S_max + E_max + 4));
  L.rank = o; o = up(o + sizeof(u32) * (size_t)(S_max + E_max + 4));
  L.table = o; o = up(o + sizeof(u64) * (size_t)L.slots_cap);
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
  p.S_max = S_max; p.E_max = E_max; p.unique = (i64*)unique; p.U_cap = U_cap;
  p.unique_ptr = (i64*)unique_ptr; p.out_row = (i64*)out_row; p.out_col = (i64*)out_col;
  p.hdr = (RelabelHeader*)(ws + L.hdr); p.item_ptr = (i64*)(ws + L.item_ptr);
  p.table_ptr = (i64*)(ws + L.table_ptr); p.tile_count = (u32*)(ws + L.tile_count);
  p.min_idx = (u32*)(ws + L.min_idx); p.rank = (u32*)(ws + L.rank);
  p.table = (u64*)(ws + L.table); p.slots_cap = L.slots_cap; p.tiles_cap = L.tiles; p.err = d_err;
  p.direct_bound = use_direct(S_max, E_max, B, id_bound) ? id_bound : 0;

  { LaunchScope ls(KID_RL_SETUP, st); relabel_setup_kernel<<<1, 1024, 0, st>>>(p); }
  const i64 items_max = S_max + E_max;
  const int wide = 148 * 8;
  int g_clear = (int)((L.slots_cap / 2 + RL_THREADS - 1) / RL_THREADS); if (g_clear > wide) g_clear = wide; if (g_clear < 1) g_clear = 1;
  { LaunchScope ls(KID_RL_CLEAR, st); relabel_clear_kernel<<<g_clear, RL_THREADS, 0, st>>>(p); }
  int g_items = (int)((items_max + RL_THREADS - 1) / RL_THREADS); if (g_items < 1) g_items = 1;
  if (g_items > 148 * 16) g_items = 148 * 16;
  { LaunchScope ls(KID_RL_INSERT, st); relabel_insert_kernel<<<g_items, RL_THREADS, 0, st>>>(p); }
  { LaunchScope ls(KID_RL_LOOKUP, st); relabel_lookup_kernel<<<g_items, RL_THREADS, 0, st>>>(p); }
  { LaunchScope ls(KID_RL_TILES, st); relabel_tiles_kernel<<<1, 1024, 0, st>>>(p); }
  { LaunchScope ls(KID_RL_SCAN, st); relabel_rank_kernel<<<(int)L.tiles, RL_THREADS, 0, st>>>(p); }
  if (out_row && E_max > 0) {
    int g_edges = (int)((E_max + RL_THREADS - 1) / RL_THREADS);
    if (g_edges > 148 * 16) g_edges = 148 * 16;
    { LaunchScope ls(KID_RL_EDGES, st); relabel_emit_kernel<<<g_edges, RL_THREADS, 0, st>>>(p); }
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
