// Per-minibatch first-occurrence unique + relabel (block construction).
//
// Every minibatch gets its own open-addressing table; the tables sit back to
// back in the workspace and are sized from the minibatch's item count, so a
// table that is being built or probed (a few MB) stays resident in the 126 MB
// L2 while the grid walks the minibatches in order.  A slot is ONE 64-bit
// word: key in the high half, payload in the low half --
//   after insert   : payload = smallest item index that carries the key
//                    (atomicMin on the whole word; the key half is equal for
//                    all contenders, so the minimum is the minimum index),
//   after the scan : payload = 0x80000000 | position of the key in `unique`.
// The item whose index equals the payload is the first occurrence; a chained
// tile prefix over the first-occurrence flags yields its output position in
// the same pass that writes `unique`, with no separate flag array or scan.
#include "gsb_common.cuh"

namespace gsb {

constexpr int RL_THREADS = 256;
constexpr int RL_ITEMS = 4;
constexpr int RL_TILE = RL_THREADS * RL_ITEMS;
constexpr u64 SLOT_EMPTY = ~0ull;
constexpr u32 SLOT_FINAL = 0x80000000u;

struct RelabelHeader {
  int ticket;
  int pad;
  i64 n_items;
  i64 n_slots;
  i64 n_edges;
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
  i64* item_ptr;   // [B+1] start of minibatch b in the interleaved item order
  i64* table_ptr;  // [B+1] start of minibatch b's table
  u64* status;
  u64* table;
  i64 slots_cap;
  int* err;
};

__host__ __device__ inline i64 table_slots_for(i64 items) { return items + (items >> 2) + 32; }

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
    if (n_items > p.S_max + p.E_max || n_slots > p.slots_cap || p.seeds_ptr[p.B] > p.S_max ||
        p.edge_ptr[p.B] > p.E_max) {
      raise(p.err, ERRBIT_CAPACITY);
      n_items = 0; n_slots = 0;  // later kernels become no-ops
    }
    p.item_ptr[p.B] = n_items;
    p.table_ptr[p.B] = n_slots;
    p.hdr->ticket = 0;
    p.hdr->n_items = n_items;
    p.hdr->n_slots = n_slots;
    p.hdr->n_edges = n_items == 0 ? 0 : p.edge_ptr[p.B];
  }
}

__global__ void relabel_clear_kernel(const RelabelParams p) {
  const i64 n = p.hdr->n_slots;
  // 16-byte stores; the table base is 256-byte aligned
  ulonglong2* t2 = reinterpret_cast<ulonglong2*>(p.table);
  const i64 n2 = n >> 1;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += (i64)gridDim.x * blockDim.x)
    t2[i] = make_ulonglong2(SLOT_EMPTY, SLOT_EMPTY);
  if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) p.table[n - 1] = SLOT_EMPTY;
}

struct Item {
  int b;
  u32 key;
  u32 idx;
  bool ok;
};

__device__ __forceinline__ Item fetch_item(const RelabelParams& p, i64 g) {
  Item it;
  it.b = find_segment(p.item_ptr, p.B, g);
  const i64 off = g - p.item_ptr[it.b];
  const i64 s0 = p.seeds_ptr[it.b];
  const i64 ns = p.seeds_ptr[it.b + 1] - s0;
  const i64 key = off < ns ? p.seeds[s0 + off] : p.coo_row[p.edge_ptr[it.b] + (off - ns)];
  it.ok = key >= 0 && key < 0xFFFFFFFFll;
  it.key = (u32)key;
  it.idx = (u32)off;
  return it;
}

__global__ void __launch_bounds__(RL_THREADS) relabel_insert_kernel(const RelabelParams p) {
  const i64 n = p.hdr->n_items;
  for (i64 g = (i64)blockIdx.x * RL_THREADS + threadIdx.x; g < n; g += (i64)gridDim.x * RL_THREADS) {
    const Item it = fetch_item(p, g);
    if (!it.ok) { raise(p.err, ERRBIT_BAD_INPUT); continue; }
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

// slot index (relative to the minibatch table) holding `key`, or -1
template <bool READ_ONLY>
__device__ __forceinline__ i64 find_slot(const u64* tab, u32 slots, u32 key, u64* word) {
  u32 pos = __umulhi(hash32(key), slots);
  for (u32 probes = 0; probes < slots; ++probes) {
    const u64 cur = READ_ONLY ? __ldg(tab + pos) : ld_relaxed(tab + pos);
    if ((u32)(cur >> 32) == key && cur != SLOT_EMPTY) { *word = cur; return pos; }
    if (cur == SLOT_EMPTY) return -1;
    pos = pos + 1 == slots ? 0 : pos + 1;
  }
  return -1;
}

__global__ void __launch_bounds__(RL_THREADS, 6) relabel_scan_kernel(const RelabelParams p) {
  __shared__ i64 s_scan[34];
  __shared__ int s_tile;
  __shared__ i64 s_base;
  if (threadIdx.x == 0) s_tile = atomicAdd(&p.hdr->ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  const i64 n = p.hdr->n_items;
  const i64 tiles = n == 0 ? 1 : (n + RL_TILE - 1) / RL_TILE;
  if (tile >= tiles) return;

  i64 slot_addr[RL_ITEMS];
  u32 keys[RL_ITEMS];
  int batch[RL_ITEMS];
  bool first[RL_ITEMS], head[RL_ITEMS];
  int nfirst = 0;
  const i64 g0 = (i64)tile * RL_TILE + (i64)threadIdx.x * RL_ITEMS;
#pragma unroll
  for (int j = 0; j < RL_ITEMS; ++j) {
    first[j] = false; head[j] = false; slot_addr[j] = -1; keys[j] = 0; batch[j] = 0;
    const i64 g = g0 + j;
    if (g < n) {
      const Item it = fetch_item(p, g);
      batch[j] = it.b;
      head[j] = it.idx == 0;
      if (it.ok) {
        const i64 base = p.table_ptr[it.b];
        const u32 slots = (u32)(p.table_ptr[it.b + 1] - base);
        u64 w = 0;
        const i64 pos = find_slot<false>(p.table + base, slots, it.key, &w);
        if (pos < 0) {
          raise(p.err, ERRBIT_KEY_MISSING);
        } else {
          first[j] = !((u32)w & SLOT_FINAL) && (u32)w == it.idx;
          slot_addr[j] = base + pos;
          keys[j] = it.key;
        }
      }
      nfirst += first[j] ? 1 : 0;
    }
  }
  i64 total;
  const i64 loff = block_exclusive_scan((i64)nfirst, s_scan, &total);
  if (threadIdx.x < 32) {
    i64 base = chained_exclusive_prefix(p.status, tile, total, p.err);
    if (threadIdx.x == 0) s_base = base;
  }
  __syncthreads();
  i64 run = s_base + loff;
#pragma unroll
  for (int j = 0; j < RL_ITEMS; ++j) {
    const i64 g = g0 + j;
    if (g >= n) break;
    if (head[j]) {
      // first item of its minibatch: the running prefix is the minibatch's
      // offset; empty minibatches directly before it share the same value
      int b = batch[j];
      p.unique_ptr[b] = run;
      while (b > 0 && p.item_ptr[b - 1] == g) p.unique_ptr[--b] = run;
    }
    if (first[j]) {
      if (run < p.U_cap && run < (i64)SLOT_FINAL) {
        p.unique[run] = (i64)keys[j];
        st_relaxed(p.table + slot_addr[j], ((u64)keys[j] << 32) | SLOT_FINAL | (u32)run);
      } else {
        raise(p.err, ERRBIT_CAPACITY);
      }
      ++run;
    }
  }
  if (tile == tiles - 1 && threadIdx.x == 0) {
    const i64 grand = s_base + total;
    int b = p.B;
    p.unique_ptr[b] = grand;
    while (b > 0 && p.item_ptr[b - 1] == n) p.unique_ptr[--b] = grand;
  }
}

__global__ void __launch_bounds__(RL_THREADS) relabel_edges_kernel(const RelabelParams p) {
  const i64 n = p.hdr->n_edges;
  // last minibatch first: the scan pass ended there, its tables are in L2
  for (i64 t = (i64)blockIdx.x * RL_THREADS + threadIdx.x; t < n; t += (i64)gridDim.x * RL_THREADS) {
    const i64 e = n - 1 - t;
    const int b = find_segment(p.edge_ptr, p.B, e);
    const i64 base = p.table_ptr[b];
    const u32 slots = (u32)(p.table_ptr[b + 1] - base);
    const i64 ubase = p.unique_ptr[b];
    const i64 rk = p.coo_row[e];
    const i64 ck = p.seeds[p.coo_col[e]];
    u64 w = 0;
    i64 r = -1, c = -1;
    if (find_slot<true>(p.table + base, slots, (u32)rk, &w) >= 0) r = (i64)((u32)w & ~SLOT_FINAL) - ubase;
    if (find_slot<true>(p.table + base, slots, (u32)ck, &w) >= 0) c = (i64)((u32)w & ~SLOT_FINAL) - ubase;
    if (r < 0 || c < 0) raise(p.err, ERRBIT_KEY_MISSING);
    p.out_row[e] = r;
    p.out_col[e] = c;
  }
}

struct RelabelLayout {
  size_t hdr, item_ptr, table_ptr, status, table, total;
  i64 slots_cap, tiles;
};

static RelabelLayout relabel_layout(i64 S_max, i64 E_max, i64 B) {
  RelabelLayout L;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  L.tiles = (S_max + E_max + RL_TILE - 1) / RL_TILE + 1;
  L.slots_cap = (S_max + E_max) + ((S_max + E_max) >> 2) + 32 * (B + 1);
  size_t o = 0;
  L.hdr = o; o = up(o + sizeof(RelabelHeader));
  L.item_ptr = o; o = up(o + sizeof(i64) * (size_t)(B + 1));
  L.table_ptr = o; o = up(o + sizeof(i64) * (size_t)(B + 1));
  L.status = o; o = up(o + sizeof(u64) * (size_t)L.tiles);
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
  p.table_ptr = (i64*)(ws + L.table_ptr); p.status = (u64*)(ws + L.status);
  p.table = (u64*)(ws + L.table); p.slots_cap = L.slots_cap; p.err = d_err;

  GSB_CUDA_OK(cudaMemsetAsync(ws + L.status, 0, sizeof(u64) * (size_t)L.tiles, st));
  { LaunchScope ls(KID_RL_SETUP, st); relabel_setup_kernel<<<1, 1024, 0, st>>>(p); }
  const i64 items_max = S_max + E_max;
  const int wide = 148 * 8;
  int g_clear = (int)((L.slots_cap / 2 + RL_THREADS - 1) / RL_THREADS); if (g_clear > wide) g_clear = wide; if (g_clear < 1) g_clear = 1;
  { LaunchScope ls(KID_RL_CLEAR, st); relabel_clear_kernel<<<g_clear, RL_THREADS, 0, st>>>(p); }
  int g_items = (int)((items_max + RL_THREADS - 1) / RL_THREADS); if (g_items < 1) g_items = 1;
  if (g_items > 148 * 16) g_items = 148 * 16;
  { LaunchScope ls(KID_RL_INSERT, st); relabel_insert_kernel<<<g_items, RL_THREADS, 0, st>>>(p); }
  { LaunchScope ls(KID_RL_SCAN, st); relabel_scan_kernel<<<(int)L.tiles, RL_THREADS, 0, st>>>(p); }
  if (out_row && E_max > 0) {
    int g_edges = (int)((E_max + RL_THREADS - 1) / RL_THREADS);
    if (g_edges > 148 * 16) g_edges = 148 * 16;
    { LaunchScope ls(KID_RL_EDGES, st); relabel_edges_kernel<<<g_edges, RL_THREADS, 0, st>>>(p); }
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
