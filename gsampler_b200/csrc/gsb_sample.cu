// Per-column fanout sampling fused with column slicing (uniform).
//
// One CTA owns a tile of consecutive column slots.  Phase 1 (thread per
// column) reads the seed and its indptr pair and derives the pick count; a
// block scan plus the chained tile prefix turns the counts into global output
// offsets in the same pass (no separate degree/scan kernels, no host read of
// the edge count).  Phase 2 (thread per column) chooses the in-column
// positions into shared memory.  Phase 3 (thread per OUTPUT edge) gathers the
// row ids and writes the three output arrays fully coalesced: consecutive
// threads write consecutive output elements, whatever the degree skew.
#include <atomic>

#include "gsb_common.cuh"

namespace gsb {

#ifndef GSB_SAMPLE_THREADS
#define GSB_SAMPLE_THREADS 256
#endif
constexpr int SAMPLE_THREADS = GSB_SAMPLE_THREADS;
#ifndef GSB_SAMPLE_MIN_CTAS
#define GSB_SAMPLE_MIN_CTAS 8  // 32 registers/thread: eight resident CTAs (2048 threads) per SM.
                               // Measured on the layer-3 launch: 72 regs 0.55 ms, 40 regs 0.41 ms,
                               // 32 regs 0.38 ms -- the kernel hides DRAM latency with occupancy.
#endif
constexpr int SAMPLE_MAX_TILE_EDGES = 8192;  // picks staged in shared memory per tile

struct SampleParams {
  const i64* indptr;
  const void* indices;
  i64 num_cols;      // columns of the graph: a seed outside [0, num_cols) is reported, never read
  const i64* seeds;  // nullable
  i64 S_max;
  const i64* d_S;    // nullable
  int K;
  int replace;
  u64 seed;
  u32 stream;
  i64* sub_indptr;
  i64* out_rows;
  i64* out_cols;  // nullable
  i64* out_sel;
  i64 E_cap;
  i64* d_num_edges;  // nullable
  u64* status;       // chained-prefix words, zeroed
  int* ticket;       // tile ticket counter, zeroed
  int* err;
  int tile_cols;
  // layered sampler only: the minibatch offsets of the column slots and a second column output,
  // the slot counted from its minibatch's first slot (= the relabelled column of the block when
  // the minibatch's seeds are distinct)
  const i64* seeds_ptr;  // nullable
  int B;
  i64* out_block_col;    // nullable
};

// HINT: 0 plain loads and stores; 1 column offsets loaded evict-last; 2 + output stores
// evict-first; 3 + the gathered row ids evict-first
template <typename IndexT, int HINT>
__global__ void __launch_bounds__(SAMPLE_THREADS, GSB_SAMPLE_MIN_CTAS)
sample_tile_kernel(const SampleParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tc = p.tile_cols;
  const int K = p.K;
  // shared layout: in_start[tc] i64 | scan scratch[33] i64 | picks[tc*K] u32 |
  //                 tmp[tc*K] u32 | lcol[tc] u32 | owner[tc*K] u8
  i64* s_in_start = reinterpret_cast<i64*>(smem_raw);
  i64* s_scan = s_in_start + tc;
  u32* s_pick = reinterpret_cast<u32*>(s_scan + 34);
  u32* s_tmp = s_pick + (size_t)tc * K;
  u32* s_lcol = s_tmp + (size_t)tc * K;
  unsigned char* s_owner = reinterpret_cast<unsigned char*>(s_lcol + tc);
  __shared__ int s_tile, s_b0;
  __shared__ i64 s_base;

  if (threadIdx.x == 0) s_tile = atomicAdd(p.ticket, 1);
  __syncthreads();
  const int tile = s_tile;
  i64 S = p.S_max;
  if (p.d_S) {
    const i64 live = *p.d_S;
    if (live > S && tile == 0 && threadIdx.x == 0) raise(p.err, ERRBIT_CAPACITY);
    S = live < S ? (live < 0 ? 0 : live) : S;
  }
  const i64 num_tiles = S == 0 ? 1 : (S + tc - 1) / tc;
  if (tile >= num_tiles) return;
  u64 keep = 0, stream = 0;
  if (HINT >= 1) keep = l2_policy_keep();
  if (HINT >= 2) stream = l2_policy_stream();

  const int lc = threadIdx.x;
  const i64 slot = (i64)tile * tc + lc;
  const bool valid = lc < tc && slot < S;
  if (p.out_block_col && threadIdx.x == 0) s_b0 = find_segment(p.seeds_ptr, p.B, (i64)tile * tc);
  i64 in_start = 0;
  u32 deg = 0;
  int cnt = 0;
  if (valid) {
    const i64 c = p.seeds ? p.seeds[slot] : slot;
    i64 d = 0;
    if ((u64)c < (u64)p.num_cols) {
      if (HINT >= 1) {
        in_start = ld_i64_keep(p.indptr + c, keep);
        d = ld_i64_keep(p.indptr + c + 1, keep) - in_start;
      } else {
        in_start = __ldg(p.indptr + c);
        d = __ldg(p.indptr + c + 1) - in_start;
      }
    }
    if ((u64)c >= (u64)p.num_cols || d < 0 || d > 0xFFFFFFFFll) {  // bad seed / offsets: an empty column
      raise(p.err, ERRBIT_BAD_INPUT);
      d = 0;
    }
    deg = (u32)d;
    cnt = p.replace ? (d == 0 ? 0 : K) : (d < (i64)K ? (int)d : K);
    s_in_start[lc] = in_start;
  }
  i64 total;
  const i64 loff = block_exclusive_scan((i64)cnt, s_scan, &total);  // (its barriers publish s_b0)
  if (p.out_block_col && valid) {
    // the slot counted from its minibatch's first slot; a tile rarely crosses a boundary
    int b = s_b0;
    while (b + 1 < p.B && slot >= __ldg(p.seeds_ptr + b + 1)) ++b;
    s_lcol[lc] = (u32)(slot - __ldg(p.seeds_ptr + b));
  }
  if (threadIdx.x < 32) {
    i64 base = chained_exclusive_prefix(p.status, tile, total, p.err);
    if (threadIdx.x == 0) s_base = base;
  }
  // Phase 2: choose positions inside the column (thread per column).
  if (valid && cnt > 0) {
    const int o = (int)loff;
    if (p.replace) {
      Philox4 blk;
      for (int k = 0; k < K; ++k) {
        if ((k & 3) == 0) blk = stream_block(p.seed, p.stream, (u64)slot, (u32)k >> 2);
        s_pick[o + k] = __umulhi(pick_word(blk, k), deg);
        s_owner[o + k] = (unsigned char)lc;
      }
    } else if (deg <= (u32)K) {
      for (int k = 0; k < cnt; ++k) {
        s_pick[o + k] = (u32)k;
        s_owner[o + k] = (unsigned char)lc;
      }
    } else {
      // Floyd's subset selection: pick k is a uniform draw from [0, deg-K+k],
      // replaced by deg-K+k itself when that value was already taken.  The
      // running set lives in a transposed shared array (bank = column).
      Philox4 blk;
      for (int k = 0; k < K; ++k) {
        if ((k & 3) == 0) blk = stream_block(p.seed, p.stream, (u64)slot, (u32)k >> 2);
        const u32 j = deg - (u32)K + (u32)k;
        const u32 t = __umulhi(pick_word(blk, k), j + 1u);
        bool dup = false;
        for (int m = 0; m < k; ++m) dup |= (s_tmp[m * tc + lc] == t);
        const u32 v = dup ? j : t;
        s_tmp[k * tc + lc] = v;
        s_pick[o + k] = v;
        s_owner[o + k] = (unsigned char)lc;
      }
    }
  }
  __syncthreads();
  const i64 base = s_base;
  if (valid) p.sub_indptr[slot] = base + loff;
  if (tile == num_tiles - 1 && threadIdx.x == 0) {
    p.sub_indptr[S] = base + total;
    if (p.d_num_edges) *p.d_num_edges = base + total;
  }
  if (base + total > p.E_cap) {
    if (threadIdx.x == 0) raise(p.err, ERRBIT_CAPACITY);
    return;
  }
  // Phase 3: thread per output edge, coalesced stores.
  const i64 col0 = (i64)tile * tc;
  for (int o = threadIdx.x; o < (int)total; o += SAMPLE_THREADS) {
    const int c = s_owner[o];
    const i64 pos = s_in_start[c] + (i64)s_pick[o];
    const i64 row = HINT >= 3 ? load_index_stream<IndexT>(p.indices, pos, stream)
                              : load_index<IndexT>(p.indices, pos);
    if (HINT >= 2) {
      st_i64_stream(p.out_rows + base + o, row, stream);
      st_i64_stream(p.out_sel + base + o, pos, stream);
      if (p.out_cols) st_i64_stream(p.out_cols + base + o, col0 + c, stream);
      if (p.out_block_col) st_i64_stream(p.out_block_col + base + o, (i64)s_lcol[c], stream);
    } else {
      p.out_rows[base + o] = row;
      p.out_sel[base + o] = pos;
      if (p.out_cols) p.out_cols[base + o] = col0 + c;
      if (p.out_block_col) p.out_block_col[base + o] = (i64)s_lcol[c];
    }
  }
}

// Column slots per tile (CTA).  `S_geom` = the number of slots the launch is laid out for: with
// few of them the tiles shrink (down to 64 slots) so that every SM still gets several rounds
// of CTAs -- the first layer of a 32 x 1024-seed super-batch is 128 tiles of 256 slots
// otherwise, fewer CTAs than the GPU has SMs.  Results do not depend on the tile size (the random streams are
// keyed by slot).
// Tiles per SM below which the tiles shrink: 16 = two rounds of the 8 CTAs an SM holds.  The
// second layer of the benchmark (410 k slots) is 1600 tiles of 256 slots -- one full round of
// resident CTAs and a second one a third full -- or 3200 tiles of 128: 1.007 -> 0.986 ms per
// step (threshold 4 -> 16; 32 halves the tiles once more and loses: 1.017 ms).
#ifndef GSB_SAMPLE_MIN_TILES_PER_SM
#define GSB_SAMPLE_MIN_TILES_PER_SM 16
#endif
static int sample_tile_cols(i64 K, i64 S_geom = -1) {
  i64 tc = SAMPLE_MAX_TILE_EDGES / K;
  if (tc > SAMPLE_THREADS) tc = SAMPLE_THREADS;
  if (tc < 1) tc = 1;
  if (S_geom >= 0)
    while (tc > 64 && (S_geom + tc - 1) / tc < GSB_SAMPLE_MIN_TILES_PER_SM * (i64)sm_count()) tc >>= 1;
  return (int)tc;
}

static size_t sample_smem_bytes(int tc, i64 K) {
  return sizeof(i64) * (size_t)(tc + 34) + (size_t)tc * K * (4 + 4 + 1) + 4 * (size_t)tc + 16;
}

}  // namespace gsb

using namespace gsb;

extern "C" size_t gsb_sample_cols_workspace_bytes(int64_t S_max, int64_t K) {
  if (S_max < 0 || K < 1) return 0;
  int tc = sample_tile_cols(K, S_max);
  size_t tiles = (size_t)((S_max + tc - 1) / tc) + 1;
  return 256 + tiles * sizeof(u64);
}

namespace gsb {

// Cache-hint level of the sampling kernel (see sample_tile_kernel).  Measured on the 2.45 M-node /
// 123.7 M-edge benchmark graph, last layer (3.7 M columns, fanout 5), per launch: level 0 0.384 ms,
// 1 0.363, 2 0.344, 3 0.357 -- keeping the offsets in L2 and streaming the stores pays, marking
// the row-id gather as a stream as well takes back part of it.
#ifndef GSB_SAMPLE_HINT
#define GSB_SAMPLE_HINT 2
#endif

template <typename IndexT>
static int launch_sample(const SampleParams& p, int tiles, size_t smem, cudaStream_t st) {
  GSB_CUDA_OK(cudaFuncSetAttribute(sample_tile_kernel<IndexT, GSB_SAMPLE_HINT>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LaunchScope ls(KID_SAMPLE, st);
  sample_tile_kernel<IndexT, GSB_SAMPLE_HINT><<<tiles, SAMPLE_THREADS, smem, st>>>(p);
  return GSB_OK;
}

int sample_launch(const int64_t* indptr, const void* indices, int indices_dtype, int64_t num_cols,
                  const int64_t* seeds, int64_t S_max, const int64_t* d_S, int64_t K, int replace,
                  uint64_t seed, uint32_t stream, int64_t* sub_indptr, int64_t* out_rows,
                  int64_t* out_cols, int64_t* out_sel, int64_t E_cap, int64_t* d_num_edges,
                  const int64_t* seeds_ptr, int64_t B, int64_t* out_block_col, int64_t S_geom,
                  void* workspace, size_t workspace_bytes, int* d_err, void* cuda_stream) {
  if (S_geom < S_max) S_geom = S_max;
  if (!indptr || !indices || !sub_indptr || S_max < 0 || E_cap < 0 || num_cols < 0) return GSB_ERR_INVALID;
  if (E_cap > 0 && (!out_rows || !out_sel)) return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  if (K < 1) return GSB_ERR_INVALID;
  if (K > SAMPLE_MAX_TILE_EDGES) return GSB_ERR_UNSUPPORTED;
  if (out_block_col && (!seeds_ptr || B < 1)) return GSB_ERR_INVALID;
  if (workspace_bytes < gsb_sample_cols_workspace_bytes(S_geom, K) || !workspace)
    return GSB_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  const int tc = sample_tile_cols(K, S_geom);
  const int tiles = S_max == 0 ? 1 : ceil_div_i(S_max, tc);
  GSB_CUDA_OK(cudaMemsetAsync(workspace, 0, 256 + (size_t)(tiles + 1) * sizeof(u64), st));
  SampleParams p;
  p.indptr = (const i64*)indptr; p.indices = indices; p.num_cols = num_cols; p.seeds = (const i64*)seeds;
  p.S_max = S_max; p.d_S = (const i64*)d_S; p.K = (int)K; p.replace = replace ? 1 : 0;
  p.seed = seed; p.stream = stream; p.sub_indptr = (i64*)sub_indptr; p.out_rows = (i64*)out_rows;
  p.out_cols = (i64*)out_cols; p.out_sel = (i64*)out_sel; p.E_cap = E_cap;
  p.d_num_edges = (i64*)d_num_edges;
  p.ticket = (int*)workspace;
  p.status = (u64*)((char*)workspace + 256);
  p.err = d_err; p.tile_cols = tc;
  p.seeds_ptr = (const i64*)seeds_ptr; p.B = (int)B; p.out_block_col = (i64*)out_block_col;
  const size_t smem = sample_smem_bytes(tc, K);
  const int rc = indices_dtype == GSB_I32 ? launch_sample<int>(p, tiles, smem, st)
                                          : launch_sample<i64>(p, tiles, smem, st);
  if (rc != GSB_OK) return rc;
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

}  // namespace gsb

extern "C" int gsb_sample_cols(const int64_t* indptr, const void* indices, int indices_dtype,
                               int64_t num_cols, const int64_t* seeds, int64_t S_max,
                               const int64_t* d_S, int64_t K,
                               int replace, uint64_t seed, uint32_t stream, int64_t* sub_indptr,
                               int64_t* out_rows, int64_t* out_cols, int64_t* out_sel,
                               int64_t E_cap, int64_t* d_num_edges, void* workspace,
                               size_t workspace_bytes, int* d_err, void* cuda_stream) {
  return gsb::sample_launch(indptr, indices, indices_dtype, num_cols, seeds, S_max, d_S, K, replace, seed,
                            stream, sub_indptr, out_rows, out_cols, out_sel, E_cap, d_num_edges, nullptr,
                            0, nullptr, S_max, workspace, workspace_bytes, d_err, cuda_stream);
}

// ---------------------------------------------------------------- fixed-scratch variant
// Some callers may not allocate device memory at all: a plugin that runs inside
// a host application's memory budget and is handed only its input and output
// buffers, or a service thread that must stay off the allocator because
// cudaMalloc/cudaFree synchronise the whole device and would stall the other
// streams of the process.  For them the tile ticket and the chained-prefix
// status words of the sampling kernel live in the array below instead of a
// caller-provided workspace.  Every GPU that loads the library holds these
// bytes until the process exits.
constexpr long long NOALLOC_MAX_TILES = 65536;  // 16.7 M column slots at fanout <= 32
constexpr size_t NOALLOC_SCRATCH_BYTES = 256 + (size_t)(NOALLOC_MAX_TILES + 1) * sizeof(unsigned long long);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
// device address of the array, per device; written once per device, read by any host thread
std::atomic<void*> g_noalloc_ptr[NOALLOC_MAX_DEVICES];
}  // namespace

extern "C" int64_t gsb_sample_cols_noalloc_max_columns(int64_t K) {
  if (K < 1 || K > gsb::SAMPLE_MAX_TILE_EDGES) return 0;
  return NOALLOC_MAX_TILES * (int64_t)gsb::sample_tile_cols(K);
}

extern "C" int gsb_sample_cols_noalloc(const int64_t* indptr, const void* indices,
                                       int indices_dtype, int64_t num_cols, const int64_t* seeds,
                                       int64_t S_max,
                                       const int64_t* d_S, int64_t K, int replace, uint64_t seed,
                                       uint32_t stream, int64_t* sub_indptr, int64_t* out_rows,
                                       int64_t* out_cols, int64_t* out_sel, int64_t E_cap,
                                       int64_t* d_num_edges, int* d_err, void* cuda_stream) {
  if (K < 1 || S_max < 0) return GSB_ERR_INVALID;
  if (K > gsb::SAMPLE_MAX_TILE_EDGES) return GSB_ERR_UNSUPPORTED;
  // sizes beyond the fixed scratch are refused, never truncated
  if (S_max > gsb_sample_cols_noalloc_max_columns(K)) return GSB_ERR_SCRATCH_LIMIT;
  int dev = -1;
  GSB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return GSB_ERR_UNSUPPORTED;
  void* scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // first call on this device: resolve the array's DEVICE address.  In host
    // code the symbol's name is only a handle; passing it to a kernel would
    // hand the kernel a host address.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return GSB_ERR_CUDA;
    g_noalloc_ptr[dev].store(p, std::memory_order_release);  // every thread resolves the same address
    scratch = p;
  }
  // the scratch keeps the previous call's ticket and status words;
  // gsb_sample_cols zeroes the part it uses on the stream before the launch
  return gsb_sample_cols(indptr, indices, indices_dtype, num_cols, seeds, S_max, d_S, K, replace, seed, stream,
                         sub_indptr, out_rows, out_cols, out_sel, E_cap, d_num_edges,
                         scratch, NOALLOC_SCRATCH_BYTES, d_err, cuda_stream);
}
