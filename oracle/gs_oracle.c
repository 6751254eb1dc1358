/*
 * CPU restatement of gSampler's matrix-centric sampling hot path.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the parity checker for the CUDA
 * library and the timed CPU baseline of the benchmark; nothing in the shipped
 * package links, loads or calls it.
 *
 * Every function names the reference file:line whose behaviour it restates
 * (paths are relative to the gSampler source tree).  The reference itself is
 * CUDA-only (its src/cpu holds one per-column sort), so this file is a port of
 * the reference's algorithms to plain C + OpenMP, not the reference's own CPU
 * code.  Deterministic stages (slicing, offsets, unique, relabel, format
 * conversion, SpMM/SDDMM) are defined by their mathematical result and are
 * pinned by the reference's own gtest fixtures (see tests/golden).  Random
 * stages come in two flavours:
 *   *_ref  : the reference's algorithm (parallel reservoir, A-Res keys, ...)
 *            driven by the same Philox4x32-10 stream layout the reference
 *            requests from cuRAND; used for the statistical comparisons.
 *            Draw VALUES are not pinned by any reference test ("parity
 *            unpinned" for cuRAND output; only distributions are compared).
 *   *_spec : the counter-based sampler the CUDA kernels implement (Floyd's
 *            subset selection over Philox4x32-10 keyed by column slot), which
 *            the kernels must reproduce bit for bit.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef int64_t i64;
typedef uint64_t u64;
typedef uint32_t u32;

#define GO_API __attribute__((visibility("default")))

GO_API void go_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

GO_API int go_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* Philox4x32-10 (Salmon et al., SC'11) -- the generator both the reference  */
/* (via cuRAND, sampling.cu:55-56) and the CUDA kernels of this repo use.    */
/* ------------------------------------------------------------------------ */
GO_API void go_philox4x32_10(const u32 ctr[4], const u32 key[2], u32 out[4]) {
  u32 c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
  u32 k0 = key[0], k1 = key[1];
  for (int r = 0; r < 10; ++r) {
    u64 p0 = (u64)0xD2511F53u * c0;
    u64 p1 = (u64)0xCD9E8D57u * c2;
    u32 n0 = (u32)(p1 >> 32) ^ c1 ^ k0;
    u32 n1 = (u32)p1;
    u32 n2 = (u32)(p0 >> 32) ^ c3 ^ k1;
    u32 n3 = (u32)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* Draw number n of the stream owned by `slot` (a column slot, walker, list
 * element ...) under (seed, stream): word n%4 of the Philox block whose
 * counter is {slot_lo, slot_hi, n/4, stream}.  This is the "spec" stream
 * layout shared with the CUDA kernels. */
static inline u32 spec_draw(u64 seed, u32 stream, u64 slot, u32 n) {
  u32 ctr[4] = {(u32)slot, (u32)(slot >> 32), n >> 2, stream};
  u32 key[2] = {(u32)seed, (u32)(seed >> 32)};
  u32 out[4];
  go_philox4x32_10(ctr, key, out);
  return out[n & 3];
}

GO_API u32 go_spec_draw(u64 seed, u32 stream, u64 slot, u32 n) {
  return spec_draw(seed, stream, slot, n);
}

/* cuRAND's Philox4_32_10 stream as the reference requests it:
 * curand_init(seed, subsequence, 0) then successive curand() calls return the
 * four words of block 0, then block 1, ... with counter = {block, 0,
 * subsequence_lo, subsequence_hi} and key = seed.  (Layout restated from the
 * public description of cuRAND's Philox generator; the draw values are not
 * pinned by any reference test.) */
typedef struct {
  u32 key[2];
  u32 sub[2];
  u32 block;
  u32 have;
  u32 out[4];
} curand_philox_t;

static inline void curand_philox_init(curand_philox_t* s, u64 seed, u64 subsequence) {
  s->key[0] = (u32)seed; s->key[1] = (u32)(seed >> 32);
  s->sub[0] = (u32)subsequence; s->sub[1] = (u32)(subsequence >> 32);
  s->block = 0; s->have = 0;
}
static inline u32 curand_philox_next(curand_philox_t* s) {
  if (s->have == 0) {
    u32 ctr[4] = {s->block, 0, s->sub[0], s->sub[1]};
    go_philox4x32_10(ctr, s->key, s->out);
    s->block++;
    s->have = 4;
  }
  u32 v = s->out[4 - s->have];
  s->have--;
  return v;
}

/* ------------------------------------------------------------------------ */
/* Column slicing A[:, seeds]                                                */
/* reference: src/cuda/slicing.cu:100-167 (OnIndptrSlicing),                 */
/*            src/cuda/batch/slicing.cu:11-96 (batch flavour, id encoding)   */
/* ------------------------------------------------------------------------ */
GO_API void go_slice_cols_count(const i64* indptr, const i64* seeds, i64 S, i64* out_indptr) {
  /* slicing.cu:133-141: degree per seed, then exclusive scan over S+1 */
  i64 acc = 0;
  for (i64 i = 0; i < S; ++i) {
    out_indptr[i] = acc;
    acc += indptr[seeds[i] + 1] - indptr[seeds[i]];
  }
  out_indptr[S] = acc;
}

/* col_bptr/B/encoding_size: when encoding_size > 0 the row id written for a
 * column of minibatch b is indices + b*encoding_size (batch/slicing.cu:24-29).
 * out_col (may be NULL) = local column id (slicing.cu:113-115),
 * out_sel = global edge position (slicing.cu:112). */
GO_API void go_slice_cols_fill(const i64* indptr, const i64* indices, const i64* seeds, i64 S,
                               const i64* out_indptr, i64* out_indices, i64* out_col, i64* out_sel,
                               const i64* col_bptr, i64 B, i64 encoding_size) {
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 i = 0; i < S; ++i) {
    i64 in_start = indptr[seeds[i]];
    i64 o = out_indptr[i];
    i64 n = out_indptr[i + 1] - o;
    i64 enc = 0;
    if (encoding_size > 0 && col_bptr) {
      i64 b = 0;
      while (b + 1 < B && col_bptr[b + 1] <= i) ++b;
      enc = b * encoding_size;
    }
    for (i64 k = 0; k < n; ++k) {
      out_indices[o + k] = indices[in_start + k] + enc;
      out_sel[o + k] = in_start + k;
      if (out_col) out_col[o + k] = i;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Per-column fanout sampling (uniform)                                      */
/* reference: src/cuda/sampling.cu:111-124 (counts), :64-73 (copy-all),      */
/*            :75-97 (reservoir), :17-46 (with replacement);                 */
/*            fused with slicing: src/cuda/fusion/slice_sampling.cu:52-124.  */
/* seeds == NULL means "column i of the operand" (plain Sampling).           */
/* ------------------------------------------------------------------------ */
GO_API void go_sample_count(const i64* indptr, const i64* seeds, i64 S, i64 K, int replace,
                            i64* out_indptr) {
  i64 acc = 0;
  for (i64 i = 0; i < S; ++i) {
    i64 c = seeds ? seeds[i] : i;
    i64 deg = indptr[c + 1] - indptr[c];
    out_indptr[i] = acc;
    if (replace) acc += (deg == 0) ? 0 : K;       /* slice_sampling.cu:117-118 */
    else acc += deg < K ? deg : K;                /* slice_sampling.cu:120 */
  }
  out_indptr[S] = acc;
}

/* The sampler the CUDA kernels implement.  Column slot i (its index in the
 * launch's seed array) owns a Philox stream; draw k of it is used for pick k.
 *  - deg <= K           : copy all, in order (sampling.cu:64-73).
 *  - without replacement: Floyd's subset selection: for k in [0,K):
 *        j = deg-K+k; t = floor(draw_k * (j+1) / 2^32);
 *        pick_k = (t already picked) ? j : t.
 *    Uniform over K-subsets like the reference's reservoir, but needs K draws
 *    instead of deg-K.
 *  - with replacement   : pick_k = floor(draw_k * deg / 2^32).
 */
GO_API void go_sample_fill_spec(const i64* indptr, const i64* indices, const i64* seeds, i64 S,
                                i64 K, int replace, u64 seed, u32 stream, const i64* out_indptr,
                                i64* out_indices, i64* out_col, i64* out_sel) {
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 i = 0; i < S; ++i) {
    i64 c = seeds ? seeds[i] : i;
    i64 in_start = indptr[c];
    i64 deg = indptr[c + 1] - in_start;
    i64 o = out_indptr[i];
    i64 n = out_indptr[i + 1] - o;
    if (replace) {
      for (i64 k = 0; k < n; ++k) {
        u32 r = spec_draw(seed, stream, (u64)i, (u32)k);
        i64 pos = (i64)(((u64)r * (u64)deg) >> 32);
        out_sel[o + k] = in_start + pos;
      }
    } else if (deg <= K) {
      for (i64 k = 0; k < n; ++k) out_sel[o + k] = in_start + k;
    } else {
      for (i64 k = 0; k < K; ++k) {
        i64 j = deg - K + k;
        u32 r = spec_draw(seed, stream, (u64)i, (u32)k);
        i64 t = (i64)(((u64)r * (u64)(j + 1)) >> 32);
        int dup = 0;
        for (i64 m = 0; m < k; ++m)
          if (out_sel[o + m] == in_start + t) { dup = 1; break; }
        out_sel[o + k] = in_start + (dup ? j : t);
      }
    }
    for (i64 k = 0; k < n; ++k) {
      out_indices[o + k] = indices[out_sel[o + k]];
      if (out_col) out_col[o + k] = i;
    }
  }
}

/* The reference's sampler: block (16,32) threads, 32 columns per block, one
 * Philox stream per threadIdx.x seeded with seed*gridDim.x+blockIdx.x
 * (sampling.cu:54-56, slice_sampling.cu:49-50); parallel reservoir with
 * AtomicMax into the slot (sampling.cu:75-90).  Executed here lane by lane;
 * the result does not depend on the interleaving because max is commutative.
 * The 32 columns of a block share their 16 streams (threadIdx.y is not part
 * of the subsequence), exactly as in the reference. */
GO_API void go_sample_fill_ref(const i64* indptr, const i64* indices, const i64* seeds, i64 S,
                               i64 K, int replace, u64 random_seed, const i64* out_indptr,
                               i64* out_indices, i64* out_col, i64* out_sel) {
  const i64 BX = 16, BY = 32;
  i64 grid = (S + BY - 1) / BY;
#pragma omp parallel for schedule(dynamic, 8)
  for (i64 blk = 0; blk < grid; ++blk) {
    for (i64 y = 0; y < BY; ++y) {
      i64 i = blk * BY + y;
      if (i >= S) break;
      i64 c = seeds ? seeds[i] : i;
      i64 in_start = indptr[c];
      i64 deg = indptr[c + 1] - in_start;
      i64 o = out_indptr[i];
      i64 n = out_indptr[i + 1] - o;
      curand_philox_t rng[16];
      for (i64 x = 0; x < BX; ++x)
        curand_philox_init(&rng[x], random_seed * (u64)grid + (u64)blk, (u64)x);
      if (replace) {
        for (i64 x = 0; x < BX; ++x)
          for (i64 idx = x; idx < n; idx += BX) {
            i64 e = (i64)(curand_philox_next(&rng[x]) % (u64)deg); /* sampling.cu:35 */
            out_sel[o + idx] = in_start + e;
          }
      } else if (deg <= n) {
        for (i64 k = 0; k < deg; ++k) out_sel[o + k] = in_start + k;
      } else {
        for (i64 k = 0; k < n; ++k) out_sel[o + k] = k;
        for (i64 x = 0; x < BX; ++x)
          for (i64 idx = n + x; idx < deg; idx += BX) {
            i64 num = (i64)(curand_philox_next(&rng[x]) % (u64)(idx + 1)); /* sampling.cu:82 */
            if (num < n && out_sel[o + num] < idx) out_sel[o + num] = idx;  /* AtomicMax */
          }
        for (i64 k = 0; k < n; ++k) out_sel[o + k] += in_start;
      }
      for (i64 k = 0; k < n; ++k) {
        out_indices[o + k] = indices[out_sel[o + k]];
        if (out_col) out_col[o + k] = i;
      }
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Weighted per-column sampling                                              */
/* reference: src/cuda/sampling_probs.cu:57-109 (A-Res keys u^(1/p), top-K), */
/*            :200-216 (counts), :112-188 (with replacement: CDF + search).  */
/* Keys are compared as log2(u)/p (monotone in u^(1/p)); draw k of column    */
/* slot i is u = (draw+1) * 2^-32 in (0,1] like curand_uniform.              */
/* Ties and float rounding make this statistical, not bit-exact.            */
/* ------------------------------------------------------------------------ */
GO_API void go_sample_probs_fill_spec(const i64* indptr, const i64* indices, const float* probs,
                                      const i64* seeds, i64 S, i64 K, int replace, u64 seed,
                                      u32 stream, const i64* out_indptr, i64* out_indices,
                                      i64* out_col, i64* out_sel) {
#pragma omp parallel for schedule(dynamic, 64)
  for (i64 i = 0; i < S; ++i) {
    i64 c = seeds ? seeds[i] : i;
    i64 in_start = indptr[c];
    i64 deg = indptr[c + 1] - in_start;
    i64 o = out_indptr[i];
    i64 n = out_indptr[i + 1] - o;
    if (replace) {
      double total = 0;
      for (i64 e = 0; e < deg; ++e) total += probs[in_start + e];
      for (i64 k = 0; k < n; ++k) {
        double u = ((double)spec_draw(seed, stream, (u64)i, (u32)k) + 1.0) * (1.0 / 4294967296.0);
        double target = u * total, run = 0;
        i64 pick = deg - 1;
        for (i64 e = 0; e < deg; ++e) {
          run += probs[in_start + e];
          if (run >= target) { pick = e; break; }
        }
        out_sel[o + k] = in_start + pick;
      }
    } else if (deg <= K) {
      for (i64 k = 0; k < n; ++k) out_sel[o + k] = in_start + k;
    } else {
      double* key = (double*)malloc(sizeof(double) * (size_t)deg);
      for (i64 e = 0; e < deg; ++e) {
        double u = ((double)spec_draw(seed, stream, (u64)i, (u32)e) + 1.0) * (1.0 / 4294967296.0);
        double p = probs[in_start + e];
        key[e] = p > 0 ? log2(u) / p : -INFINITY;
      }
      for (i64 k = 0; k < K; ++k) { /* K largest keys, ties to the lower position */
        i64 best = -1;
        for (i64 e = 0; e < deg; ++e)
          if (!isnan(key[e]) && (best < 0 || key[e] > key[best])) best = e;
        out_sel[o + k] = in_start + best;
        key[best] = NAN;
      }
      free(key);
    }
    for (i64 k = 0; k < n; ++k) {
      out_indices[o + k] = indices[out_sel[o + k]];
      if (out_col) out_col[o + k] = i;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* First-occurrence unique + relabel                                         */
/* reference: src/cuda/unique_reindex.cu:80-151 (Unique: table keeps the     */
/* minimum index per key, an item is "first" iff table[key]==its index, scan */
/* of the flags gives its output slot), :153-172 (Relabel = table lookup),   */
/* :179-199 (TensorRelabel = unique(cat(mapping)), relabel(cat(data))).      */
/* ------------------------------------------------------------------------ */
typedef struct {
  i64* keys;
  i64* vals;
  u64 mask;
} omap_t;

static u64 mix64(u64 x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
  return x;
}
static void omap_init(omap_t* m, i64 n) {
  u64 cap = 16;
  while (cap < (u64)n * 2 + 2) cap <<= 1;
  m->keys = (i64*)malloc(sizeof(i64) * cap);
  m->vals = (i64*)malloc(sizeof(i64) * cap);
  m->mask = cap - 1;
  for (u64 i = 0; i < cap; ++i) m->keys[i] = INT64_MIN;
}
static void omap_free(omap_t* m) { free(m->keys); free(m->vals); }
/* returns pointer to the value slot; *fresh = 1 if the key was inserted now */
static i64* omap_get(omap_t* m, i64 key, int insert, int* fresh) {
  u64 p = mix64((u64)key) & m->mask;
  for (;;) {
    if (m->keys[p] == key) { if (fresh) *fresh = 0; return &m->vals[p]; }
    if (m->keys[p] == INT64_MIN) {
      if (!insert) return NULL;
      m->keys[p] = key; if (fresh) *fresh = 1; return &m->vals[p];
    }
    p = (p + 1) & m->mask;
  }
}

/* unique_reindex.cu:80-151,174-177: returns U, writes out[0..U) */
GO_API i64 go_unique_first(const i64* in, i64 n, i64* out) {
  omap_t m; omap_init(&m, n);
  i64 U = 0;
  for (i64 i = 0; i < n; ++i) {
    int fresh; i64* v = omap_get(&m, in[i], 1, &fresh);
    if (fresh) { *v = U; out[U++] = in[i]; }
  }
  omap_free(&m);
  return U;
}

/* unique_reindex.cu:179-199 with graph.cc:577-591: mapping = [seeds, rows];
 * data = (cols given as global ids, rows).  A key absent from the mapping
 * relabels to -1 (SearchForValue miss, unique_reindex.cu:53-55). */
GO_API i64 go_relabel(const i64* map_a, i64 na, const i64* map_b, i64 nb, const i64* data_a,
                      i64 da, const i64* data_b, i64 db, i64* out_unique, i64* out_a, i64* out_b) {
  omap_t m; omap_init(&m, na + nb);
  i64 U = 0;
  for (i64 i = 0; i < na + nb; ++i) {
    i64 k = i < na ? map_a[i] : map_b[i - na];
    int fresh; i64* v = omap_get(&m, k, 1, &fresh);
    if (fresh) { *v = U; out_unique[U++] = k; }
  }
  for (i64 i = 0; i < da; ++i) { i64* v = omap_get(&m, data_a[i], 0, NULL); out_a[i] = v ? *v : -1; }
  for (i64 i = 0; i < db; ++i) { i64* v = omap_get(&m, data_b[i], 0, NULL); out_b[i] = v ? *v : -1; }
  omap_free(&m);
  return U;
}

/* Per-minibatch unique + relabel.
 * reference: src/cuda/batch/batch_relabel.cu:91-213 (insert / prefix / unique
 * kernels: the item order inside minibatch b is [seeds_b..., rows_b...],
 * :138-160), :353-374 (relabel both COO arrays to batch-local ids), :376-466
 * (driver: unique_ptr = prefix[seeds_ptr+coo_ptr]), src/batch_graph.cc:214-284.
 * coo_col holds GLOBAL seed ids (batch_graph.cc:226).  Returns total U. */
GO_API i64 go_batch_coo_relabel(const i64* seeds, const i64* seeds_ptr, i64 B, const i64* coo_col,
                                const i64* coo_row, const i64* coo_ptr, i64* out_unique,
                                i64* out_unique_ptr, i64* out_row, i64* out_col) {
  i64* counts = (i64*)calloc((size_t)B + 1, sizeof(i64));
  /* pass 1: per-batch unique into a scratch laid out at the batch's item offset */
  i64 total_items = seeds_ptr[B] + coo_ptr[B];
  i64* scratch = (i64*)malloc(sizeof(i64) * (size_t)(total_items > 0 ? total_items : 1));
#pragma omp parallel for schedule(dynamic, 1)
  for (i64 b = 0; b < B; ++b) {
    i64 s0 = seeds_ptr[b], s1 = seeds_ptr[b + 1], e0 = coo_ptr[b], e1 = coo_ptr[b + 1];
    i64 n = (s1 - s0) + (e1 - e0);
    omap_t m; omap_init(&m, n);
    i64* uq = scratch + s0 + e0;
    i64 U = 0;
    for (i64 i = s0; i < s1; ++i) {
      int fresh; i64* v = omap_get(&m, seeds[i], 1, &fresh);
      if (fresh) { *v = U; uq[U++] = seeds[i]; }
    }
    for (i64 e = e0; e < e1; ++e) {
      int fresh; i64* v = omap_get(&m, coo_row[e], 1, &fresh);
      if (fresh) { *v = U; uq[U++] = coo_row[e]; }
    }
    for (i64 e = e0; e < e1; ++e) {
      i64* vr = omap_get(&m, coo_row[e], 0, NULL);
      i64* vc = omap_get(&m, coo_col[e], 0, NULL);
      out_row[e] = vr ? *vr : -1;
      out_col[e] = vc ? *vc : -1;
    }
    counts[b] = U;
    omap_free(&m);
  }
  i64 acc = 0;
  for (i64 b = 0; b < B; ++b) { out_unique_ptr[b] = acc; acc += counts[b]; }
  out_unique_ptr[B] = acc;
#pragma omp parallel for schedule(dynamic, 1)
  for (i64 b = 0; b < B; ++b)
    memcpy(out_unique + out_unique_ptr[b], scratch + seeds_ptr[b] + coo_ptr[b],
           sizeof(i64) * (size_t)counts[b]);
  free(scratch); free(counts);
  return acc;
}

/* ------------------------------------------------------------------------ */
/* Format conversion                                                         */
/* reference: src/cuda/format_transform.cu:23-46 (CSC->COO: col[e] =         */
/* upper_bound(indptr,e)-1), :66-86,121-142 (COO->CSC: stable sort by the    */
/* key then indptr by upper-bound search; skipped when already sorted).      */
/* ------------------------------------------------------------------------ */
GO_API void go_csc2coo(const i64* indptr, i64 ncols, i64* out_col) {
#pragma omp parallel for schedule(static)
  for (i64 c = 0; c < ncols; ++c)
    for (i64 e = indptr[c]; e < indptr[c + 1]; ++e) out_col[e] = c;
}

/* stable counting sort by key in [0,nkeys): out_indptr[nkeys+1], out_val = val
 * permuted, out_perm = source position (the reference's sort_index). */
GO_API void go_coo2csc(const i64* key, const i64* val, i64 nnz, i64 nkeys, i64* out_indptr,
                       i64* out_val, i64* out_perm) {
  memset(out_indptr, 0, sizeof(i64) * (size_t)(nkeys + 1));
  for (i64 e = 0; e < nnz; ++e) out_indptr[key[e] + 1]++;
  for (i64 c = 0; c < nkeys; ++c) out_indptr[c + 1] += out_indptr[c];
  i64* cur = (i64*)malloc(sizeof(i64) * (size_t)(nkeys + 1));
  memcpy(cur, out_indptr, sizeof(i64) * (size_t)(nkeys + 1));
  for (i64 e = 0; e < nnz; ++e) {
    i64 p = cur[key[e]]++;
    out_val[p] = val[e];
    if (out_perm) out_perm[p] = e;
  }
  free(cur);
}

static int cmp_i64(const void* a, const void* b) {
  i64 x = *(const i64*)a, y = *(const i64*)b;
  return (x > y) - (x < y);
}

/* src/cpu/sort_indices.cc:27-48: per-column qsort under an OpenMP parallel
 * for -- the one piece of CPU code the reference owns; restated unchanged in
 * structure (parallel over columns, libc qsort per segment). */
GO_API void go_sort_indices(const i64* indptr, i64 ncols, i64* indices) {
#pragma omp parallel for schedule(dynamic, 64)
  for (i64 c = 0; c < ncols; ++c)
    qsort(indices + indptr[c], (size_t)(indptr[c + 1] - indptr[c]), sizeof(i64), cmp_i64);
}

/* src/cuda/compact.cu:10-30: sorted unique + remap by upper_bound-1.
 * returns U; out_unique[U] sorted; out_compact[n]. */
GO_API i64 go_compact(const i64* in, i64 n, i64* out_unique, i64* out_compact) {
  i64* tmp = (i64*)malloc(sizeof(i64) * (size_t)(n > 0 ? n : 1));
  memcpy(tmp, in, sizeof(i64) * (size_t)n);
  qsort(tmp, (size_t)n, sizeof(i64), cmp_i64);
  i64 U = 0;
  for (i64 i = 0; i < n; ++i)
    if (i == 0 || tmp[i] != tmp[i - 1]) out_unique[U++] = tmp[i];
  free(tmp);
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < n; ++i) {
    i64 lo = 0, hi = U; /* upper bound */
    while (lo < hi) { i64 mid = (lo + hi) >> 1; if (out_unique[mid] <= in[i]) lo = mid + 1; else hi = mid; }
    out_compact[i] = lo - 1;
  }
  return U;
}

/* src/cuda/batch/encoding_decoding.cu:99-122: decode id = enc % size, batch =
 * enc / size, ptr[b+1] = upper_bound(batch ids, b) (input sorted by batch). */
GO_API void go_batch_offsets(const i64* enc, i64 n, i64 B, i64 size, i64* out_ptr, i64* out_dec) {
  for (i64 b = 0; b <= B; ++b) out_ptr[b] = 0;
  for (i64 i = 0; i < n; ++i) {
    i64 b = enc[i] / size;
    out_dec[i] = enc[i] - b * size;
  }
  for (i64 b = 0; b < B; ++b) {
    i64 lo = 0, hi = n;
    while (lo < hi) { i64 mid = (lo + hi) >> 1; if (enc[mid] / size <= b) lo = mid + 1; else hi = mid; }
    out_ptr[b + 1] = lo;
  }
}

/* ------------------------------------------------------------------------ */
/* Row slicing on a CSC operand (keep edges whose row is in the set, relabel */
/* the row to its position in the set)                                       */
/* reference: src/cuda/slicing.cu:184-298 (hash membership, per-column       */
/* degree, mask, compaction).  Two-call protocol: count then fill.           */
/* With duplicates in row_ids the reference's map keeps one position per     */
/* key (last writer); callers pass distinct ids (outputs of list sampling).  */
/* ------------------------------------------------------------------------ */
GO_API i64 go_slice_rows(const i64* indptr, const i64* indices, i64 ncols, const i64* row_ids,
                         i64 R, i64* out_indptr, i64* out_indices, i64* out_sel) {
  omap_t m; omap_init(&m, R);
  for (i64 i = 0; i < R; ++i) { int f; i64* v = omap_get(&m, row_ids[i], 1, &f); *v = i; }
  i64 acc = 0;
  for (i64 c = 0; c < ncols; ++c) {
    out_indptr[c] = acc;
    for (i64 e = indptr[c]; e < indptr[c + 1]; ++e) {
      i64* v = omap_get(&m, indices[e], 0, NULL);
      if (v) {
        if (out_indices) { out_indices[acc] = *v; out_sel[acc] = e; }
        ++acc;
      }
    }
  }
  out_indptr[ncols] = acc;
  omap_free(&m);
  return acc;
}

/* ------------------------------------------------------------------------ */
/* SpMM / SDDMM with scalar features (the LADIES uses)                       */
/* reference: src/cuda/spmm.cu:107-148 (CSC: out[dst] = sum_e e[eid]),       */
/* :23-56 (COO atomics), src/cuda/fusion/fused_csc_e_square_sum.cu:21-63,    */
/* src/cuda/sddmm.cu:23-61 (out[e] = op(lhs[sel], rhs[sel])); Python pre-ops */
/* python/gs/ops/sddmm.py:23-25 (div -> mul by 1/x).                         */
/* Sums are accumulated in double here so that the checker is not itself a   */
/* source of fp32 ordering noise; the kernels are compared within 1e-5 rel.  */
/* ------------------------------------------------------------------------ */
/* target: 0 = scatter by row (u), 2 = by column (v). square!=0 -> sum e^2 */
GO_API void go_edge_sum(const i64* row, const i64* col, const float* e, i64 nnz, int target,
                        int square, i64 nout, float* out) {
  double* acc = (double*)calloc((size_t)(nout > 0 ? nout : 1), sizeof(double));
  for (i64 i = 0; i < nnz; ++i) {
    double v = e[i];
    if (square) v = v * v;
    acc[target == 0 ? row[i] : col[i]] += v;
  }
  for (i64 i = 0; i < nout; ++i) out[i] = (float)acc[i];
  free(acc);
}

/* out[e] = e[e] op node[idx[e]]; op: 0 add 1 sub 2 mul 3 div.  div is
 * computed as mul by the fp32 reciprocal like python/gs/ops/sddmm.py:23-25. */
GO_API void go_edge_op_node(const i64* idx, const float* e, const float* node, i64 nnz, int op,
                            float* out) {
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < nnz; ++i) {
    float n = node[idx[i]];
    float v;
    switch (op) {
      case 0: v = e[i] + n; break;
      case 1: v = e[i] - n; break;
      case 2: v = e[i] * n; break;
      default: v = e[i] * (1.0f / n); break;
    }
    out[i] = v;
  }
}

/* ------------------------------------------------------------------------ */
/* Collective (layer-wise) sampling                                          */
/* reference: src/cuda/list_sampling.cu:20-68 (uniform: reservoir/AtomicMax, */
/* or rand%n), src/cuda/list_sampling_probs.cu:11-83 (weighted w/o           */
/* replacement: A-Res key u^(1/p), p<=0 -> -1, sort descending, first K;     */
/* with replacement: inclusive scan + upper bound),                          */
/* src/cuda/batch/list_sampling_probs.cu:29-100 (segmented variant).         */
/* "spec" stream: element i owns slot i, draw 0.  Keys are log2(u)/p.        */
/* ------------------------------------------------------------------------ */
typedef struct { double key; i64 idx; } kv_t;
static int cmp_kv_desc(const void* a, const void* b) {
  const kv_t* x = (const kv_t*)a; const kv_t* y = (const kv_t*)b;
  if (x->key > y->key) return -1;
  if (x->key < y->key) return 1;
  return (x->idx > y->idx) - (x->idx < y->idx);
}
static int cmp_i64_asc(const void* a, const void* b) {
  i64 x = *(const i64*)a, y = *(const i64*)b;
  return (x > y) - (x < y);
}
/* Weighted, without replacement, over the candidates [begin,end): the K largest
 * keys (ties to the lower index) -- the set the reference obtains by sorting
 * all keys descending and keeping the first K (list_sampling_probs.cu:47-77).
 * The picks are returned in ASCENDING INDEX order (the reference returns them
 * in descending key order, i.e. a random order; nothing downstream depends on
 * it).
 * probs == NULL selects uniformly by reservoir sampling (Algorithm R), as the
 * reference does (list_sampling.cu:47-64): the first K candidates fill the K
 * slots, candidate j >= K draws num = floor(u * (j + 1)) and, when num < K,
 * replaces slot num; processed in order, a slot ends up with the LAST (largest)
 * candidate that drew it, which is what the reference's AtomicMax computes in
 * parallel.  Picks are returned in slot order.
 * returns the number of picks written (min(K, n)). */
GO_API i64 go_list_sample_probs_spec(const float* probs, i64 begin, i64 end, i64 K, u64 seed,
                                     u32 stream, i64* out_idx) {
  i64 n = end - begin;
  if (n <= K) { for (i64 i = 0; i < n; ++i) out_idx[i] = begin + i; return n; }
  if (!probs) {
    for (i64 j = 0; j < K; ++j) out_idx[j] = begin + j;
    for (i64 j = K; j < n; ++j) {
      u32 d = spec_draw(seed, stream, (u64)(begin + j), 0);
      u64 num = ((u64)d * (u64)(j + 1)) >> 32;
      if (num < (u64)K) out_idx[num] = begin + j;
    }
    return K;
  }
  kv_t* kv = (kv_t*)malloc(sizeof(kv_t) * (size_t)n);
  for (i64 i = 0; i < n; ++i) {
    u32 d = spec_draw(seed, stream, (u64)(begin + i), 0);
    double u = ((double)d + 1.0) * (1.0 / 4294967296.0);
    double p = probs[begin + i];
    kv[i].key = p > 0 ? log2(u) / p : -INFINITY;
    kv[i].idx = begin + i;
  }
  qsort(kv, (size_t)n, sizeof(kv_t), cmp_kv_desc);
  for (i64 k = 0; k < K; ++k) out_idx[k] = kv[k].idx;
  free(kv);
  qsort(out_idx, (size_t)K, sizeof(i64), cmp_i64_asc);
  return K;
}

/* with replacement over [0,n): K independent draws; uniform when probs == NULL
 * (list_sampling.cu:32-46), else by inverse CDF (list_sampling_probs.cu:25-46);
 * draw k is word k of slot 0's stream. */
GO_API i64 go_list_sample_replace_spec(const float* probs, i64 n, i64 K, u64 seed, u32 stream,
                                       i64* out_idx) {
  double total = 0;
  if (probs) for (i64 i = 0; i < n; ++i) total += probs[i] > 0 ? probs[i] : 0;
  for (i64 k = 0; k < K; ++k) {
    u32 d = spec_draw(seed, stream, 0, (u32)k);
    if (!probs) { out_idx[k] = (i64)(((u64)d * (u64)n) >> 32); continue; }
    double target = ((double)d + 1.0) * (1.0 / 4294967296.0) * total, run = 0;
    i64 pick = n - 1;
    for (i64 i = 0; i < n; ++i) { run += probs[i] > 0 ? probs[i] : 0; if (run >= target) { pick = i; break; } }
    out_idx[k] = pick;
  }
  return K;
}

/* ------------------------------------------------------------------------ */
/* Random walks                                                              */
/* reference: src/cuda/fusion/random_walk.cu:10-47 (uniform step over the    */
/* column's entries, -1 after a dead end, trace stored step-major [L+1,N]),  */
/* src/cuda/fusion/node2vec.cu:20-137 (rejection-sampled second-order step;  */
/* previous node of the first step is the walker's index, :89).              */
/* Walker w owns spec stream slot w; draws are consumed in order.            */
/* Departures from the reference, both where it would read out of bounds:    */
/*  - x = floor(u*deg) is clamped to deg-1 (u can be 1.0, node2vec.cu:108);  */
/*  - a previous node outside [0,num_nodes) counts as "not connected"        */
/*    (node2vec.cu:89 seeds it with the thread id).                          */
/* ------------------------------------------------------------------------ */
GO_API void go_random_walk_spec(const i64* indptr, const i64* indices, const i64* seeds, i64 N,
                                i64 L, u64 seed, u32 stream, i64* out /* [(L+1)*N] */) {
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 w = 0; w < N; ++w) {
    i64 cur = seeds[w];
    out[w] = cur;
    u32 n = 0;
    for (i64 s = 0; s < L; ++s) {
      i64 pick = -1;
      if (cur >= 0) {
        i64 st = indptr[cur], deg = indptr[cur + 1] - st;
        if (deg > 0) {
          u32 r = spec_draw(seed, stream, (u64)w, n++);
          pick = indices[st + (i64)(((u64)r * (u64)deg) >> 32)];
        }
      }
      out[(s + 1) * N + w] = pick;
      cur = pick;
    }
  }
}

static int col_contains(const i64* indptr, const i64* indices, i64 num_nodes, i64 src, i64 dst) {
  if (src < 0 || src >= num_nodes) return 0;
  i64 lo = indptr[src], hi = indptr[src + 1];
  while (lo < hi) { i64 mid = (lo + hi) >> 1; if (indices[mid] < dst) lo = mid + 1; else hi = mid; }
  return lo < indptr[src + 1] && indices[lo] == dst;
}

GO_API void go_node2vec_spec(const i64* indptr, const i64* indices, i64 num_nodes, const i64* seeds,
                             i64 N, i64 L, double p, double q, u64 seed, u32 stream, i64* out) {
  double max_scale = p > q ? p : q;
  double rej = max_scale > 1.0 ? max_scale : 1.0;
  double acc = (p < q ? p : q); if (acc > 1.0) acc = 1.0;
#pragma omp parallel for schedule(dynamic, 256)
  for (i64 w = 0; w < N; ++w) {
    i64 cur = seeds[w], last = w;
    out[w] = cur;
    u32 n = 0;
    for (i64 s = 0; s < L; ++s) {
      i64 pick = -1;
      if (cur >= 0) {
        i64 st = indptr[cur], deg = indptr[cur + 1] - st;
        if (deg == 1) pick = indices[st];
        else if (deg > 1) {
          for (;;) {
            double u1 = ((double)spec_draw(seed, stream, (u64)w, n++) + 1.0) * (1.0 / 4294967296.0);
            int y = (int)floor(u1 * max_scale);
            if ((double)y >= rej) continue;
            double u2 = ((double)spec_draw(seed, stream, (u64)w, n++) + 1.0) * (1.0 / 4294967296.0);
            i64 x = (i64)floor(u2 * (double)deg);
            if (x >= deg) x = deg - 1;
            i64 cand = indices[st + x];
            if ((double)y < acc) { pick = cand; break; }
            double h;
            if (cand == last) h = p;
            else if (col_contains(indptr, indices, num_nodes, last, cand)) h = q;
            else h = 1.0;
            if ((double)y < h) { pick = cand; break; }
          }
        }
      }
      last = cur;
      cur = pick;
      out[(s + 1) * N + w] = pick;
    }
  }
}
