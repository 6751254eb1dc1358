// Edge-map / reduce operators on sampled sub-matrices: generalised SpMM
// (out[dst] = reduce over the edges of dst of op(u[src], e[edge])) and SDDMM
// (out[edge] = op(lhs[sel], rhs[sel])), fp32, with the fused forms the LADIES /
// FastGCN samplers use (sum of e^2, sum of e / u[src]).
//
// These are streaming, HBM-bound kernels: scalar features (the samplers' case)
// are reduced with a warp per segment, lanes across the segment's edges and a
// shuffle reduction, so one long column does not serialise on a single thread;
// wider features put the lanes across the feature dimension.
#include <math_constants.h>

#include "gsb_common.cuh"

namespace gsb {

enum { OP_ADD = 0, OP_SUB, OP_MUL, OP_DIV, OP_COPY_LHS, OP_COPY_RHS, OP_SQUARE_RHS, OP_RDIV };
enum { RED_SUM = 0, RED_MAX, RED_MIN };

__device__ __forceinline__ float apply_op(int op, float l, float r) {
  switch (op) {
    case OP_ADD: return l + r;
    case OP_SUB: return l - r;
    case OP_MUL: return l * r;
    case OP_DIV: return l / r;
    case OP_COPY_LHS: return l;
    case OP_COPY_RHS: return r;
    case OP_SQUARE_RHS: return r * r;
    default: return r / l;  // OP_RDIV
  }
}
__host__ __device__ inline bool op_uses_lhs(int op) { return op != OP_COPY_RHS && op != OP_SQUARE_RHS; }
__host__ __device__ inline bool op_uses_rhs(int op) { return op != OP_COPY_LHS; }

struct SpmmParams {
  const i64* indptr;
  const void* indices;
  const i64* e_ids;  // nullable: storage position -> edge feature row
  i64 nseg;
  int op, reduce;
  const float* u; i64 u_len;
  const float* e; i64 e_len;
  const i64* u_off; const i64* e_off;  // nullable broadcast offsets, [out_len]
  float* out; i64 out_len;
  i64* arg_u; i64* arg_e;  // nullable
};

constexpr int EO_THREADS = 256;

// Scalar output per segment: warp per segment, lanes over edges.
template <typename IndexT>
__global__ void __launch_bounds__(EO_THREADS) spmm_scalar_kernel(const SpmmParams p) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * EO_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * EO_THREADS) >> 5;
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  for (i64 seg = warp0; seg < p.nseg; seg += nwarps) {
    const i64 st = __ldg(p.indptr + seg), en = __ldg(p.indptr + seg + 1);
    float acc = p.reduce == RED_SUM ? 0.f : (p.reduce == RED_MAX ? -CUDART_INF_F : CUDART_INF_F);
    i64 au = -1, ae = -1;
    for (i64 i = st + lane; i < en; i += 32) {
      const i64 cid = ul || p.arg_u ? load_index<IndexT>(p.indices, i) : 0;
      const i64 eid = p.e_ids ? __ldg(p.e_ids + i) : i;
      const float l = ul ? __ldg(p.u + cid * p.u_len) : 0.f;
      const float r = ur ? __ldg(p.e + eid * p.e_len) : 0.f;
      const float v = apply_op(p.op, l, r);
      if (p.reduce == RED_SUM) acc += v;
      else if ((p.reduce == RED_MAX && v > acc) || (p.reduce == RED_MIN && v < acc)) { acc = v; au = cid; ae = eid; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float o = __shfl_xor_sync(0xffffffffu, acc, d);
      const i64 ou = __shfl_xor_sync(0xffffffffu, au, d), oe = __shfl_xor_sync(0xffffffffu, ae, d);
      if (p.reduce == RED_SUM) acc += o;
      else if ((p.reduce == RED_MAX && (o > acc || (o == acc && oe >= 0 && (ae < 0 || oe < ae)))) ||
               (p.reduce == RED_MIN && (o < acc || (o == acc && oe >= 0 && (ae < 0 || oe < ae))))) {
        acc = o; au = ou; ae = oe;
      }
    }
    if (lane == 0) {
      if (p.reduce == RED_SUM) {
        p.out[seg] += acc;  // the caller zero-fills `out` (accumulate semantics)
      } else {
        p.out[seg] = en > st ? acc : 0.f;  // empty segment -> 0
        if (p.arg_u && ul) p.arg_u[seg] = en > st ? au : 0;
        if (p.arg_e && ur) p.arg_e[seg] = en > st ? ae : 0;
      }
    }
  }
}

// Scalar sum per segment, the samplers' case.  Same arithmetic as the kernel above (lanes stride
// over the segment, then a butterfly), but a warp takes 32 consecutive segments at a time: their
// bounds arrive with one coalesced load instead of 32 dependent ones, the edge loads of
// neighbouring segments fall into the same lines, and the 32 results leave with one coalesced
// read-modify-write.  Short segments (a whole graph's columns) are latency-bound otherwise.
template <typename IndexT>
__global__ void __launch_bounds__(EO_THREADS) spmm_scalar_sum_kernel(const SpmmParams p) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * EO_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * EO_THREADS) >> 5;
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  const float* __restrict__ uf = p.u;
  const float* __restrict__ ef = p.e;
  const i64* __restrict__ eids = p.e_ids;
  for (i64 seg0 = warp0 * 32; seg0 < p.nseg; seg0 += nwarps * 32) {
    const i64 mine = seg0 + lane;
    const i64 my_st = mine < p.nseg ? __ldg(p.indptr + mine) : 0;
    const i64 my_en = mine < p.nseg ? __ldg(p.indptr + mine + 1) : 0;
    const int live = p.nseg - seg0 < 32 ? (int)(p.nseg - seg0) : 32;
    float res = 0.f;
    for (int j = 0; j < live; ++j) {
      const i64 st = __shfl_sync(0xffffffffu, my_st, j), en = __shfl_sync(0xffffffffu, my_en, j);
      float acc = 0.f;
      if (p.op == OP_COPY_RHS && !eids && p.e_len == 1) {
        for (i64 i = st + lane; i < en; i += 32) acc += __ldg(ef + i);
      } else {
        for (i64 i = st + lane; i < en; i += 32) {
          const i64 cid = ul ? load_index<IndexT>(p.indices, i) : 0;
          const i64 eid = eids ? __ldg(eids + i) : i;
          const float l = ul ? __ldg(uf + cid * p.u_len) : 0.f;
          const float r = ur ? __ldg(ef + eid * p.e_len) : 0.f;
          acc += apply_op(p.op, l, r);
        }
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
      if (lane == j) res = acc;
    }
    if (mine < p.nseg) p.out[mine] += res;  // the caller zero-fills `out` (accumulate semantics)
  }
}

// Feature vectors: warp per segment, lanes over the feature dimension.
template <typename IndexT>
__global__ void __launch_bounds__(EO_THREADS) spmm_vector_kernel(const SpmmParams p) {
  const int lane = threadIdx.x & 31;
  const i64 warp0 = ((i64)blockIdx.x * EO_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * EO_THREADS) >> 5;
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  for (i64 seg = warp0; seg < p.nseg; seg += nwarps) {
    const i64 st = __ldg(p.indptr + seg), en = __ldg(p.indptr + seg + 1);
    for (i64 f = lane; f < p.out_len; f += 32) {
      const i64 lo = p.u_off ? p.u_off[f] : (p.u_len == 1 ? 0 : f);
      const i64 ro = p.e_off ? p.e_off[f] : (p.e_len == 1 ? 0 : f);
      float acc = p.reduce == RED_SUM ? 0.f : (p.reduce == RED_MAX ? -CUDART_INF_F : CUDART_INF_F);
      i64 au = 0, ae = 0;
      for (i64 i = st; i < en; ++i) {
        const i64 cid = load_index<IndexT>(p.indices, i);
        const i64 eid = p.e_ids ? __ldg(p.e_ids + i) : i;
        const float l = ul ? __ldg(p.u + cid * p.u_len + lo) : 0.f;
        const float r = ur ? __ldg(p.e + eid * p.e_len + ro) : 0.f;
        const float v = apply_op(p.op, l, r);
        if (p.reduce == RED_SUM) acc += v;
        else if ((p.reduce == RED_MAX && v > acc) || (p.reduce == RED_MIN && v < acc)) { acc = v; au = cid; ae = eid; }
      }
      const i64 o = seg * p.out_len + f;
      if (p.reduce == RED_SUM) {
        p.out[o] += acc;
      } else {
        p.out[o] = en > st ? acc : 0.f;
        if (p.arg_u && ul) p.arg_u[o] = au;
        if (p.arg_e && ur) p.arg_e[o] = ae;
      }
    }
  }
}

struct CooParams {
  const i64* row; const i64* col; const i64* e_ids; i64 nnz;
  int op;
  const float* lhs; i64 lhs_len; int lhs_target;
  const float* rhs; i64 rhs_len; int rhs_target;
  const i64* lhs_off; const i64* rhs_off;
  float* out; i64 out_len;
  int out_target;  // SpMM on COO: 0 = scatter to row, 2 = to col (unused by SDDMM)
};

__device__ __forceinline__ i64 select_target(int target, i64 src, i64 eid, i64 dst) {
  return target == 0 ? src : (target == 1 ? eid : dst);
}

// out[eid, f] = op(lhs[sel_l], rhs[sel_r]); thread per (edge, feature)
__global__ void __launch_bounds__(EO_THREADS) sddmm_coo_kernel(const CooParams p) {
  const i64 total = p.nnz * p.out_len;
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  for (i64 t = (i64)blockIdx.x * EO_THREADS + threadIdx.x; t < total; t += (i64)gridDim.x * EO_THREADS) {
    const i64 ed = t / p.out_len, f = t - ed * p.out_len;
    const i64 src = __ldg(p.row + ed), dst = __ldg(p.col + ed);
    const i64 eid = p.e_ids ? __ldg(p.e_ids + ed) : ed;
    const i64 lo = p.lhs_off ? p.lhs_off[f] : (p.lhs_len == 1 ? 0 : f);
    const i64 ro = p.rhs_off ? p.rhs_off[f] : (p.rhs_len == 1 ? 0 : f);
    const float l = ul ? __ldg(p.lhs + select_target(p.lhs_target, src, eid, dst) * p.lhs_len + lo) : 0.f;
    const float r = ur ? __ldg(p.rhs + select_target(p.rhs_target, src, eid, dst) * p.rhs_len + ro) : 0.f;
    p.out[eid * p.out_len + f] = apply_op(p.op, l, r);
  }
}

// out[eid, f] = sum_k lhs[sel_l, off_l(f) * reduce + k] * rhs[sel_r, off_r(f) * reduce + k];
// warp per (edge, f), lanes over k.
__global__ void __launch_bounds__(EO_THREADS) sddmm_coo_dot_kernel(const CooParams p, i64 reduce) {
  const int lane = threadIdx.x & 31;
  const i64 total = p.nnz * p.out_len;
  const i64 warp0 = ((i64)blockIdx.x * EO_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * EO_THREADS) >> 5;
  for (i64 t = warp0; t < total; t += nwarps) {
    const i64 ed = t / p.out_len, f = t - ed * p.out_len;
    const i64 src = __ldg(p.row + ed), dst = __ldg(p.col + ed);
    const i64 eid = p.e_ids ? __ldg(p.e_ids + ed) : ed;
    const i64 lo = p.lhs_off ? p.lhs_off[f] : (p.lhs_len == reduce ? 0 : f);
    const i64 ro = p.rhs_off ? p.rhs_off[f] : (p.rhs_len == reduce ? 0 : f);
    const float* l = p.lhs + select_target(p.lhs_target, src, eid, dst) * p.lhs_len + lo * reduce;
    const float* r = p.rhs + select_target(p.rhs_target, src, eid, dst) * p.rhs_len + ro * reduce;
    float acc = 0.f;
    for (i64 k = lane; k < reduce; k += 32) acc += __ldg(l + k) * __ldg(r + k);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) p.out[eid * p.out_len + f] = acc;
  }
}

// sum-SpMM on an unsorted COO: atomicAdd per (edge, feature).  lhs = node
// feature of the OTHER endpoint, rhs = edge feature.
__global__ void __launch_bounds__(EO_THREADS) spmm_coo_sum_kernel(const CooParams p) {
  const i64 total = p.nnz * p.out_len;
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  for (i64 t = (i64)blockIdx.x * EO_THREADS + threadIdx.x; t < total; t += (i64)gridDim.x * EO_THREADS) {
    const i64 ed = t / p.out_len, f = t - ed * p.out_len;
    const i64 r0 = __ldg(p.row + ed), c0 = __ldg(p.col + ed);
    const i64 src = p.out_target == 2 ? r0 : c0;  // feature side
    const i64 dst = p.out_target == 2 ? c0 : r0;  // reduced side
    const i64 eid = p.e_ids ? __ldg(p.e_ids + ed) : ed;
    const i64 lo = p.lhs_off ? p.lhs_off[f] : (p.lhs_len == 1 ? 0 : f);
    const i64 ro = p.rhs_off ? p.rhs_off[f] : (p.rhs_len == 1 ? 0 : f);
    const float l = ul ? __ldg(p.lhs + src * p.lhs_len + lo) : 0.f;
    const float r = ur ? __ldg(p.rhs + eid * p.rhs_len + ro) : 0.f;
    atomicAdd(p.out + dst * p.out_len + f, apply_op(p.op, l, r));
  }
}

// Scalar features on both sides (the samplers' case): no index arithmetic per element, and only
// the endpoint arrays the operands actually select are read.
__global__ void __launch_bounds__(EO_THREADS) sddmm_coo_scalar_kernel(const CooParams p) {
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  const bool need_row = (ul && p.lhs_target == 0) || (ur && p.rhs_target == 0);
  const bool need_col = (ul && p.lhs_target == 2) || (ur && p.rhs_target == 2);
  const i64* __restrict__ row = p.row;
  const i64* __restrict__ col = p.col;
  const i64* __restrict__ eids = p.e_ids;
  const float* __restrict__ lhs = p.lhs;
  const float* __restrict__ rhs = p.rhs;
  float* __restrict__ out = p.out;
  // four independent, coalesced edges per thread and step: the loads of all four are in flight
  // before the first gather is needed
  const i64 step = (i64)gridDim.x * EO_THREADS * 4;
  for (i64 base = (i64)blockIdx.x * EO_THREADS * 4 + threadIdx.x; base < p.nnz; base += step) {
    i64 src[4], dst[4], eid[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const i64 ed = base + k * EO_THREADS;
      const bool in = ed < p.nnz;
      src[k] = need_row && in ? __ldg(row + ed) : 0;
      dst[k] = need_col && in ? __ldg(col + ed) : 0;
      eid[k] = eids && in ? __ldg(eids + ed) : ed;
    }
    float l[4], r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool in = base + k * EO_THREADS < p.nnz;
      l[k] = ul && in ? __ldg(lhs + select_target(p.lhs_target, src[k], eid[k], dst[k])) : 0.f;
      r[k] = ur && in ? __ldg(rhs + select_target(p.rhs_target, src[k], eid[k], dst[k])) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (base + k * EO_THREADS < p.nnz) out[eid[k]] = apply_op(p.op, l[k], r[k]);
  }
}

// Scalar sum over an unsorted COO.  Neighbouring edges that reduce into the same node (always,
// when the COO is in the order of the reduced side) are summed inside the warp first, so that one
// atomic per run reaches memory instead of one per edge.
__global__ void __launch_bounds__(EO_THREADS) spmm_coo_sum_scalar_kernel(const CooParams p) {
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  const int lane = threadIdx.x & 31;
  const i64* __restrict__ red = p.out_target == 2 ? p.col : p.row;   // reduced side
  const i64* __restrict__ feat = p.out_target == 2 ? p.row : p.col;  // feature side
  const i64* __restrict__ eids = p.e_ids;
  const float* __restrict__ lhs = p.lhs;
  const float* __restrict__ rhs = p.rhs;
  const i64 step = (i64)gridDim.x * EO_THREADS * 4;
  // whole CTAs stay in the loop (the shuffles need full warps); four coalesced groups per step
  for (i64 base = (i64)blockIdx.x * EO_THREADS * 4; base < p.nnz; base += step) {
    i64 dst[4];
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const i64 ed = base + k * EO_THREADS + threadIdx.x;
      dst[k] = -1 - lane;  // distinct per lane: a dead lane joins no run
      v[k] = 0.f;
      if (ed < p.nnz) {
        dst[k] = __ldg(red + ed);
        const i64 eid = eids ? __ldg(eids + ed) : ed;
        const float l = ul ? __ldg(lhs + __ldg(feat + ed)) : 0.f;
        const float r = ur ? __ldg(rhs + eid) : 0.f;
        v[k] = apply_op(p.op, l, r);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const i64 prev = __shfl_up_sync(0xffffffffu, dst[k], 1);
      const bool head = lane == 0 || prev != dst[k];
      float acc = v[k];
      if (__any_sync(0xffffffffu, !head)) {
        // runs of equal targets: suffix sums inside each run, the head holds the run's total
        const unsigned heads = __ballot_sync(0xffffffffu, head);
        const unsigned above = lane == 31 ? 0u : heads >> (lane + 1);
        const int run_end = above ? lane + __ffs(above) - 1 : 31;  // last lane of this lane's run
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const float o = __shfl_down_sync(0xffffffffu, acc, d);
          if (lane + d <= run_end) acc += o;
        }
      }
      if (dst[k] >= 0 && head) atomicAdd(p.out + dst[k], acc);
    }
  }
}

// Two u-op-v edge maps over one COO: out1[eid, f] = op(lhs1[row, .], rhs1[col, .]) and
// out2[eid, f] = op(lhs2[row, .], rhs2[col, .]).  The endpoints of an edge (and its id) are read
// once for both maps; with scalar operands four coalesced edges per thread are in flight.
struct PairParams {
  const i64* row; const i64* col; const i64* e_ids; i64 nnz;
  int op;
  const float* lhs1; const float* rhs1; float* out1;
  const float* lhs2; const float* rhs2; float* out2;
  i64 lhs_len, rhs_len;
  const i64* lhs_off; const i64* rhs_off;
  i64 out_len;
};

__global__ void __launch_bounds__(EO_THREADS) u_op_v_pair_scalar_kernel(const PairParams p) {
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  const i64* __restrict__ row = p.row;
  const i64* __restrict__ col = p.col;
  const i64* __restrict__ eids = p.e_ids;
  const i64 step = (i64)gridDim.x * EO_THREADS * 4;
  for (i64 base = (i64)blockIdx.x * EO_THREADS * 4 + threadIdx.x; base < p.nnz; base += step) {
    i64 src[4], dst[4], eid[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const i64 ed = base + k * EO_THREADS;
      const bool in = ed < p.nnz;
      src[k] = ul && in ? __ldg(row + ed) : 0;
      dst[k] = ur && in ? __ldg(col + ed) : 0;
      eid[k] = eids && in ? __ldg(eids + ed) : ed;
    }
    float l1[4], r1[4], l2[4], r2[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool in = base + k * EO_THREADS < p.nnz;
      l1[k] = ul && in ? __ldg(p.lhs1 + src[k]) : 0.f;
      r1[k] = ur && in ? __ldg(p.rhs1 + dst[k]) : 0.f;
      l2[k] = ul && in ? __ldg(p.lhs2 + src[k]) : 0.f;
      r2[k] = ur && in ? __ldg(p.rhs2 + dst[k]) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (base + k * EO_THREADS < p.nnz) {
        p.out1[eid[k]] = apply_op(p.op, l1[k], r1[k]);
        p.out2[eid[k]] = apply_op(p.op, l2[k], r2[k]);
      }
  }
}

__global__ void __launch_bounds__(EO_THREADS) u_op_v_pair_kernel(const PairParams p) {
  const i64 total = p.nnz * p.out_len;
  const bool ul = op_uses_lhs(p.op), ur = op_uses_rhs(p.op);
  for (i64 t = (i64)blockIdx.x * EO_THREADS + threadIdx.x; t < total; t += (i64)gridDim.x * EO_THREADS) {
    const i64 ed = t / p.out_len, f = t - ed * p.out_len;
    const i64 src = __ldg(p.row + ed), dst = __ldg(p.col + ed);
    const i64 eid = p.e_ids ? __ldg(p.e_ids + ed) : ed;
    const i64 lo = src * p.lhs_len + (p.lhs_off ? p.lhs_off[f] : (p.lhs_len == 1 ? 0 : f));
    const i64 ro = dst * p.rhs_len + (p.rhs_off ? p.rhs_off[f] : (p.rhs_len == 1 ? 0 : f));
    const float l1 = ul ? __ldg(p.lhs1 + lo) : 0.f, r1 = ur ? __ldg(p.rhs1 + ro) : 0.f;
    const float l2 = ul ? __ldg(p.lhs2 + lo) : 0.f, r2 = ur ? __ldg(p.rhs2 + ro) : 0.f;
    p.out1[eid * p.out_len + f] = apply_op(p.op, l1, r1);
    p.out2[eid * p.out_len + f] = apply_op(p.op, l2, r2);
  }
}

// grid cap in CTAs per SM for the streaming edge kernels: 123.7 M edges, cap 16 / 64: SDDMM 0.63 / 0.57 ms,
// COO sums 0.78 / 0.73 ms (more, shorter CTAs even out the tail and the atomics' hot rows)
#ifndef GSB_WIDE_GRID
#define GSB_WIDE_GRID 64
#endif
static int wide_grid(i64 work_items, int per_block) {
  i64 g = (work_items + per_block - 1) / per_block;
  if (g > sm_count() * GSB_WIDE_GRID) g = sm_count() * GSB_WIDE_GRID;
  return g < 1 ? 1 : (int)g;
}

}  // namespace gsb

using namespace gsb;

extern "C" int gsb_spmm_segmented(const int64_t* indptr, const void* indices, int indices_dtype,
                                  const int64_t* e_ids, int64_t nseg, int op, int reduce,
                                  const float* u, int64_t u_len, const float* e, int64_t e_len,
                                  const int64_t* u_off, const int64_t* e_off, float* out,
                                  int64_t out_len, int64_t* arg_u, int64_t* arg_e,
                                  void* cuda_stream) {
  if (nseg == 0) return GSB_OK;
  if (!indptr || !indices || !out || nseg < 0 || out_len < 1) return GSB_ERR_INVALID;
  if (op < OP_ADD || op > OP_RDIV || reduce < RED_SUM || reduce > RED_MIN) return GSB_ERR_INVALID;
  if ((op_uses_lhs(op) && (!u || u_len < 1)) || (op_uses_rhs(op) && (!e || e_len < 1)))
    return GSB_ERR_INVALID;
  if (indices_dtype != GSB_I32 && indices_dtype != GSB_I64) return GSB_ERR_INVALID;
  SpmmParams p{(const i64*)indptr, indices, (const i64*)e_ids, nseg, op, reduce, u, u_len, e, e_len,
               (const i64*)u_off, (const i64*)e_off, out, out_len, (i64*)arg_u, (i64*)arg_e};
  cudaStream_t st = (cudaStream_t)cuda_stream;
  const int grid = wide_grid(nseg, EO_THREADS / 32);
  LaunchScope ls(KID_EDGE_SUM, st);
  const bool scalar = out_len == 1;
  const bool scalar_sum = scalar && reduce == RED_SUM && !u_off && !e_off;
  if (scalar_sum) {
    const int g32 = wide_grid((nseg + 31) / 32, EO_THREADS / 32);
    if (indices_dtype == GSB_I32) spmm_scalar_sum_kernel<int><<<g32, EO_THREADS, 0, st>>>(p);
    else spmm_scalar_sum_kernel<i64><<<g32, EO_THREADS, 0, st>>>(p);
  } else if (indices_dtype == GSB_I32) {
    if (scalar) spmm_scalar_kernel<int><<<grid, EO_THREADS, 0, st>>>(p);
    else spmm_vector_kernel<int><<<grid, EO_THREADS, 0, st>>>(p);
  } else {
    if (scalar) spmm_scalar_kernel<i64><<<grid, EO_THREADS, 0, st>>>(p);
    else spmm_vector_kernel<i64><<<grid, EO_THREADS, 0, st>>>(p);
  }
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

static int check_coo(const int64_t* row, const int64_t* col, int64_t nnz, int op, const float* lhs,
                     int64_t lhs_len, const float* rhs, int64_t rhs_len, float* out,
                     int64_t out_len) {
  if (nnz < 0 || out_len < 1 || !row || !col || !out) return GSB_ERR_INVALID;
  if (op < OP_ADD || op > OP_RDIV) return GSB_ERR_INVALID;
  if ((op_uses_lhs(op) && (!lhs || lhs_len < 1)) || (op_uses_rhs(op) && (!rhs || rhs_len < 1)))
    return GSB_ERR_INVALID;
  return GSB_OK;
}

extern "C" int gsb_sddmm_coo(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                             int64_t nnz, int op, const float* lhs, int64_t lhs_len, int lhs_target,
                             const float* rhs, int64_t rhs_len, int rhs_target,
                             const int64_t* lhs_off, const int64_t* rhs_off, float* out,
                             int64_t out_len, void* cuda_stream) {
  if (nnz == 0) return GSB_OK;
  int rc = check_coo(row, col, nnz, op, lhs, lhs_len, rhs, rhs_len, out, out_len);
  if (rc != GSB_OK) return rc;
  if (lhs_target < 0 || lhs_target > 2 || rhs_target < 0 || rhs_target > 2) return GSB_ERR_INVALID;
  CooParams p{(const i64*)row, (const i64*)col, (const i64*)e_ids, nnz, op, lhs, lhs_len, lhs_target,
              rhs, rhs_len, rhs_target, (const i64*)lhs_off, (const i64*)rhs_off, out, out_len, 0};
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_EDGE_OP, st);
  if (out_len == 1 && (!op_uses_lhs(op) || lhs_len == 1) && (!op_uses_rhs(op) || rhs_len == 1) &&
      !lhs_off && !rhs_off)
    sddmm_coo_scalar_kernel<<<wide_grid(nnz, EO_THREADS * 4), EO_THREADS, 0, st>>>(p);
  else
    sddmm_coo_kernel<<<wide_grid(nnz * out_len, EO_THREADS), EO_THREADS, 0, st>>>(p);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_u_op_v_pair(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                               int64_t nnz, int op, const float* lhs1, const float* rhs1, float* out1,
                               const float* lhs2, const float* rhs2, float* out2, int64_t lhs_len,
                               int64_t rhs_len, const int64_t* lhs_off, const int64_t* rhs_off,
                               int64_t out_len, void* cuda_stream) {
  if (nnz == 0) return GSB_OK;
  int rc = check_coo(row, col, nnz, op, lhs1, lhs_len, rhs1, rhs_len, out1, out_len);
  if (rc == GSB_OK) rc = check_coo(row, col, nnz, op, lhs2, lhs_len, rhs2, rhs_len, out2, out_len);
  if (rc != GSB_OK) return rc;
  PairParams p{(const i64*)row, (const i64*)col, (const i64*)e_ids, nnz, op, lhs1, rhs1, out1,
               lhs2, rhs2, out2, lhs_len, rhs_len, (const i64*)lhs_off, (const i64*)rhs_off, out_len};
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_EDGE_OP, st);
  if (out_len == 1 && (!op_uses_lhs(op) || lhs_len == 1) && (!op_uses_rhs(op) || rhs_len == 1) &&
      !lhs_off && !rhs_off)
    u_op_v_pair_scalar_kernel<<<wide_grid(nnz, EO_THREADS * 4), EO_THREADS, 0, st>>>(p);
  else
    u_op_v_pair_kernel<<<wide_grid(nnz * out_len, EO_THREADS), EO_THREADS, 0, st>>>(p);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_spmm_coo_sum(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                                int64_t nnz, int op, int u_target, const float* u, int64_t u_len,
                                const float* e, int64_t e_len, const int64_t* u_off,
                                const int64_t* e_off, float* out, int64_t out_len,
                                void* cuda_stream) {
  if (nnz == 0) return GSB_OK;
  int rc = check_coo(row, col, nnz, op, u, u_len, e, e_len, out, out_len);
  if (rc != GSB_OK) return rc;
  if (u_target != 0 && u_target != 2) return GSB_ERR_INVALID;
  // u_target 0: features live on rows, the sum goes to columns; 2: the reverse
  CooParams p{(const i64*)row, (const i64*)col, (const i64*)e_ids, nnz, op, u, u_len, 0, e, e_len, 1,
              (const i64*)u_off, (const i64*)e_off, out, out_len, u_target == 0 ? 2 : 0};
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_EDGE_SUM, st);
  if (out_len == 1 && (!op_uses_lhs(op) || u_len == 1) && (!op_uses_rhs(op) || e_len == 1) &&
      !u_off && !e_off)
    spmm_coo_sum_scalar_kernel<<<wide_grid(nnz, EO_THREADS * 4), EO_THREADS, 0, st>>>(p);
  else
    spmm_coo_sum_kernel<<<wide_grid(nnz * out_len, EO_THREADS), EO_THREADS, 0, st>>>(p);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}

extern "C" int gsb_sddmm_coo_dot(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                                 int64_t nnz, const float* lhs, int64_t lhs_len, int lhs_target,
                                 const float* rhs, int64_t rhs_len, int rhs_target,
                                 const int64_t* lhs_off, const int64_t* rhs_off, int64_t reduce,
                                 float* out, int64_t out_len, void* cuda_stream) {
  if (nnz == 0) return GSB_OK;
  if (!row || !col || !lhs || !rhs || !out || nnz < 0 || reduce < 1 || out_len < 1 ||
      lhs_len < reduce || rhs_len < reduce || lhs_len % reduce || rhs_len % reduce)
    return GSB_ERR_INVALID;
  if (lhs_target < 0 || lhs_target > 2 || rhs_target < 0 || rhs_target > 2) return GSB_ERR_INVALID;
  CooParams p{(const i64*)row, (const i64*)col, (const i64*)e_ids, nnz, OP_MUL, lhs, lhs_len, lhs_target,
              rhs, rhs_len, rhs_target, (const i64*)lhs_off, (const i64*)rhs_off, out, out_len, 0};
  cudaStream_t st = (cudaStream_t)cuda_stream;
  LaunchScope ls(KID_EDGE_OP, st);
  sddmm_coo_dot_kernel<<<wide_grid(nnz * out_len * 32, EO_THREADS), EO_THREADS, 0, st>>>(p, reduce);
  GSB_CUDA_OK(cudaGetLastError());
  return GSB_OK;
}
