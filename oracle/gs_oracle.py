"""numpy front-end of the CPU restatement in ``gs_oracle.c``.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke``
and by the CPU-baseline leg of ``bench.py``.  The shipped package never imports
this module and has no CPU fallback.

Each wrapper allocates numpy outputs and calls the C function of the same
name; the C source cites the reference file:line each one restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libgs_oracle.so")


def build(force: bool = False) -> str:
    """Compile ``gs_oracle.c`` (gcc + OpenMP) if the library is missing or stale."""
    src = os.path.join(_HERE, "gs_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libgs_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.go_unique_first.restype = C.c_int64
        _lib.go_relabel.restype = C.c_int64
        _lib.go_batch_coo_relabel.restype = C.c_int64
        _lib.go_compact.restype = C.c_int64
        _lib.go_slice_rows.restype = C.c_int64
        _lib.go_list_sample_probs_spec.restype = C.c_int64
        _lib.go_list_sample_replace_spec.restype = C.c_int64
        _lib.go_spec_draw.restype = C.c_uint32
        _lib.go_num_threads.restype = C.c_int
        # a launcher may have pinned OMP_NUM_THREADS to 1 and an OpenMP runtime loaded before this
        # library has read it already: GS_ORACLE_THREADS states the thread count explicitly
        if os.environ.get("GS_ORACLE_THREADS", "").isdigit():
            _lib.go_set_num_threads(int(os.environ["GS_ORACLE_THREADS"]))
    return _lib


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().go_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads of the following calls (a launcher may have pinned OMP_NUM_THREADS to 1
    before this process could say otherwise)."""
    lib().go_set_num_threads(int(n))


def philox4x32_10(ctr, key):
    c = np.asarray(ctr, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    out = np.zeros(4, dtype=np.uint32)
    lib().go_philox4x32_10(_p(c), _p(k), _p(out))
    return out


def spec_draw(seed, stream, slot, n) -> int:
    return int(lib().go_spec_draw(C.c_uint64(seed), C.c_uint32(stream), C.c_uint64(slot),
                                  C.c_uint32(n)))


# --------------------------------------------------------------------------- slicing
def slice_cols(indptr, indices, seeds, col_bptr=None, encoding_size=0, with_coo=True):
    """A[:, seeds] -> (sub_indptr, sub_indices, coo_col, select_index)."""
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    S = seeds.size
    out_indptr = np.empty(S + 1, np.int64)
    lib().go_slice_cols_count(_p(indptr), _p(seeds), C.c_int64(S), _p(out_indptr))
    E = int(out_indptr[S])
    oi, oc, os_ = np.empty(E, np.int64), np.empty(E, np.int64), np.empty(E, np.int64)
    bp = None if col_bptr is None else _i64(col_bptr)
    B = 0 if bp is None else bp.size - 1
    lib().go_slice_cols_fill(_p(indptr), _p(indices), _p(seeds), C.c_int64(S), _p(out_indptr),
                             _p(oi), _p(oc) if with_coo else None, _p(os_), _p(bp), C.c_int64(B),
                             C.c_int64(encoding_size))
    return out_indptr, oi, (oc if with_coo else None), os_


# --------------------------------------------------------------------------- sampling
def _sample(fn, indptr, indices, seeds, K, replace, extra):
    indptr, indices = _i64(indptr), _i64(indices)
    sd = None if seeds is None else _i64(seeds)
    S = indptr.size - 1 if sd is None else sd.size
    out_indptr = np.empty(S + 1, np.int64)
    lib().go_sample_count(_p(indptr), _p(sd), C.c_int64(S), C.c_int64(K), C.c_int(int(replace)),
                          _p(out_indptr))
    E = int(out_indptr[S])
    oi, oc, os_ = np.empty(E, np.int64), np.empty(E, np.int64), np.empty(E, np.int64)
    fn(_p(indptr), _p(indices), _p(sd), C.c_int64(S), C.c_int64(K), C.c_int(int(replace)), *extra,
       _p(out_indptr), _p(oi), _p(oc), _p(os_))
    return out_indptr, oi, oc, os_


def sample_spec(indptr, indices, seeds, K, replace=False, seed=0, stream=0):
    """Floyd/Philox sampler the CUDA kernels must reproduce bit for bit."""
    return _sample(lib().go_sample_fill_spec, indptr, indices, seeds, K, replace,
                   (C.c_uint64(seed), C.c_uint32(stream)))


def sample_ref(indptr, indices, seeds, K, replace=False, random_seed=7777):
    """The reference's reservoir sampler with its cuRAND-Philox stream layout."""
    return _sample(lib().go_sample_fill_ref, indptr, indices, seeds, K, replace,
                   (C.c_uint64(random_seed),))


def sample_probs_spec(indptr, indices, probs, seeds, K, replace=False, seed=0, stream=0):
    indptr, indices, probs = _i64(indptr), _i64(indices), _f32(probs)
    sd = None if seeds is None else _i64(seeds)
    S = indptr.size - 1 if sd is None else sd.size
    out_indptr = np.empty(S + 1, np.int64)
    lib().go_sample_count(_p(indptr), _p(sd), C.c_int64(S), C.c_int64(K), C.c_int(int(replace)),
                          _p(out_indptr))
    E = int(out_indptr[S])
    oi, oc, os_ = np.empty(E, np.int64), np.empty(E, np.int64), np.empty(E, np.int64)
    lib().go_sample_probs_fill_spec(_p(indptr), _p(indices), _p(probs), _p(sd), C.c_int64(S),
                                    C.c_int64(K), C.c_int(int(replace)), C.c_uint64(seed),
                                    C.c_uint32(stream), _p(out_indptr), _p(oi), _p(oc), _p(os_))
    return out_indptr, oi, oc, os_


# --------------------------------------------------------------------------- unique / relabel
def unique_first(ids):
    ids = _i64(ids)
    out = np.empty(ids.size, np.int64)
    U = lib().go_unique_first(_p(ids), C.c_int64(ids.size), _p(out))
    return out[:U].copy()


def relabel(col_seeds, coo_row, coo_col_local):
    """GraphRelabel: returns (frontier, new_row, new_col)."""
    col_seeds, coo_row, cl = _i64(col_seeds), _i64(coo_row), _i64(coo_col_local)
    coo_col = col_seeds[cl] if cl.size else cl
    uq = np.empty(col_seeds.size + coo_row.size, np.int64)
    oa, ob = np.empty(coo_col.size, np.int64), np.empty(coo_row.size, np.int64)
    U = lib().go_relabel(_p(col_seeds), C.c_int64(col_seeds.size), _p(coo_row),
                         C.c_int64(coo_row.size), _p(_i64(coo_col)), C.c_int64(coo_col.size),
                         _p(coo_row), C.c_int64(coo_row.size), _p(uq), _p(oa), _p(ob))
    return uq[:U].copy(), ob, oa


def batch_coo_relabel(seeds, seeds_ptr, coo_col_global, coo_row, coo_ptr):
    """BatchCOORelabel: (unique, unique_ptr, out_row, out_col)."""
    seeds, seeds_ptr = _i64(seeds), _i64(seeds_ptr)
    cc, cr, cp = _i64(coo_col_global), _i64(coo_row), _i64(coo_ptr)
    B = seeds_ptr.size - 1
    uq = np.empty(seeds.size + cr.size, np.int64)
    up = np.empty(B + 1, np.int64)
    orow, ocol = np.empty(cr.size, np.int64), np.empty(cr.size, np.int64)
    U = lib().go_batch_coo_relabel(_p(seeds), _p(seeds_ptr), C.c_int64(B), _p(cc), _p(cr), _p(cp),
                                   _p(uq), _p(up), _p(orow), _p(ocol))
    return uq[:U].copy(), up, orow, ocol


# --------------------------------------------------------------------------- formats
def csc2coo(indptr):
    indptr = _i64(indptr)
    col = np.empty(int(indptr[-1]), np.int64)
    lib().go_csc2coo(_p(indptr), C.c_int64(indptr.size - 1), _p(col))
    return col


def coo2csc(key, val, nkeys):
    key, val = _i64(key), _i64(val)
    indptr = np.empty(nkeys + 1, np.int64)
    ov, perm = np.empty(val.size, np.int64), np.empty(val.size, np.int64)
    lib().go_coo2csc(_p(key), _p(val), C.c_int64(key.size), C.c_int64(nkeys), _p(indptr), _p(ov),
                     _p(perm))
    return indptr, ov, perm


def sort_indices(indptr, indices):
    indptr = _i64(indptr)
    out = _i64(indices).copy()
    lib().go_sort_indices(_p(indptr), C.c_int64(indptr.size - 1), _p(out))
    return out


def compact(ids):
    ids = _i64(ids)
    uq, cp = np.empty(ids.size, np.int64), np.empty(ids.size, np.int64)
    U = lib().go_compact(_p(ids), C.c_int64(ids.size), _p(uq), _p(cp))
    return uq[:U].copy(), cp


def batch_offsets(enc, B, size):
    enc = _i64(enc)
    ptr, dec = np.empty(B + 1, np.int64), np.empty(enc.size, np.int64)
    lib().go_batch_offsets(_p(enc), C.c_int64(enc.size), C.c_int64(B), C.c_int64(size), _p(ptr),
                           _p(dec))
    return ptr, dec


def slice_rows(indptr, indices, row_ids):
    indptr, indices, row_ids = _i64(indptr), _i64(indices), _i64(row_ids)
    nc = indptr.size - 1
    oip = np.empty(nc + 1, np.int64)
    E = lib().go_slice_rows(_p(indptr), _p(indices), C.c_int64(nc), _p(row_ids),
                            C.c_int64(row_ids.size), _p(oip), None, None)
    oi, os_ = np.empty(E, np.int64), np.empty(E, np.int64)
    lib().go_slice_rows(_p(indptr), _p(indices), C.c_int64(nc), _p(row_ids),
                        C.c_int64(row_ids.size), _p(oip), _p(oi), _p(os_))
    return oip, oi, os_


def batch_slice_cols_rows(indptr, indices, cols, col_ptr, rows, row_ptr):
    """Per-minibatch column + row selection, BatchCSCColRowSlicingCUDA
    (src/cuda/fusion/column_row_slicing.cu:154-362; hash insert :283-292, query kernel
    :219-264): minibatch b keeps, of its columns, the entries whose row id is in its own row
    list; a kept entry is renamed to the position of its row id in the whole ``rows`` array
    (:289, the value stored is ``ele``).  Returns (out_indptr, out_indices, position of the
    entry in the operand).  Row ids are distinct within a minibatch in every caller; for a
    repeated id this restatement takes the smallest position."""
    indptr, indices = _i64(indptr), _i64(indices)
    cols, col_ptr, rows, row_ptr = _i64(cols), _i64(col_ptr), _i64(rows), _i64(row_ptr)
    oip = np.zeros(cols.size + 1, np.int64)
    oi, osel = [], []
    for b in range(col_ptr.size - 1):
        pos = {}
        for i in range(int(row_ptr[b]), int(row_ptr[b + 1])):
            pos.setdefault(int(rows[i]), i)
        for s in range(int(col_ptr[b]), int(col_ptr[b + 1])):
            c = int(cols[s])
            n = 0
            for e in range(int(indptr[c]), int(indptr[c + 1])):
                p = pos.get(int(indices[e]))
                if p is not None:
                    oi.append(p)
                    osel.append(e)
                    n += 1
            oip[s + 1] = n
    return np.cumsum(oip), np.asarray(oi, np.int64), np.asarray(osel, np.int64)


# --------------------------------------------------------------------------- SpMM / SDDMM
def edge_sum(row, col, e, target, nout, square=False):
    row, col, e = _i64(row), _i64(col), _f32(e)
    out = np.zeros(nout, np.float32)
    lib().go_edge_sum(_p(row), _p(col), _p(e), C.c_int64(e.size), C.c_int(target),
                      C.c_int(int(square)), C.c_int64(nout), _p(out))
    return out


_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3}


def edge_op_node(idx, e, node, op):
    idx, e, node = _i64(idx), _f32(e), _f32(node)
    out = np.empty(e.size, np.float32)
    lib().go_edge_op_node(_p(idx), _p(e), _p(node), C.c_int64(e.size), C.c_int(_OPS[op]), _p(out))
    return out


# --------------------------------------------------------------------------- list sampling
def list_sample_probs_spec(probs, K, seed=0, stream=0, range_ptr=None, n=None):
    """K of the candidates of every segment without replacement: weighted (A-Res keys) in
    ascending index order; ``probs`` None -> uniform over ``n`` candidates by reservoir sampling,
    in slot order (list_sampling.cu:47-64)."""
    if probs is not None:
        probs = _f32(probs)
        n = probs.size
    if range_ptr is None:
        out = np.empty(min(K, n), np.int64)
        m = lib().go_list_sample_probs_spec(_p(probs), C.c_int64(0), C.c_int64(n), C.c_int64(K),
                                            C.c_uint64(seed), C.c_uint32(stream), _p(out))
        return out[:m]
    rp = _i64(range_ptr)
    outs, optr = [], [0]
    for b in range(rp.size - 1):
        n_b = int(rp[b + 1] - rp[b])
        out = np.empty(min(K, n_b), np.int64)
        m = lib().go_list_sample_probs_spec(_p(probs), C.c_int64(int(rp[b])),
                                            C.c_int64(int(rp[b + 1])), C.c_int64(K),
                                            C.c_uint64(seed), C.c_uint32(stream), _p(out))
        outs.append(out[:m])
        optr.append(optr[-1] + m)
    return (np.concatenate(outs) if outs else np.empty(0, np.int64)), np.asarray(optr, np.int64)


def list_sample_spec(n, K, replace=False, seed=0, stream=0):
    if replace:
        return list_sample_replace_spec(None, n, K, seed, stream)
    return list_sample_probs_spec(None, K, seed, stream, n=n)


def list_sample_replace_spec(probs, n, K, seed=0, stream=0):
    pr = None if probs is None else _f32(probs)
    out = np.empty(K, np.int64)
    lib().go_list_sample_replace_spec(_p(pr), C.c_int64(n), C.c_int64(K), C.c_uint64(seed),
                                      C.c_uint32(stream), _p(out))
    return out


# --------------------------------------------------------------------------- walks
def random_walk_spec(indptr, indices, seeds, L, seed=0, stream=0):
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    out = np.empty((L + 1) * seeds.size, np.int64)
    lib().go_random_walk_spec(_p(indptr), _p(indices), _p(seeds), C.c_int64(seeds.size),
                              C.c_int64(L), C.c_uint64(seed), C.c_uint32(stream), _p(out))
    return out  # step-major [(L+1), N] flattened, as the reference stores it


def node2vec_spec(indptr, indices, seeds, L, p, q, seed=0, stream=0):
    indptr, indices, seeds = _i64(indptr), _i64(indices), _i64(seeds)
    out = np.empty((L + 1) * seeds.size, np.int64)
    lib().go_node2vec_spec(_p(indptr), _p(indices), C.c_int64(indptr.size - 1), _p(seeds),
                           C.c_int64(seeds.size), C.c_int64(L), C.c_double(p), C.c_double(q),
                           C.c_uint64(seed), C.c_uint32(stream), _p(out))
    return out


# --------------------------------------------------------------------------- composed samplers
def graphsage_batch(indptr, indices, seeds, seeds_ptr, fanouts, seed=0, sampler="spec", stream_base=0):
    """The super-batch GraphSAGE sampler of examples/graphsage/graphsage_e2e.py:37-44
    (A[:, seeds::ptr] -> individual_sampling -> all_nodes -> to_dgl_block per layer),
    executed stage by stage with the restated operators.  Returns one dict per layer."""
    seeds, seeds_ptr = _i64(seeds), _i64(seeds_ptr)
    layers = []
    for li, K in enumerate(fanouts):
        if sampler == "spec":
            sip, rows, cols, sel = sample_spec(indptr, indices, seeds, K, False, seed, stream_base + li)
        else:
            sip, rows, cols, sel = sample_ref(indptr, indices, seeds, K, False)
        edge_ptr = sip[seeds_ptr]                      # batch_graph.cc:203
        uq, up, orow, ocol = batch_coo_relabel(seeds, seeds_ptr, seeds[cols], rows, edge_ptr)
        layers.append(dict(sub_indptr=sip, rows=rows, cols=cols, select=sel, edge_ptr=edge_ptr,
                           unique=uq, unique_ptr=up, block_row=orow, block_col=ocol,
                           seeds=seeds, seeds_ptr=seeds_ptr))
        seeds, seeds_ptr = uq, up
    return layers
