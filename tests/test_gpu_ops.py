"""GPU tests of the operators around the GraphSAGE path: slicing across the compressed
dimension, COO slicing, SpMM / SDDMM and their fused forms, collective (list) sampling, random
walks / node2vec, column sort, compact -- each against the CPU oracle -- and the LADIES and
node2vec samplers of the reference's examples written against this package's Matrix API."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def host(t):
    return t.cpu().numpy()


def cuda(a, dtype=torch.int64):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).cuda()


def rand_csc(rng, n, avg, heavy=0):
    deg = rng.poisson(avg, n)
    deg[rng.integers(0, n, max(n // 10, 1))] = 0
    if heavy:
        deg[rng.integers(0, n, heavy)] = rng.integers(200, 1500, heavy)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, indptr[-1]).astype(np.int64)
    return indptr, indices


def new_graph(gsb, indptr, indices, seed=99, idx_dtype=torch.int64):
    n = indptr.size - 1
    g = gsb.Graph(n, n)
    g._CAPI_LoadCSC(cuda(indptr), cuda(indices, idx_dtype))
    g._CAPI_SetSeed(seed)
    return g


@pytest.fixture(scope="module")
def graph():
    return rand_csc(np.random.default_rng(21), 3000, 12, heavy=10)


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_row_slicing_on_csc(gsb, oracle, graph, idx_dtype):
    indptr, indices = graph
    rng = np.random.default_rng(1)
    rows = rng.permutation(3000)[:700].astype(np.int64)
    A = new_graph(gsb, indptr, indices, idx_dtype=idx_dtype)
    sub, sel = A._CAPI_Slicing(cuda(rows), 0, gsb._CSC, gsb._CSC + gsb._COO)
    eip, eids, esel = oracle.slice_rows(indptr, indices, rows)
    assert np.array_equal(host(sub._CAPI_GetCSCIndptr()), eip)
    assert np.array_equal(host(sub._CAPI_GetCSCIndices()), eids)
    assert np.array_equal(host(sel), esel)
    assert np.array_equal(host(sub._CAPI_GetCOORows()), eids)
    assert np.array_equal(host(sub._CAPI_GetCOOCols()), oracle.csc2coo(eip))
    assert (sub._CAPI_GetNumRows(), sub._CAPI_GetNumCols(), sub._CAPI_GetNumEdges()) == (700, 3000, eids.size)
    # the CSC-only form (no segment of the kept entries is produced)
    sub2, sel2 = A._CAPI_Slicing(cuda(rows), 0, gsb._CSC, gsb._CSC)
    assert np.array_equal(host(sub2._CAPI_GetCSCIndptr()), eip)
    assert np.array_equal(host(sub2._CAPI_GetCSCIndices()), eids)
    assert np.array_equal(host(sel2), esel)
    # empty selection
    sub, sel = A._CAPI_Slicing(cuda(np.empty(0, np.int64)), 0, gsb._CSC, gsb._CSC)
    assert sel.numel() == 0 and not host(sub._CAPI_GetCSCIndptr()).any()


def test_row_slicing_over_thousands_of_tiles(gsb, oracle):
    """2.4 M entries = 2300 tiles of 1024: every thread of the one-CTA tile scan owns several tiles,
    columns start anywhere inside a tile, runs of empty columns cross tile borders."""
    rng = np.random.default_rng(33)
    n = 200000
    indptr, indices = rand_csc(rng, n, 12, heavy=20)
    rows = rng.permutation(n)[:n // 3].astype(np.int64)
    A = new_graph(gsb, indptr, indices)
    eip, eids, esel = oracle.slice_rows(indptr, indices, rows)
    for fmt in (gsb._CSC, gsb._CSC + gsb._COO):
        sub, sel = A._CAPI_Slicing(cuda(rows), 0, gsb._CSC, fmt)
        assert np.array_equal(host(sub._CAPI_GetCSCIndptr()), eip)
        assert np.array_equal(host(sub._CAPI_GetCSCIndices()), eids)
        assert np.array_equal(host(sel), esel)
    assert np.array_equal(host(sub._CAPI_GetCOOCols()), oracle.csc2coo(eip))
    # column slice of the same graph: the tile search of the fill pass over 150 000 column slots
    seeds = rng.integers(0, n, 150000).astype(np.int64)
    sub, sel = A._CAPI_Slicing(cuda(seeds), 1, gsb._CSC, gsb._CSC + gsb._COO)
    deg = np.diff(indptr)[seeds]
    want_ptr = np.concatenate([[0], np.cumsum(deg)])
    want_sel = np.concatenate([np.arange(indptr[c], indptr[c + 1]) for c in seeds] + [np.empty(0, np.int64)])
    assert np.array_equal(host(sub._CAPI_GetCSCIndptr()), want_ptr)
    assert np.array_equal(host(sel), want_sel)
    assert np.array_equal(host(sub._CAPI_GetCSCIndices()), indices[want_sel])
    assert np.array_equal(host(sub._CAPI_GetCOOCols()), np.repeat(np.arange(seeds.size), deg))


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_batch_col_row_slicing(gsb, oracle, graph, idx_dtype):
    """Induced sub-matrices per minibatch (ShaDow-style): _CAPI_BatchColRowSlcing."""
    indptr, indices = graph
    rng = np.random.default_rng(4)
    B = 5
    ncol = np.array([200, 0, 333, 1, 150])
    nrow = np.array([900, 50, 0, 2999, 400])
    cols = np.concatenate([rng.integers(0, 3000, n) for n in ncol]).astype(np.int64)
    rows = np.concatenate([rng.permutation(3000)[:n] for n in nrow]).astype(np.int64)
    col_ptr = np.concatenate([[0], np.cumsum(ncol)]).astype(np.int64)
    row_ptr = np.concatenate([[0], np.cumsum(nrow)]).astype(np.int64)
    A = new_graph(gsb, indptr, indices, idx_dtype=idx_dtype)
    sub, sel = A._CAPI_BatchColRowSlcing(cuda(cols), cuda(col_ptr), cuda(rows), cuda(row_ptr))
    eip, eids, esel = oracle.batch_slice_cols_rows(indptr, indices, cols, col_ptr, rows, row_ptr)
    assert esel.size > 100
    assert np.array_equal(host(sub._CAPI_GetCSCIndptr()), eip)
    assert np.array_equal(host(sub._CAPI_GetCSCIndices()), eids)
    assert np.array_equal(host(sel), esel)
    assert np.array_equal(host(sub._CAPI_GetCOORows()), eids)
    assert np.array_equal(host(sub._CAPI_GetCOOCols()), oracle.csc2coo(eip))
    assert np.array_equal(host(sub._CAPI_GetEdgeBptr()), eip[col_ptr])
    assert (sub._CAPI_GetNumRows(), sub._CAPI_GetNumCols(), sub._CAPI_GetNumEdges()) == (
        rows.size, cols.size, eids.size)
    # every kept entry: its row id is rows[new id] and belongs to the entry's own minibatch
    assert np.array_equal(rows[eids], indices[esel])
    b_of_edge = np.searchsorted(col_ptr, oracle.csc2coo(eip), side="right") - 1
    assert np.all((eids >= row_ptr[b_of_edge]) & (eids < row_ptr[b_of_edge + 1]))
    # through the BatchMatrix surface, with edge data carried along
    m = gsb.Matrix(A)
    w = torch.arange(indices.size, dtype=torch.float32).cuda()
    m.edata["w"] = w
    bm = gsb.BatchMatrix()
    bm.load_from_matrix(m, False)
    subm = bm[cuda(rows)::cuda(row_ptr), cuda(cols)::cuda(col_ptr)]
    assert np.array_equal(host(subm.edata["w"]), esel.astype(np.float32))
    # no rows at all
    sub, sel = A._CAPI_BatchColRowSlcing(cuda(cols), cuda(col_ptr), cuda(np.empty(0, np.int64)),
                                         cuda(np.zeros(B + 1, np.int64)))
    assert sel.numel() == 0 and not host(sub._CAPI_GetCSCIndptr()).any()


def test_slicing_on_coo(gsb, oracle, graph):
    indptr, indices = graph
    col = oracle.csc2coo(indptr)
    A = gsb.Graph(3000, 3000)
    A._CAPI_LoadCOO(cuda(indices), cuda(col), False, True)
    rng = np.random.default_rng(2)
    rows = rng.permutation(3000)[:500].astype(np.int64)
    sub, sel = A._CAPI_Slicing(cuda(rows), 0, gsb._COO, gsb._COO)
    pos = np.full(3000, -1)
    pos[rows] = np.arange(500)
    keep = np.flatnonzero(pos[indices] >= 0)
    assert np.array_equal(host(sel), keep)
    assert np.array_equal(host(sub._CAPI_GetCOORows()), pos[indices[keep]])
    assert np.array_equal(host(sub._CAPI_GetCOOCols()), col[keep])
    cols = rng.permutation(3000)[:400].astype(np.int64)
    sub, sel = A._CAPI_Slicing(cuda(cols), 1, gsb._COO, gsb._COO)
    pos = np.full(3000, -1)
    pos[cols] = np.arange(400)
    keep = np.flatnonzero(pos[col] >= 0)
    assert np.array_equal(host(sel), keep)
    assert np.array_equal(host(sub._CAPI_GetCOOCols()), pos[col[keep]])


def test_spmm_sddmm_against_oracle(gsb, oracle, graph):
    indptr, indices = graph
    n, E = indptr.size - 1, indices.size
    col = oracle.csc2coo(indptr)
    rng = np.random.default_rng(3)
    w = (rng.random(E) + 0.01).astype(np.float32)
    A = new_graph(gsb, indptr, indices)
    m = gsb.Matrix(A)
    m.edata["w"] = cuda(w, torch.float32)
    tol = dict(rtol=1e-5, atol=1e-6)
    # column sums (CSC, one warp per column) and row sums (COO atomics / CSR)
    assert np.allclose(host(m.sum("w", axis=0)), oracle.edge_sum(indices, col, w, 2, n), **tol)
    assert np.allclose(host(m.sum("w", axis=1)), oracle.edge_sum(indices, col, w, 0, n), **tol)
    A._CAPI_GetCSRIndptr()                     # now a CSR exists: the segmented kernel runs
    assert np.allclose(host(m.sum("w", axis=1)), oracle.edge_sum(indices, col, w, 0, n), **tol)
    # fused sum of squares
    assert np.allclose(host(gsb.ops.e_square_sum(m, m.edata["w"], 0, gsb._CSC)),
                       oracle.edge_sum(indices, col, w, 2, n, square=True), **tol)
    # e / node (SDDMM with the Python-side div -> mul rewrite)
    node = (rng.random(n) + 0.5).astype(np.float32)
    got = m.div("w", cuda(node, torch.float32), axis=1).edata["w"]
    assert np.allclose(host(got), oracle.edge_op_node(indices, w, node, "div"), **tol)
    got = m.div("w", cuda(node, torch.float32), axis=0).edata["w"]
    assert np.allclose(host(got), oracle.edge_op_node(col, w, node, "div"), **tol)
    # e / u summed per column, fused
    got = gsb.ops.e_div_u_sum(m, m.edata["w"], cuda(node, torch.float32), 0, gsb._CSC)
    want = oracle.edge_sum(indices, col, oracle.edge_op_node(indices, w, node, "div"), 2, n)
    # fp32 sums of positive terms in any order: compared with the fp64 sum of the same terms;
    # 1e-5 relative, and for segments long enough that rounding alone can exceed it the
    # statistical bound 4 * sqrt(terms) * 2^-24 (a 2 500-term hub: 1.2e-5)
    want64 = np.bincount(col, weights=w.astype(np.float64) / node.astype(np.float64)[indices], minlength=n)
    bound = np.maximum(1e-5, 4 * np.sqrt(np.diff(indptr)) * 2.0 ** -24)
    assert np.all(np.abs(host(got).astype(np.float64) - want64) <= bound * want64 + 1e-7)
    # vector features with broadcasting and a max reducer
    u = rng.random((n, 4)).astype(np.float32)
    e = rng.random((E, 1)).astype(np.float32)
    out = gsb.ops.gspmm(m, "mul", "max", cuda(u, torch.float32), cuda(e, torch.float32), 0, gsb._CSC)
    ref = np.zeros((n, 4), np.float32)
    for c in range(n):
        s, t = indptr[c], indptr[c + 1]
        if t > s:
            ref[c] = (u[indices[s:t]] * e[s:t]).max(axis=0)
    assert np.allclose(host(out), ref, **tol)
    out = gsb.ops.gsddmm(m, "add", cuda(u, torch.float32), cuda(u[:, :1].copy(), torch.float32), "u", "v")
    assert np.allclose(host(out), u[indices] + u[col, :1], **tol)
    # dot over the last feature dimension: plain vectors, multi-head, and one shared operand
    v = rng.random((n, 40)).astype(np.float32)
    out = gsb.ops.gsddmm(m, "dot", cuda(v, torch.float32), cuda(v, torch.float32), "u", "v")
    assert out.shape == (E, 1)
    assert np.allclose(host(out)[:, 0], (v[indices] * v[col]).sum(-1), rtol=1e-5, atol=1e-5)
    h = rng.random((n, 3, 8)).astype(np.float32)
    out = gsb.ops.gsddmm(m, "dot", cuda(h, torch.float32), cuda(h, torch.float32), "u", "v")
    assert out.shape == (E, 3, 1)
    assert np.allclose(host(out)[..., 0], (h[indices] * h[col]).sum(-1), rtol=1e-5, atol=1e-5)
    h1 = rng.random((n, 1, 8)).astype(np.float32)
    out = gsb.ops.gsddmm(m, "dot", cuda(h, torch.float32), cuda(h1, torch.float32), "v", "u")
    assert np.allclose(host(out)[..., 0], (h[col] * h1[indices]).sum(-1), rtol=1e-5, atol=1e-5)
    ew = rng.random((E, 8)).astype(np.float32)
    out = gsb.ops.gsddmm(m, "dot", cuda(ew, torch.float32), cuda(h1[:, 0].copy(), torch.float32), "e", "v")
    assert np.allclose(host(out)[:, 0], (ew * h1[col, 0]).sum(-1), rtol=1e-5, atol=1e-5)


def test_list_sampling(gsb, oracle):
    from scipy import stats

    ops = torch.ops.gs_ops
    ops._CAPI_SetListSamplingSeed(31)
    # uniform without replacement: bit-exact with the oracle (integer keys)
    got = host(ops._CAPI_ListSampling(5000, 400, False))
    assert np.array_equal(got, oracle.list_sample_spec(5000, 400, False, seed=31, stream=0))
    got = host(ops._CAPI_ListSampling(100, 400, False))
    assert got.tolist() == list(range(100))
    got = host(ops._CAPI_ListSampling(5000, 64, True))
    assert np.array_equal(got, oracle.list_sample_spec(5000, 64, True, seed=31, stream=2))
    # weighted: zero-weight items never win while positive ones remain; high overlap with the
    # double-precision oracle (fp32 keys may reorder near-ties at the threshold)
    rng = np.random.default_rng(4)
    probs = rng.random(20000).astype(np.float32)
    probs[:3000] = 0
    ops._CAPI_SetListSamplingSeed(5)
    got = host(ops._CAPI_ListSamplingWithProbs(cuda(probs, torch.float32), 2000, False))
    want = oracle.list_sample_probs_spec(probs, 2000, seed=5, stream=0)
    assert got.size == 2000 and np.unique(got).size == 2000 and np.all(np.diff(got) > 0)
    assert np.all(probs[got] > 0)
    assert np.intersect1d(got, want).size >= 1990
    # segments, including one shorter than K and an empty one
    rp = np.array([0, 50, 50, 9000, 20000])
    idx, optr = ops._CAPI_BatchListSamplingWithProbs(cuda(probs, torch.float32), 300, False, cuda(rp))
    idx, optr = host(idx), host(optr)
    assert optr.tolist() == [0, 50, 50, 350, 650]
    assert idx[:50].tolist() == list(range(50))
    for b in (2, 3):
        seg = idx[optr[b]:optr[b + 1]]
        assert np.all((seg >= rp[b]) & (seg < rp[b + 1])) and np.unique(seg).size == 300
    idx, optr = ops._CAPI_BatchListSampling(10, False, cuda(np.array([0, 4, 104])))
    assert host(optr).tolist() == [0, 4, 14]
    # distribution: K = 1 of 8 weighted items, many independent calls
    w = np.array([1, 2, 3, 4, 0.5, 0.5, 6, 3], np.float32)
    big = np.tile(w, 4000)
    rp = np.arange(4001) * 8
    idx, _ = ops._CAPI_BatchListSamplingWithProbs(cuda(big, torch.float32), 1, False, cuda(rp))
    cnt = np.bincount(host(idx) % 8, minlength=8)
    w64 = w.astype(np.float64)
    assert stats.chisquare(cnt, 4000 * w64 / w64.sum()).pvalue > 0.01
    # with replacement, weighted
    got = host(ops._CAPI_ListSamplingWithProbs(cuda(w, torch.float32), 16000, True))
    assert stats.chisquare(np.bincount(got, minlength=8), 16000 * w64 / w64.sum()).pvalue > 0.01
    # uniform reservoir: 3 of 12 in 6000 independent segments -- distinct picks inside every
    # segment, bit-exact with the oracle, every item equally likely
    rp = np.arange(6001) * 12
    ops._CAPI_SetListSamplingSeed(9)
    idx, optr = ops._CAPI_BatchListSampling(3, False, cuda(rp))
    idx, optr = host(idx), host(optr)
    assert optr.tolist() == (np.arange(6001) * 3).tolist()
    want, _ = oracle.list_sample_probs_spec(None, 3, seed=9, stream=0, range_ptr=rp, n=int(rp[-1]))
    assert np.array_equal(idx, want)
    picks = idx.reshape(6000, 3)
    assert np.all(picks // 12 == np.arange(6000)[:, None])
    assert np.all(np.sort(picks, axis=1)[:, 1:] != np.sort(picks, axis=1)[:, :-1])
    assert stats.chisquare(np.bincount(idx % 12, minlength=12)).pvalue > 0.01


def test_walk_entry_points_all_widths(oracle, graph):
    """gsb_random_walk / gsb_node2vec through the C ABI with 64-bit or 32-bit offsets and 64-bit or
    32-bit row ids (the host layer always hands a small graph the 32-bit copies): the four
    combinations give the oracle's traces bit for bit."""
    from tests import abi

    indptr, indices = graph
    srt = oracle.sort_indices(indptr, indices)
    rng = np.random.default_rng(16)
    seeds = cuda(rng.integers(0, 3000, 4000).astype(np.int64))
    want_rw = oracle.random_walk_spec(indptr, srt, host(seeds), 9, 5, 3)
    want_n2v = oracle.node2vec_spec(indptr, srt, host(seeds), 9, 0.5, 2.0, 5, 4)
    ip64, ip32 = cuda(indptr), cuda(indptr).to(torch.int32)
    for ids in (cuda(srt), cuda(srt, torch.int32)):
        for a, b in ((ip64, None), (None, ip32), (ip64, ip32)):
            tr, err = abi.random_walk(a, ids, seeds, 9, 5, 3, indptr32=b)
            assert err == 0 and np.array_equal(host(tr), want_rw)
            tr, err = abi.random_walk(a, ids, seeds, 9, 5, 4, indptr32=b, node2vec=(0.5, 2.0))
            assert err == 0 and np.array_equal(host(tr), want_n2v)


def test_list_sampling_whole_list_without_offsets(oracle):
    """gsb_list_sample with range == NULL (one list [0, n), uniform): the reservoir spec's picks,
    nothing read or written besides them; K >= n returns the whole list."""
    from tests import abi

    for n, K in ((100000, 500), (5000, 4999), (300, 300), (300, 1000)):
        got, err = abi.list_sample_whole(n, K, 11, 2)
        assert err == 0
        assert np.array_equal(host(got), oracle.list_sample_spec(n, K, seed=11, stream=2))


def test_walks_bit_exact(gsb, oracle, graph):
    indptr, indices = graph
    srt = oracle.sort_indices(indptr, indices)
    rng = np.random.default_rng(6)
    seeds = rng.integers(0, 3000, 5000).astype(np.int64)
    for idx_dtype in (torch.int64, torch.int32):
        A = new_graph(gsb, indptr, indices, seed=77, idx_dtype=idx_dtype)
        A._CAPI_SortCSCIndices()
        assert np.array_equal(host(A._CAPI_GetCSCIndices()), srt)
        tr = A._CAPI_RandomWalk(cuda(seeds), 12)
        assert tuple(tr.shape) == (5000, 13)
        assert np.array_equal(host(tr).reshape(-1), oracle.random_walk_spec(indptr, srt, seeds, 12, 77, 0))
        tr = A._CAPI_Node2Vec(cuda(seeds), 12, 2.0, 0.5)
        assert np.array_equal(host(tr).reshape(-1), oracle.node2vec_spec(indptr, srt, seeds, 12, 2.0, 0.5, 77, 1))
        tr = A._CAPI_Node2Vec(cuda(seeds), 5, 0.25, 4.0)
        assert np.array_equal(host(tr).reshape(-1), oracle.node2vec_spec(indptr, srt, seeds, 5, 0.25, 4.0, 77, 2))


def test_reference_walk_fixture(gsb):
    with open(os.path.join(HERE, "golden", "reference_fixtures.json")) as f:
        c = json.load(f)["walks"]
    indptr, indices = np.asarray(c["indptr"]), np.asarray(c["indices"])
    A = new_graph(gsb, indptr, indices)
    L, seeds = c["walk_length"], c["seeds"]
    for walk in (A._CAPI_RandomWalk(cuda(seeds), L), A._CAPI_Node2Vec(cuda(seeds), L, c["p"], c["q"])):
        t = host(walk.reshape(-1, len(seeds)))          # step-major, as the reference's test reads it
        assert t[0].tolist() == seeds
        for w in range(len(seeds)):
            for s in range(L):
                a, b = t[s, w], t[s + 1, w]
                assert b == -1 or b in indices[indptr[a]:indptr[a + 1]]
        assert t[:, 3].tolist() == [1, 0, -1, -1]


def test_compact_and_index_search(gsb, oracle, graph):
    indptr, indices = graph
    A = new_graph(gsb, indptr, indices)
    sub, _ = A._CAPI_Slicing(cuda(np.arange(100)), 1, gsb._CSC, gsb._CSC + gsb._COO)
    g2, frontier = sub._CAPI_Compact(0)
    uq, cp = oracle.compact(host(sub._CAPI_GetCSCIndices()))
    assert np.array_equal(host(frontier), uq) and np.array_equal(host(g2._CAPI_GetCSCIndices()), cp)
    assert g2._CAPI_GetNumRows() == uq.size
    # the COO and the CSC of one graph in different edge orders: each is mapped in its own order
    rng = np.random.default_rng(2)
    n, nnz = 5000, 60000
    row, col = rng.integers(0, n, nnz) * 3 % n, rng.integers(0, 700, nnz)
    g = gsb.Graph(n, 700)
    g._CAPI_LoadCOO(cuda(row), cuda(col), False, False)
    csc_rows = host(g._CAPI_GetCSCIndices())                 # grouped by column: another order than `row`
    assert not np.array_equal(csc_rows, row)
    for axis, ids in ((0, row), (1, col)):
        g3, fr = g._CAPI_Compact(axis)
        uq = np.unique(ids)
        assert np.array_equal(host(fr), uq)
        got = host(g3._CAPI_GetCOORows() if axis == 0 else g3._CAPI_GetCOOCols())
        assert np.array_equal(got, np.searchsorted(uq, ids))
        assert (g3._CAPI_GetNumRows() if axis == 0 else g3._CAPI_GetNumCols()) == uq.size
        if axis == 0:
            assert np.array_equal(host(g3._CAPI_GetCSCIndices()), np.searchsorted(uq, csc_rows))
    data = cuda(np.array([7, 3, 9, 11]))
    keys = cuda(np.array([9, 4, 7, 11, 3]))
    assert host(torch.ops.gs_ops._CAPI_IndexSearch(data, keys)).tolist() == [2, -1, 0, 3, 1]
    # a large table with repeated values (the smallest position wins), absent keys, ids beyond 2^32, shaped keys
    big = rng.integers(0, 2 ** 40, 300_000)
    big[rng.integers(0, big.size, 50_000)] = big[rng.integers(0, 1000, 50_000)]
    look = np.concatenate([big[rng.integers(0, big.size, 100_000)], rng.integers(2 ** 41, 2 ** 42, 20_000)]).reshape(400, 300)
    first = {}
    for i, v in enumerate(big.tolist()):
        first.setdefault(v, i)
    want = np.array([first.get(v, -1) for v in look.reshape(-1).tolist()]).reshape(look.shape)
    assert np.array_equal(host(torch.ops.gs_ops._CAPI_IndexSearch(cuda(big), cuda(look))), want)
    assert host(torch.ops.gs_ops._CAPI_IndexSearch(cuda(np.empty(0, np.int64)), keys)).tolist() == [-1] * 5
    gsb.check_async_errors()


def test_ladies_sampler_layer(gsb, oracle):
    """One LADIES layer (examples/ladies/ladies.py:7-21 of the reference) on the Matrix API; every
    deterministic stage is recomputed with the oracle from the rows the GPU selected."""
    rng = np.random.default_rng(9)
    indptr, indices = rand_csc(rng, 4000, 60)
    n, E = indptr.size - 1, indices.size
    w = (rng.random(E) + 0.05).astype(np.float32)
    m = gsb.Matrix(new_graph(gsb, indptr, indices))
    m.edata["w"] = cuda(w, torch.float32)
    torch.ops.gs_ops._CAPI_SetListSamplingSeed(3)
    seeds = rng.permutation(n)[:128].astype(np.int64)
    K = 500

    subA = m[:, cuda(seeds)]
    subA.edata["p"] = subA.edata["w"] ** 2
    prob = subA.sum("p", axis=1)
    sampleA, select_index = subA.collective_sampling(K, prob, False)
    sampleA = sampleA.div("w", prob[select_index], axis=1)
    out = sampleA.sum("w", axis=0)
    sampleA = sampleA.div("w", out, axis=0)
    nodes = sampleA.all_nodes()
    block = sampleA.to_dgl_block(prefetch_edata={"w"})

    sip, srows, scols, ssel = oracle.slice_cols(indptr, indices, seeds)
    p_ref = oracle.edge_sum(srows, scols, w[ssel], 0, n, square=True)
    assert np.allclose(host(prob), p_ref, rtol=1e-5, atol=1e-7)
    sel = host(select_index)
    assert sel.size == K and np.unique(sel).size == K and np.all(p_ref[sel] > 0)
    # row slice of the column slice, taken on the CSR view like Matrix.__getitem__ does
    csr_ip, csr_cols, perm = oracle.coo2csc(srows, scols, n)
    rip, rcols, rloc, rsel = oracle.slice_cols(csr_ip, csr_cols, sel)
    edge_w = w[ssel][perm][rsel]
    w1 = oracle.edge_op_node(rloc, edge_w, p_ref[sel], "div")
    colsum = oracle.edge_sum(rloc, rcols, w1, 2, seeds.size)
    w2 = oracle.edge_op_node(rcols, w1, colsum, "div")
    # every stage is held to 1e-5 relative on its own (asserts above and in
    # test_spmm_sddmm_against_oracle); `out` chains two such stages (w / prob, then the sum) and
    # the final weights three, so their bounds are 2e-5 and 3e-5
    assert np.allclose(host(out), colsum, rtol=2e-5, atol=1e-7)
    assert np.array_equal(host(sampleA._graph._CAPI_GetCOORows()), rloc)
    assert np.array_equal(host(sampleA._graph._CAPI_GetCOOCols()), rcols)
    assert np.allclose(host(sampleA.edata["w"]), w2, rtol=3e-5, atol=1e-7)
    # frontier and block: unique(cat(seeds, selected rows that carry an edge)), relabelled COO
    frontier, nrow, ncol = oracle.relabel(seeds, sel[rloc], rcols)
    assert np.array_equal(host(block.srcdata["_ID"]), frontier)
    assert np.array_equal(host(block.row), nrow) and np.array_equal(host(block.col), ncol)
    assert np.allclose(host(block.edata["w"]), w2, rtol=3e-5, atol=1e-7)
    assert np.array_equal(np.sort(host(nodes)), np.sort(frontier))


def test_ladies_layer_native_call(gsb, oracle):
    """The same layer through the single native call (Matrix.ladies_layer): every stage is
    recomputed on the host from the rows the GPU picked; the kept edges stay in column order."""
    rng = np.random.default_rng(19)
    indptr, indices = rand_csc(rng, 5000, 50, heavy=5)
    n, E = indptr.size - 1, indices.size
    w = (rng.random(E) + 0.05).astype(np.float32)
    m = gsb.Matrix(new_graph(gsb, indptr, indices))
    m.edata["w"] = cuda(w, torch.float32)
    torch.ops.gs_ops._CAPI_SetListSamplingSeed(3)
    seeds = rng.permutation(n)[:200].astype(np.int64)
    K = 600
    block, nodes, picked = m.ladies_layer(cuda(seeds), K)
    picked = host(picked)
    sip, srows, scols, ssel = oracle.slice_cols(indptr, indices, seeds)
    p_ref = oracle.edge_sum(srows, scols, w[ssel], 0, n, square=True)
    assert picked.size == K and np.unique(picked).size == K and np.all(p_ref[picked] > 0)
    assert np.all(np.diff(picked) > 0)                      # ascending, like _CAPI_ListSamplingWithProbs
    spec = oracle.list_sample_probs_spec(p_ref, K, seed=3, stream=0)
    assert np.intersect1d(picked, spec).size >= K - 2        # same draw up to fp32 summation order of p
    mask = np.isin(srows, picked)
    pos = np.full(n, -1)
    pos[picked] = np.arange(K)
    kept_rows, kept_cols = srows[mask], scols[mask]
    assert np.array_equal(host(block.edata["_ID"]), ssel[mask])
    w1 = w[ssel][mask] / p_ref[kept_rows]
    colsum = np.bincount(kept_cols, weights=w1, minlength=seeds.size)
    assert np.allclose(host(block.edata["w"]), w1 / colsum[kept_cols], rtol=5e-5, atol=1e-7)
    frontier, nrow, ncol = oracle.relabel(seeds, kept_rows, kept_cols)
    assert np.array_equal(host(nodes), frontier) and np.array_equal(host(block.srcdata["_ID"]), frontier)
    assert np.array_equal(host(block.row), nrow) and np.array_equal(host(block.col), ncol)
    assert block.num_src == frontier.size and block.num_dst == seeds.size
    # a second layer on the new frontier runs, and K larger than the row count is clamped
    block2, nodes2, picked2 = m.ladies_layer(nodes, 10 ** 7)
    assert picked2.numel() == n and block2.num_dst == nodes.numel()


def test_node2vec_sampler_api(gsb, oracle, graph):
    """examples/node2vec/node2vec.py:10-29 of the reference on this package's Matrix."""
    indptr, indices = graph
    m = gsb.Matrix(new_graph(gsb, indptr, indices, seed=5))
    m._graph._CAPI_SortCSCIndices()
    seeds = np.random.default_rng(0).integers(0, 3000, 128).astype(np.int64)

    def node2vec_sampler(A, seeds, walk_length, p, q):
        return A.node2vec(seeds, walk_length, p, q)

    # (no timing runs at compile time, so that the first call draws from the graph's stream 0)
    fn = gsb.jit.compile(func=node2vec_sampler, args=(m, cuda(seeds), 80, 2.0, 0.5), try_compact=False,
                         format_select=False)
    paths = fn(m, cuda(seeds), 80, 2.0, 0.5)
    srt = oracle.sort_indices(indptr, indices)
    assert np.array_equal(host(paths).reshape(-1), oracle.node2vec_spec(indptr, srt, seeds, 80, 2.0, 0.5, 5, 0))


@pytest.mark.parametrize("dtype,width", [(torch.float32, 100), (torch.float32, 128), (torch.float16, 7),
                                         (torch.int64, 1), (torch.uint8, 3), (torch.float32, 0)])
def test_gather_rows_device_and_pinned(gsb, dtype, width):
    """Feature fetch: rows gathered from GPU memory and, in place, from pinned host memory."""
    g = torch.Generator()
    g.manual_seed(3)
    n = 5000
    shape = (n,) if width == 0 else (n, width)
    data = (torch.rand(shape, generator=g) * 200).to(dtype)
    idx = torch.randint(0, n, (12345,), generator=g)
    want = data[idx]
    got = gsb.gather_rows(data.cuda(), idx.cuda())
    assert got.dtype == dtype and got.shape == want.shape and torch.equal(got.cpu(), want)
    got = gsb.gather_rows(data.pin_memory(), idx.cuda())
    assert got.is_cuda and torch.equal(got.cpu(), want)
    assert gsb.gather_rows(data.cuda(), idx[:0].cuda()).shape[0] == 0
    gsb.check_async_errors()
    with pytest.raises(RuntimeError):
        gsb.gather_rows(data, idx.cuda())          # pageable host memory is rejected


def test_gather_rows_reports_bad_index(gsb):
    data = torch.arange(40, dtype=torch.float32).view(10, 4).cuda()
    out = gsb.gather_rows(data, cuda(np.array([1, 10, 3, -1])))
    assert torch.equal(out[0].cpu(), data[1].cpu()) and torch.equal(out[2].cpu(), data[3].cpu())
    with pytest.raises(RuntimeError):
        gsb.check_async_errors()
    gsb.check_async_errors()                        # the word is cleared by the report


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_graph_in_pinned_host_memory(gsb, oracle, graph, idx_dtype):
    """A CSC kept in pinned host memory is sliced / sampled in place, with the same results as
    the GPU-resident graph (same seed, same streams)."""
    indptr, indices = graph
    n = indptr.size - 1
    rng = np.random.default_rng(12)
    seeds = cuda(rng.integers(0, n, 800))
    ptr = cuda(np.array([0, 300, 300, 800]))

    def make(pinned):
        ip, ix = torch.from_numpy(indptr), torch.from_numpy(indices).to(idx_dtype)
        g = gsb.Graph(n, n)
        if pinned:
            g._CAPI_LoadCSC(ip.pin_memory(), ix.pin_memory())
        else:
            g._CAPI_LoadCSC(ip.cuda(), ix.cuda())
        g._CAPI_SetSeed(5)
        return g

    dev, pin = make(False), make(True)
    for fn in (lambda g: g._CAPI_Slicing(seeds, 1, gsb._CSC, gsb._CSC + gsb._COO),
               lambda g: g._CAPI_SlicingSampling(1, seeds, 7, False, gsb._CSC, gsb._CSC + gsb._COO),
               lambda g: g._CAPI_BatchFusedSlicingSampling(seeds, ptr, 4, True)):
        (ga, sa), (gb, sb) = fn(dev), fn(pin)
        assert sb.is_cuda and torch.equal(sa, sb)
        assert torch.equal(ga._CAPI_GetCSCIndptr(), gb._CAPI_GetCSCIndptr())
        assert torch.equal(ga._CAPI_GetCSCIndices(), gb._CAPI_GetCSCIndices())
        assert torch.equal(ga._CAPI_GetCOOCols(), gb._CAPI_GetCOOCols())
    la = dev._CAPI_BatchGraphSAGE(seeds, ptr, [5, 3])
    lb = pin._CAPI_BatchGraphSAGE(seeds, ptr, [5, 3])
    assert len(la) == len(lb) and all(torch.equal(a.cpu(), b.cpu()) for a, b in zip(la, lb))
    # pre-allocated pipeline on the pinned graph
    smp = gsb.GraphSAGESampler(torch.from_numpy(indptr).pin_memory(),
                               torch.from_numpy(indices).to(idx_dtype).pin_memory(), 3, 800, [5, 3], seed=5)
    smp.sample(seeds, ptr)
    counts = smp.counts()
    ref = oracle.graphsage_batch(indptr, indices, host(seeds), host(ptr), [5, 3], seed=5)
    for l in range(2):
        S, E, U = counts[l]
        assert (S, E, U) == (ref[l]["seeds"].size, ref[l]["rows"].size, ref[l]["unique"].size)
        assert np.array_equal(host(smp.layers[l]["unique"][:U]), ref[l]["unique"])
        assert np.array_equal(host(smp.layers[l]["block_row"][:E]), ref[l]["block_row"])


def test_lazy_slice_with_edge_data_in_pinned_host_memory(gsb, graph):
    """``A[:, seeds].individual_sampling(...)`` runs as one fused kernel (the slice is lazy) and then
    gathers the PARENT's edge data with the fused edge index: the same values as slicing first and
    sampling the slice, also when the edge data lives in pinned host memory, and also when the
    parent's edge data is edited between the slice and the sampling."""
    indptr, indices = graph
    n, E = indptr.size - 1, indices.size
    rng = np.random.default_rng(21)
    w = torch.from_numpy(rng.random(E).astype(np.float32))
    seeds = cuda(rng.permutation(n)[:500])
    results = []
    for where in ("device", "pinned"):
        for lazy in (True, False):
            m = gsb.Matrix(new_graph(gsb, indptr, indices, seed=8))
            m.edata["w"] = w.cuda() if where == "device" else w.clone().pin_memory()
            sub = m[:, seeds]
            if not lazy:
                sub.num_edges()                      # any other use materialises the slice first
            else:
                m.edata["extra"] = m.edata["w"]      # an edit of the parent after the slice: not seen by it
            s = sub.individual_sampling(6, None, False)
            assert "extra" not in s.edata
            assert s.edata["w"].is_cuda
            results.append((s.edata["w"], s._graph._CAPI_GetCOORows(), s._graph._CAPI_GetCOOCols()))
    for r in results[1:]:
        assert all(torch.equal(a, b) for a, b in zip(results[0], r))
