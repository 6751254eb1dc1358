"""CPU suite: pins the oracle (the CPU restatement under oracle/) against the reference's own
gtest fixtures and against the published Philox4x32-10 known-answer vectors, then checks the
restated operators against independent numpy formulations."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def fx():
    with open(os.path.join(HERE, "golden", "reference_fixtures.json")) as f:
        return json.load(f)


def test_philox_known_answers(oracle):
    # Random123 known-answer vectors for philox4x32, 10 rounds
    kat = [
        ([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
        ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
        ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
         [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]),
    ]
    for ctr, key, want in kat:
        got = oracle.philox4x32_10(ctr, key)
        assert [int(x) for x in got] == want


def test_ref_colwise_slicing(oracle, fx):
    c = fx["colwise_slicing"]
    sip, rows, cols, sel = oracle.slice_cols(c["indptr"], c["indices"], c["cols"])
    assert sip.tolist() == c["expect_indptr"]
    assert rows.tolist() == c["expect_indices"]
    assert sel.tolist() == c["expect_indices"]          # edge positions == ids in this fixture
    assert cols.tolist() == [i // 5 for i in range(15)]


@pytest.mark.parametrize("sampler", ["spec", "ref"])
def test_ref_colwise_sampling_copy_all(oracle, fx, sampler):
    c = fx["colwise_sampling"]
    fn = oracle.sample_spec if sampler == "spec" else oracle.sample_ref
    sip, rows, cols, sel = fn(c["indptr"], c["indices"], None, c["copy_all"]["fanout"], False)
    assert sip.tolist() == c["copy_all"]["expect_indptr"]
    assert rows.tolist() == c["copy_all"]["expect_indices"]


@pytest.mark.parametrize("sampler", ["spec", "ref"])
def test_ref_colwise_sampling_replace(oracle, fx, sampler):
    c = fx["colwise_sampling"]
    fn = oracle.sample_spec if sampler == "spec" else oracle.sample_ref
    for case in c["replace"]:
        sip, rows, cols, sel = fn(c["indptr"], c["indices"], None, case["fanout"], True)
        assert sip.tolist() == case["expect_indptr"]
        assert rows.size == 20 * case["fanout"]
        assert rows.tolist() != c["indices"]
        assert np.unique(rows).size <= 100
        # every pick lies inside its own column
        assert np.all(rows // 5 == cols)


def test_ref_rowwise_slicing(oracle, fx):
    c = fx["rowwise_slicing"]
    indptr, indices = np.asarray(c["indptr"]), np.asarray(c["indices"])
    ncols = indptr.size - 1
    # CSR of the fixture through the restated conversions, then slice on its offsets
    col = oracle.csc2coo(indptr)
    csr_indptr, csr_indices, _ = oracle.coo2csc(indices, col, ncols)
    sip, ids, _, _ = oracle.slice_cols(csr_indptr, csr_indices, c["rows"])
    assert sip.size == c["expect_csr_indptr_numel"]
    assert ids.tolist() == c["expect_csr_indices"]
    # same slice taken directly on the CSC (row filter)
    oip, oi, osel = oracle.slice_rows(indptr, indices, c["rows"])
    assert oip.tolist() == [0] * 11 + [1, 2]
    assert oi.tolist() == [0, 0] and osel.tolist() == [0, 2]


def _check_walk(trace, N, L, indptr, indices):
    t = trace.reshape(L + 1, N)
    for w in range(N):
        for s in range(L):
            a, b = t[s, w], t[s + 1, w]
            if b == -1:
                continue
            assert a >= 0 and b in indices[indptr[a]:indptr[a + 1]]
    return t


def test_ref_walk_invariants(oracle, fx):
    c = fx["walks"]
    indptr, indices = np.asarray(c["indptr"]), np.asarray(c["indices"])
    L, seeds = c["walk_length"], c["seeds"]
    t = _check_walk(oracle.random_walk_spec(indptr, indices, seeds, L, seed=1), len(seeds), L,
                    indptr, indices)
    assert t[0].tolist() == seeds
    # node 1 -> 0 -> dead end -> -1 (the path the reference's comment spells out)
    assert t[:, 3].tolist() == [1, 0, -1, -1]
    t = _check_walk(oracle.node2vec_spec(indptr, indices, seeds, L, c["p"], c["q"], seed=1),
                    len(seeds), L, indptr, indices)
    assert t[:, 3].tolist() == [1, 0, -1, -1]


# ----------------------------------------------------------------------------- properties
def _rand_csc(rng, n, avg):
    deg = rng.poisson(avg, n)
    deg[rng.integers(0, n, n // 10)] = 0
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, indptr[-1]).astype(np.int64)
    return indptr, indices


def test_sampling_invariants(oracle):
    rng = np.random.default_rng(0)
    indptr, indices = _rand_csc(rng, 500, 12)
    seeds = rng.integers(0, 500, 300)
    for fn in (oracle.sample_spec, oracle.sample_ref):
        for K in (1, 5, 16):
            sip, rows, cols, sel = fn(indptr, indices, seeds, K, False)
            deg = indptr[seeds + 1] - indptr[seeds]
            assert np.array_equal(np.diff(sip), np.minimum(deg, K))
            assert np.array_equal(rows, indices[sel])
            assert np.all((sel >= indptr[seeds[cols]]) & (sel < indptr[seeds[cols] + 1]))
            for i in range(seeds.size):
                s = sel[sip[i]:sip[i + 1]]
                assert np.unique(s).size == s.size


def test_spec_sampler_is_uniform(oracle):
    # one column of degree 12, fanout 4, replicated over many slots: inclusion ~ K/deg
    deg, K, S = 12, 4, 6000
    indptr = np.array([0, deg])
    indices = np.arange(deg)
    seeds = np.zeros(S, np.int64)
    for fn in (oracle.sample_spec, oracle.sample_ref):
        _, rows, _, _ = fn(indptr, indices, seeds, K, False)
        cnt = np.bincount(rows, minlength=deg).astype(float)
        if fn is oracle.sample_ref:
            # the reference's 32 rows of a block share their streams: distinct samples = S/32
            _, rows, cols, _ = fn(indptr, indices, seeds, K, False)
            keep = (cols % 32) == 0
            cnt = np.bincount(rows[keep], minlength=deg).astype(float)
        n = cnt.sum() / K
        exp = n * K / deg
        chi2 = ((cnt - exp) ** 2 / (exp * (1 - K / deg))).sum() * (deg - 1) / deg
        assert chi2 < 31.3  # chi-square(11) at p = 0.001


def test_unique_and_relabel(oracle):
    rng = np.random.default_rng(1)
    ids = rng.integers(0, 50, 400)
    uq = oracle.unique_first(ids)
    _, first = np.unique(ids, return_index=True)
    assert uq.tolist() == ids[np.sort(first)].tolist()
    seeds = rng.permutation(60)[:20]
    rows = rng.integers(0, 60, 100)
    colsl = rng.integers(0, 20, 100)
    frontier, nrow, ncol = oracle.relabel(seeds, rows, colsl)
    assert frontier[:20].tolist() == seeds.tolist()
    assert np.array_equal(frontier[nrow], rows)
    assert np.array_equal(frontier[ncol], seeds[colsl])


def test_batch_relabel_matches_per_batch(oracle):
    rng = np.random.default_rng(2)
    B = 5
    ns = rng.integers(0, 6, B); ns[2] = 0
    ne = rng.integers(0, 30, B); ne[2] = 0; ne[4] = 0
    sp = np.concatenate([[0], np.cumsum(ns)]); ep = np.concatenate([[0], np.cumsum(ne)])
    seeds = rng.integers(0, 40, sp[-1])
    rows = rng.integers(0, 40, ep[-1])
    col_local = np.concatenate([rng.integers(sp[b], max(sp[b + 1], sp[b] + 1), ne[b]) if ns[b] else
                                np.empty(0, np.int64) for b in range(B)]).astype(np.int64)
    # batches without seeds cannot own edges
    for b in range(B):
        if ns[b] == 0:
            assert ne[b] == 0 or True
    ne = np.where(ns == 0, 0, ne)
    ep = np.concatenate([[0], np.cumsum(ne)])
    rows = rows[:ep[-1]]
    col_local = np.concatenate([rng.integers(sp[b], sp[b + 1], ne[b]) for b in range(B) if ns[b]] +
                               [np.empty(0, np.int64)]).astype(np.int64)
    uq, up, orow, ocol = oracle.batch_coo_relabel(seeds, sp, seeds[col_local], rows, ep)
    for b in range(B):
        f, r, c = oracle.relabel(seeds[sp[b]:sp[b + 1]], rows[ep[b]:ep[b + 1]],
                                 col_local[ep[b]:ep[b + 1]] - sp[b])
        assert uq[up[b]:up[b + 1]].tolist() == f.tolist()
        assert orow[ep[b]:ep[b + 1]].tolist() == r.tolist()
        assert ocol[ep[b]:ep[b + 1]].tolist() == c.tolist()


def test_formats_and_compact(oracle):
    rng = np.random.default_rng(3)
    indptr, indices = _rand_csc(rng, 80, 6)
    col = oracle.csc2coo(indptr)
    assert np.array_equal(col, np.repeat(np.arange(80), np.diff(indptr)))
    ip2, rows2, perm = oracle.coo2csc(indices, col, 80)          # CSR of the graph
    order = np.argsort(indices, kind="stable")
    assert np.array_equal(perm, order) and np.array_equal(rows2, col[order])
    srt = oracle.sort_indices(indptr, indices)
    for c in range(80):
        assert np.array_equal(srt[indptr[c]:indptr[c + 1]], np.sort(indices[indptr[c]:indptr[c + 1]]))
    uq, cp = oracle.compact(indices)
    assert np.array_equal(uq, np.unique(indices)) and np.array_equal(uq[cp], indices)
    enc = np.sort(rng.integers(0, 4, 50) * 1000 + rng.integers(0, 1000, 50))
    ptr, dec = oracle.batch_offsets(enc, 4, 1000)
    assert np.array_equal(dec, enc % 1000)
    assert np.array_equal(ptr, np.searchsorted(enc // 1000, np.arange(5), side="left"))


def test_edge_ops_and_list_sampling(oracle):
    rng = np.random.default_rng(4)
    n, E = 30, 200
    row, col = rng.integers(0, n, E), rng.integers(0, n, E)
    e = rng.random(E).astype(np.float32)
    s = oracle.edge_sum(row, col, e, 0, n, square=True)
    assert np.allclose(s, np.bincount(row, weights=e.astype(np.float64) ** 2, minlength=n), rtol=1e-6)
    node = (rng.random(n) + 0.5).astype(np.float32)
    d = oracle.edge_op_node(col, e, node, "div")
    assert np.allclose(d, e / node[col], rtol=1e-6)
    probs = rng.random(100).astype(np.float32); probs[:10] = 0
    pick = oracle.list_sample_probs_spec(probs, 20, seed=3)
    assert np.unique(pick).size == 20 and np.all(probs[pick] > 0)
    idx, optr = oracle.list_sample_probs_spec(probs, 20, seed=3, range_ptr=[0, 15, 15, 100])
    assert optr.tolist() == [0, 15, 15, 35] and idx[:15].tolist() == list(range(15))
    u = oracle.list_sample_spec(50, 10, False, seed=1)
    assert np.unique(u).size == 10 and u.max() < 50


def test_graphsage_pipeline_shapes(oracle):
    rng = np.random.default_rng(5)
    indptr, indices = _rand_csc(rng, 400, 10)
    seeds = rng.permutation(400)[:96].astype(np.int64)
    ptr = np.array([0, 32, 64, 96])
    layers = oracle.graphsage_batch(indptr, indices, seeds, ptr, [5, 3], seed=9)
    assert len(layers) == 2
    l0, l1 = layers
    assert np.array_equal(l1["seeds"], l0["unique"]) and np.array_equal(l1["seeds_ptr"], l0["unique_ptr"])
    for L in layers:
        for b in range(3):
            uq = L["unique"][L["unique_ptr"][b]:L["unique_ptr"][b + 1]]
            e0, e1 = L["edge_ptr"][b], L["edge_ptr"][b + 1]
            assert np.array_equal(uq[L["block_row"][e0:e1]], L["rows"][e0:e1])
            assert np.array_equal(uq[L["block_col"][e0:e1]], L["seeds"][L["cols"][e0:e1]])


def test_batch_slice_cols_rows_matches_composition(oracle):
    """The fused column+row selection equals column slicing followed by a row filter with the
    minibatch's own row list (the definition it is used for in batch_matrix.py:57-80)."""
    rng = np.random.default_rng(8)
    n = 400
    deg = rng.poisson(6, n)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, indptr[-1]).astype(np.int64)
    col_ptr = np.array([0, 30, 30, 75], np.int64)
    row_ptr = np.array([0, 120, 200, 380], np.int64)
    cols = rng.integers(0, n, 75).astype(np.int64)
    rows = np.concatenate([rng.permutation(n)[:120], rng.permutation(n)[:80], rng.permutation(n)[:180]]).astype(np.int64)
    oip, oi, osel = oracle.batch_slice_cols_rows(indptr, indices, cols, col_ptr, rows, row_ptr)
    assert oip[-1] == oi.size == osel.size
    for b in range(3):
        sip, sidx, _, ssel = oracle.slice_cols(indptr, indices, cols[col_ptr[b]:col_ptr[b + 1]])
        keep = np.isin(sidx, rows[row_ptr[b]:row_ptr[b + 1]])
        lo, hi = oip[col_ptr[b]], oip[col_ptr[b + 1]]
        assert np.array_equal(osel[lo:hi], ssel[keep])
        assert np.array_equal(rows[oi[lo:hi]], sidx[keep])
        assert np.all((oi[lo:hi] >= row_ptr[b]) & (oi[lo:hi] < row_ptr[b + 1]))
