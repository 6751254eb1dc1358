"""Parity against the reference's OWN CUDA implementation (tier-2 oracle): the reference's kernel
files compiled unmodified into ``oracle/_ref/gs_ref.so`` by ``oracle/build_ref.py`` and run on the
same GPU.  Deterministic stages must agree bit for bit; the samplers are compared statistically
(the reference draws from cuRAND with a constant seed, this library from its own counter-based
streams).  Skipped when the file has not been built."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref

    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref/gs_ref.so not built (python oracle/build_ref.py needs the reference tree)")
    return mod


def cuda(a, dtype=torch.int64):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def graph():
    rng = np.random.default_rng(5)
    n = 20000
    deg = rng.poisson(14, n)
    deg[rng.integers(0, n, 40)] = rng.integers(300, 2500, 40)
    deg[rng.integers(0, n, n // 20)] = 0
    deg[rng.integers(0, n, 30)] = 50
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg] +
                             [np.empty(0, np.int64)]).astype(np.int64)
    return indptr, indices


def new_graph(gsb, indptr, indices, seed=7777):
    n = indptr.size - 1
    g = gsb.Graph(n, n)
    g._CAPI_LoadCSC(cuda(indptr), cuda(indices))
    g._CAPI_SetSeed(seed)
    return g


def test_column_slicing_equals_reference(gsb, ref, graph):
    indptr, indices = graph
    rng = np.random.default_rng(1)
    seeds = cuda(rng.integers(0, indptr.size - 1, 3000))
    r_indptr, r_col, r_rows, r_sel = ref.slice_cols(cuda(indptr), cuda(indices), seeds, True)
    sub, sel = new_graph(gsb, indptr, indices)._CAPI_Slicing(seeds, 1, gsb._CSC, gsb._CSC + gsb._COO)
    assert torch.equal(sub._CAPI_GetCSCIndptr(), r_indptr)
    assert torch.equal(sub._CAPI_GetCSCIndices(), r_rows)
    assert torch.equal(sub._CAPI_GetCOOCols(), r_col)
    assert torch.equal(sel, r_sel)
    # super-batch form, no encoding
    ptr = cuda(np.array([0, 700, 700, 1900, 3000]))
    b_indptr, b_col, b_rows, b_sel, b_eptr = ref.batch_slice_cols(cuda(indptr), cuda(indices), seeds, ptr,
                                                                  True, False, 0)
    sub, sel = new_graph(gsb, indptr, indices)._CAPI_BatchColSlicing(seeds, ptr, False)
    assert torch.equal(sub._CAPI_GetCSCIndptr(), b_indptr)
    assert torch.equal(sub._CAPI_GetCSCIndices(), b_rows)
    assert torch.equal(sel, b_sel)
    assert torch.equal(sub._CAPI_GetEdgeBptr(), b_eptr)


def test_new_sampler_through_reference_relabel(gsb, ref, graph):
    """The edge set drawn by this library's sampler, relabelled by the reference's
    BatchCOORelabelCUDA, reproduces this library's node lists and relabelled COO bit for bit,
    layer after layer."""
    indptr, indices = graph
    rng = np.random.default_rng(2)
    seeds = cuda(rng.permutation(indptr.size - 1)[:6 * 400])
    ptr = cuda(np.arange(7) * 400)
    out = new_graph(gsb, indptr, indices, seed=99)._CAPI_BatchGraphSAGE(seeds, ptr, [10, 5, 3])
    cur_seeds, cur_ptr = seeds, ptr
    for l in range(3):
        sub, rows, cols, sel, eptr, uq, up, brow, bcol = out[9 * l:9 * l + 9]
        r_uq, r_up, r_row, r_col, r_eptr = ref.batch_coo_relabel(cur_seeds, cur_ptr, cur_seeds[cols], rows, eptr)
        assert torch.equal(r_uq, uq) and torch.equal(r_up, up)
        assert torch.equal(r_row, brow) and torch.equal(r_col, bcol)
        cur_seeds, cur_ptr = uq, up


def test_unique_and_relabel_equal_reference(gsb, ref, graph):
    indptr, indices = graph
    rng = np.random.default_rng(3)
    A = new_graph(gsb, indptr, indices)
    seeds = cuda(rng.integers(0, indptr.size - 1, 1500))          # with repeats
    sub, _ = A._CAPI_SlicingSampling(1, seeds, 8, False, gsb._CSC, gsb._COO)
    rows, cols = sub._CAPI_GetCOORows(), sub._CAPI_GetCOOCols()
    no_map = torch.empty(0, dtype=torch.int64, device="cuda")      # row ids are graph ids already
    want = ref.tensor_unique(torch.cat([seeds, rows]))
    assert torch.equal(sub._CAPI_GetValidNodes(seeds, no_map), want)
    r_uq, (r_col, r_row) = ref.tensor_relabel([seeds, rows], [seeds[cols], rows])
    uq, new_row, new_col, _ = sub._CAPI_GraphRelabel(seeds, no_map)
    assert torch.equal(uq, r_uq) and torch.equal(new_row, r_row) and torch.equal(new_col, r_col)


def test_sampler_against_reference_sampler(gsb, ref, graph):
    """Invariants of both samplers, exact agreement where nothing is random (degree <= fanout),
    and a chi-square two-sample test of the per-edge inclusion counts at p > 0.01."""
    from scipy import stats

    indptr, indices = graph
    n = indptr.size - 1
    deg = np.diff(indptr)
    K = 6
    # (1) copy-all branch: identical output
    small = np.flatnonzero(deg <= K)[:2000]
    r_indptr, r_col, r_rows, r_sel = ref.fused_slice_sample(cuda(indptr), cuda(indices), K, cuda(small), False, True)
    sub, sel = new_graph(gsb, indptr, indices)._CAPI_SlicingSampling(1, cuda(small), K, False, gsb._CSC,
                                                                     gsb._CSC + gsb._COO)
    assert torch.equal(sub._CAPI_GetCSCIndptr(), r_indptr) and torch.equal(sub._CAPI_GetCSCIndices(), r_rows)
    assert torch.equal(sel, r_sel)
    # (2) one column of degree 40..60 sampled many times in a single call of each sampler.  The
    # reference seeds cuRAND per block and per lane only (curand_init(seed * grid + blockIdx.x,
    # threadIdx.x), fusion/slice_sampling.cu:50-51), so the 32 rows of a block repeat each other:
    # one row per block is an independent draw.
    v = int(np.flatnonzero((deg >= 40) & (deg <= 60))[0])
    rows_per_block, draws = 32, 20000
    reps = rows_per_block * draws
    many = cuda(np.full(reps, v))
    counts = []
    for name in ("reference", "ours"):
        if name == "reference":
            ip, _, rows, sel = ref.fused_slice_sample(cuda(indptr), cuda(indices), K, many, False, True)
        else:
            sub, sel = new_graph(gsb, indptr, indices, seed=2024)._CAPI_SlicingSampling(
                1, many, K, False, gsb._CSC, gsb._CSC + gsb._COO)
            ip, rows = sub._CAPI_GetCSCIndptr(), sub._CAPI_GetCSCIndices()
        ip, rows, sel = host(ip), host(rows), host(sel)
        assert np.array_equal(np.diff(ip), np.full(reps, K))                   # min(deg, K) per column
        assert np.all((sel >= indptr[v]) & (sel < indptr[v + 1]))              # edges of the slice
        assert np.array_equal(indices[sel], rows)
        per_col = np.sort(sel.reshape(reps, K), axis=1)
        assert np.all(per_col[:, 1:] != per_col[:, :-1])                       # no duplicates
        independent = sel.reshape(reps, K)[::rows_per_block]
        counts.append(np.bincount(independent.ravel() - indptr[v], minlength=deg[v]))
    exact = [stats.chisquare(c, np.full(deg[v], draws * K / deg[v])).pvalue for c in counts]
    chi2, p, _, _ = stats.chi2_contingency(np.stack(counts))
    assert p > 0.01, (chi2, p, exact)
    assert min(exact) > 0.001, exact       # each also against the exact inclusion probability K / deg


def test_fused_col_row_slicing_equals_reference(gsb, ref, graph):
    indptr, indices = graph
    n = indptr.size - 1
    rng = np.random.default_rng(6)
    ncol, nrow = np.array([300, 150, 500]), np.array([2000, 6000, 900])
    cols = cuda(np.concatenate([rng.integers(0, n, k) for k in ncol]))
    rows = cuda(np.concatenate([rng.permutation(n)[:k] for k in nrow]))
    col_ptr = cuda(np.concatenate([[0], np.cumsum(ncol)]))
    row_ptr = cuda(np.concatenate([[0], np.cumsum(nrow)]))
    r_indptr, r_ids, r_sel = ref.batch_col_row_slicing(cuda(indptr), cuda(indices), cols, col_ptr, rows,
                                                       row_ptr, n)
    sub, sel = new_graph(gsb, indptr, indices)._CAPI_BatchColRowSlcing(cols, col_ptr, rows, row_ptr)
    assert torch.equal(sub._CAPI_GetCSCIndptr(), r_indptr)
    assert torch.equal(sub._CAPI_GetCSCIndices(), r_ids)
    # the reference's index counts positions in the column slice; this library's counts
    # positions in the operand -- the two meet through the column slice's own index
    _, _, _, slice_sel = ref.slice_cols(cuda(indptr), cuda(indices), cols, True)
    assert torch.equal(sel, slice_sel[r_sel])


def test_walks_against_reference(gsb, ref, graph):
    """First-step distribution of both walkers from one start node (two-sample chi-square), and
    the trace invariant the reference's own tests check: every step follows an edge."""
    from scipy import stats

    indptr, indices = graph
    deg = np.diff(indptr)
    v = int(np.flatnonzero((deg >= 20) & (deg <= 30))[0])
    reps, L = 20000, 4
    start = cuda(np.full(reps, v))
    A = new_graph(gsb, indptr, indices, seed=5)
    traces = {"reference": host(ref.random_walk(start, L, cuda(indices), cuda(indptr))).reshape(L + 1, reps),
              "ours": host(A._CAPI_RandomWalk(start, L)).reshape(L + 1, reps)}
    firsts = []
    for name, tr in traces.items():
        assert np.all(tr[0] == v)
        for s in range(L):
            a, b = tr[s], tr[s + 1]
            live = a >= 0
            assert np.all(b[~live] == -1)
            ok = [(b[i] == -1 and deg[a[i]] == 0) or b[i] in indices[indptr[a[i]]:indptr[a[i] + 1]]
                  for i in np.flatnonzero(live)[:400]]
            assert all(ok), name
        firsts.append(np.bincount(np.searchsorted(indices[indptr[v]:indptr[v + 1]], tr[1]), minlength=deg[v]))
    assert stats.chi2_contingency(np.stack(firsts))[1] > 0.01


def test_spmm_sddmm_against_reference_kernels(gsb, ref, graph):
    """fp32 edge-probability kernels (SpMM sums over rows / columns, SDDMM edge maps, multi-head
    dot) within 1e-5 relative of the reference's SpMMCSC / SpMMCOO / SDDMMCOO on the same graph."""
    indptr, indices = graph
    n, E = indptr.size - 1, indices.size
    rng = np.random.default_rng(9)
    tol = dict(rtol=1e-5, atol=1e-6)
    w = cuda(rng.random(E) + 0.01, torch.float32)
    ip, ix = cuda(indptr), cuda(indices)
    col = torch.repeat_interleave(torch.arange(n, device="cuda"), ip[1:] - ip[:-1])
    dummy = torch.zeros(1, 1, device="cuda")
    aux = lambda shape: torch.zeros(shape, dtype=torch.int64, device="cuda")  # noqa: E731
    A = new_graph(gsb, indptr, indices)
    m = gsb.Matrix(A)
    m.edata["w"] = w
    # column sums on the CSC, row sums on the COO (atomics in both implementations)
    out = torch.zeros(n, 1, device="cuda")
    ref.spmm_csc("copy_rhs", "sum", ip, ix, dummy, w[:, None], out, aux((n, 1)), aux((n, 1)))
    assert np.allclose(host(m.sum("w", axis=0)), host(out)[:, 0], **tol)
    out = torch.zeros(n, 1, device="cuda")
    ref.spmm_coo("copy_rhs", "sum", ix, col, dummy, w[:, None], out, 2, aux((n, 1)), aux((n, 1)))
    # atomics in both implementations, so the order of the additions differs: each side is held
    # to the fp64 sum of the same fp32 terms -- 1e-5 relative, and for rows long enough that
    # rounding alone can exceed it the statistical bound 4 * sqrt(terms) * 2^-24
    want64 = np.bincount(indices, weights=host(w).astype(np.float64), minlength=n)
    terms = np.bincount(indices, minlength=n)
    bound = np.maximum(1e-5, 4 * np.sqrt(terms) * 2.0 ** -24) * want64 + 1e-7
    assert np.all(np.abs(host(m.sum("w", axis=1)).astype(np.float64) - want64) <= bound)
    assert np.all(np.abs(host(out)[:, 0].astype(np.float64) - want64) <= bound)
    # vector features, broadcast, max reducer
    u = cuda(rng.random((n, 4)), torch.float32)
    e = cuda(rng.random((E, 1)), torch.float32)
    out = torch.zeros(n, 4, device="cuda")
    ref.spmm_csc("mul", "max", ip, ix, u, e, out, aux((n, 4)), aux((n, 4)))
    got = gsb.ops.gspmm(m, "mul", "max", u, e, 0, gsb._CSC)
    deg = host(ip[1:] - ip[:-1])
    assert np.allclose(host(got)[deg > 0], host(out)[deg > 0], **tol)
    # SDDMM: e * node on either endpoint, u + v on vectors, multi-head dot
    node = cuda(rng.random((n, 1)) + 0.5, torch.float32)
    for target, name in ((0, "u"), (2, "v")):
        out = torch.zeros(E, 1, device="cuda")
        ref.sddmm_coo("mul", ix, col, w[:, None], node, out, 1, target)
        got = gsb.ops.gsddmm(m, "mul", w, node[:, 0].contiguous(), "e", name)
        assert np.allclose(host(got), host(out)[:, 0], **tol)
    out = torch.zeros(E, 4, device="cuda")
    ref.sddmm_coo("add", ix, col, u, u, out, 0, 2)
    assert np.allclose(host(gsb.ops.gsddmm(m, "add", u, u, "u", "v")), host(out), **tol)
    h = cuda(rng.random((n, 3, 8)), torch.float32)
    out = torch.zeros(E, 3, 1, device="cuda")
    ref.sddmm_coo("dot", ix, col, h, h, out, 0, 2)
    assert np.allclose(host(gsb.ops.gsddmm(m, "dot", h, h, "u", "v")), host(out), rtol=1e-5, atol=1e-5)


def test_weighted_samplers_against_reference(gsb, ref):
    """Per-column weighted sampling without replacement and the segmented (batch) list sampler:
    both sides implement A-Res (largest u^(1/w) keys).  Per-column sampling: the per-item
    inclusion counts of 20 000 independent draws agree (chi-square two-sample, p > 0.01).  List
    sampling: see the note at the end.  Zero-weight items never win on either side."""
    from scipy import stats

    rng = np.random.default_rng(10)
    deg, K, reps = 40, 5, 20000
    wts = (rng.random(deg) + 0.05).astype(np.float32)
    wts[[3, 17]] = 0.0
    # a CSC whose `reps` columns are copies of one weighted column
    indptr = cuda(np.arange(reps + 1) * deg)
    indices = cuda(np.tile(np.arange(deg), reps))
    probs = cuda(np.tile(wts, reps), torch.float32)
    r_ip, _, r_rows, r_sel = ref.sample_cols_probs(indptr, indices, probs, K, False, True)
    g = gsb.Graph(deg, reps)
    g._CAPI_LoadCSC(indptr, indices)
    g._CAPI_SetSeed(31)
    sub, sel = g._CAPI_SamplingProbs(1, probs, K, False, gsb._CSC, gsb._CSC)
    counts = []
    for ip, rows in ((r_ip, r_rows), (sub._CAPI_GetCSCIndptr(), sub._CAPI_GetCSCIndices())):
        assert np.array_equal(np.diff(host(ip)), np.full(reps, K))
        picks = host(rows).reshape(reps, K)
        s = np.sort(picks, axis=1)
        assert np.all(s[:, 1:] != s[:, :-1])
        c = np.bincount(picks.ravel(), minlength=deg)
        assert c[3] == 0 and c[17] == 0
        counts.append(c)
    keep = wts > 0
    assert stats.chi2_contingency(np.stack(counts)[:, keep])[1] > 0.01
    # segmented list sampling: `reps` segments with the same weights
    rng_ptr = cuda(np.arange(reps + 1) * deg)
    r_idx, r_out_ptr = ref.batch_list_sampling_probs(probs, K, False, rng_ptr)
    torch.ops.gs_ops._CAPI_SetListSamplingSeed(77)
    o_idx, o_out_ptr = torch.ops.gs_ops._CAPI_BatchListSamplingWithProbs(probs, K, False, rng_ptr)
    counts = []
    for idx, optr in ((r_idx, r_out_ptr), (o_idx, o_out_ptr)):
        assert np.array_equal(host(optr), np.arange(reps + 1) * K)
        local = host(idx).reshape(reps, K) - (np.arange(reps) * deg)[:, None]
        assert local.min() >= 0 and local.max() < deg
        s = np.sort(local, axis=1)
        assert np.all(s[:, 1:] != s[:, :-1])
        c = np.bincount(local.ravel(), minlength=deg)
        assert c[3] == 0 and c[17] == 0
        counts.append(c)
    # A-Res inclusion probabilities by Monte Carlo on the host (2 M draws): tells which side is
    # off if the two-sample test fails
    mc = np.zeros(deg)
    g2 = np.random.default_rng(123)
    for _ in range(20):
        keys = np.where(wts > 0, g2.random((100000, deg)) ** (1.0 / np.maximum(wts, 1e-30)), -1.0)
        mc += np.bincount(np.argpartition(-keys, K - 1, axis=1)[:, :K].ravel(), minlength=deg)
    expect = mc[keep] / mc[keep].sum() * reps * K
    fit = [stats.chisquare(c[keep], expect).pvalue for c in counts]
    # The reference seeds one XORWOW generator per item with item_index * 7777 and uses its first
    # output (batch/list_sampling_probs.cu:73-80); those first outputs are correlated enough that
    # the reference itself misses the exact A-Res frequencies (measured p ~ 1e-12 here), so an
    # exact two-sample agreement cannot be asked for.  Required: this library fits the exact
    # frequencies, and the two samplers' inclusion frequencies are within 0.02 in total variation.
    assert fit[1] > 0.01, fit
    f_ref, f_ours = counts[0][keep] / counts[0].sum(), counts[1][keep] / counts[1].sum()
    tv = 0.5 * np.abs(f_ref - f_ours).sum()      # total variation distance of the two frequency vectors
    assert tv < 0.02, (fit, tv)


@pytest.mark.parametrize("p,q", [(2.0, 0.5), (0.25, 4.0)])
def test_node2vec_second_order_bias_against_reference(gsb, ref, p, q):
    """The p/q bias of the second step (src/cuda/fusion/node2vec.cu:99-127): 20 000 walkers start
    at one node v, so the step-2 candidate is judged against previous node v -- a return to v,
    a neighbour of v, or neither.  The three class counts (overall and per intermediate node)
    of this library and of the reference's FusedNode2VecCUDA agree (chi-square two-sample,
    p > 0.01) and show the bias the parameters ask for."""
    from scipy import stats

    rng = np.random.default_rng(12)
    n, reps = 300, 20000
    adj = rng.random((n, n)) < 0.06
    adj = np.triu(adj, 1)
    adj = adj | adj.T                                       # symmetric, no self-loops: triangles exist
    # The reference starts every walker's "previous node" at its thread index and looks that index
    # up in the offsets (node2vec.cu:88,113 -> CheckConnect :46-64) without a bound: with more
    # walkers than nodes it reads past the end of the arrays (an illegal access was seen on the
    # GPU with 20 000 walkers on the 300-node graph alone).  So the graph gets one node per walker,
    # the extra ones on a ring so that every node has neighbours and every lookup stays in bounds.
    N = reps + 1000
    cols = [np.flatnonzero(adj[:, c]) for c in range(n)]
    for c in range(n, N):
        cols.append(np.array(sorted({n + (c - n - 1) % (N - n), n + (c - n + 1) % (N - n)})))
    deg = np.array([c.size for c in cols])
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate(cols).astype(np.int64)         # sorted columns
    v = int(np.argmax(deg[:n]))
    start = cuda(np.full(reps, v))
    ours = host(new_graph(gsb, indptr, indices, seed=41)._CAPI_Node2Vec(start, 2, p, q)).reshape(3, reps)
    theirs = host(ref.node2vec(start, 2, cuda(indices), cuda(indptr), p, q)).reshape(3, reps)
    nbr_v = np.zeros(N, bool)
    nbr_v[:n] = adj[:, v]
    tables = []
    for tr in (ours, theirs):
        assert np.all(tr[0] == v) and np.all(tr[1] < n) and np.all(adj[tr[1], v])   # step 1 follows an edge into v's list
        assert np.all(tr[2] < n) and np.all(adj[tr[2], tr[1]])                      # and so does step 2
        cls = np.where(tr[2] == v, 0, np.where(nbr_v[tr[2]], 1, 2))    # return / neighbour of v / other
        tables.append(np.bincount(cls, minlength=3))
    chi2, pval, _, _ = stats.chi2_contingency(np.stack(tables))
    assert pval > 0.01, (tables, pval)
    # first step: uniform over v's list on both sides
    firsts = np.stack([np.bincount(np.searchsorted(indices[indptr[v]:indptr[v + 1]], tr[1]), minlength=deg[v])
                       for tr in (ours, theirs)])
    assert stats.chi2_contingency(firsts)[1] > 0.01
    # both against the exact class probabilities of the rule (node2vec.cu:99-127): y is uniform on
    # {0 .. max(p,q)-1} (integer max here), a candidate is accepted iff y < min(p,q,1) or y < h
    # with h = p for a return, q for a neighbour of the previous node, 1 otherwise
    ms = int(max(p, q))
    accept = {k: np.ceil(min(max(h, min(p, q, 1.0)), ms)) / ms for k, h in ((0, p), (1, q), (2, 1.0))}
    expect = np.zeros(3)
    for c in indices[indptr[v]:indptr[v + 1]]:
        cand = indices[indptr[c]:indptr[c + 1]]
        if cand.size == 1:
            w = np.ones(1)
        else:
            w = np.array([accept[0 if x == v else (1 if nbr_v[x] else 2)] for x in cand])
        cls = np.where(cand == v, 0, np.where(nbr_v[cand], 1, 2))
        expect += np.bincount(cls, weights=w / w.sum(), minlength=3) / deg[v]
    for t in tables:
        assert stats.chisquare(t, expect * reps).pvalue > 0.001, (t, expect * reps)


def test_sampler_chi_square_grid_against_reference_sampler(gsb, ref):
    """The configurations' fanouts against the reference's FusedCSCColSlicingSamplingCUDA
    (src/cuda/fusion/slice_sampling.cu:43-96) and the exact inclusion probability K / deg: K in
    {5, 10, 15, 25} x degree in {K+1, 2K, 50, 500}.  Degree K+1 is where Floyd's "replace by j"
    branch and the reference's reservoir differ most."""
    from scipy import stats

    Ks = (5, 10, 15, 25)
    degs = sorted({d for K in Ks for d in (K + 1, 2 * K, 50, 500)})
    indptr = np.concatenate([[0], np.cumsum(degs)]).astype(np.int64)
    indices = np.concatenate([np.arange(d) for d in degs]).astype(np.int64)
    d_ip, d_ix = cuda(indptr), cuda(indices)
    rows_per_block, draws = 32, 12000       # the reference repeats one draw over the 32 rows of a block
    reps = rows_per_block * draws
    worst = 1.0
    for K in Ks:
        for d in (K + 1, 2 * K, 50, 500):
            c = degs.index(d)
            many = cuda(np.full(reps, c))
            _, _, r_rows, r_sel = ref.fused_slice_sample(d_ip, d_ix, K, many, False, True)
            sub, o_sel = new_graph(gsb, indptr, indices, seed=1000 + 31 * K + d)._CAPI_SlicingSampling(
                1, many, K, False, gsb._CSC, gsb._CSC + gsb._COO)
            counts = []
            for sel, stride in ((host(r_sel), rows_per_block), (host(o_sel), 1)):
                assert sel.size == reps * K
                per_col = sel.reshape(reps, K) - indptr[c]
                assert per_col.min() >= 0 and per_col.max() < d
                s = np.sort(per_col, axis=1)
                assert np.all(s[:, 1:] != s[:, :-1])                   # K distinct edges per column
                counts.append(np.bincount(per_col[::stride].ravel(), minlength=d).astype(float))
            p_inc = K / d
            for cnt in counts:                                          # each against the exact K / deg
                m = cnt.sum() / K
                chi2 = ((cnt - m * p_inc) ** 2 / (m * p_inc * (1 - p_inc))).sum() * (d - 1) / d
                pv = stats.chi2.sf(chi2, d - 1)
                worst = min(worst, pv)
                assert pv > 0.001, (K, d, pv)
            pv = stats.chi2_contingency(np.stack(counts))[1]           # and against each other
            assert pv > 0.01 / 4, (K, d, pv)   # 16 cells: a per-cell bound of 0.0025 keeps the family near 0.04
    assert worst > 1e-4


def test_benchmark_size_super_batch_through_reference_relabel(gsb, ref):
    """One super-batch of the benchmark's shape (32 x 1024 seeds, fanouts [15, 10, 5], the
    2.45 M-node / 123.7 M-edge power-law graph; 23 M relabel items in the last layer): every
    layer's sampled edges through the reference's BatchCOORelabelCUDA
    (src/cuda/batch/batch_relabel.cu:376-499) reproduce this library's node lists, offsets and
    relabelled COO bit for bit; the sampling invariants hold at that size."""
    from gsampler_b200 import synth

    n, nnz = 2449029, 123718280
    indptr, indices = synth.powerlaw_csc(n, nnz, exponent=2.1, max_degree=20000, seed=2024, device="cuda")
    g = torch.Generator()
    g.manual_seed(7)
    seeds = torch.randperm(n, generator=g)[:32 * 1024].cuda()
    ptr = (torch.arange(33) * 1024).cuda()
    A = gsb.Graph(n, n)
    A._CAPI_LoadCSC(indptr, indices)
    A._CAPI_SetSeed(5)
    fanouts = [15, 10, 5]
    out = A._CAPI_BatchGraphSAGE(seeds, ptr, fanouts)
    cur_seeds, cur_ptr = seeds, ptr
    for l, K in enumerate(fanouts):
        sub, rows, cols, sel, eptr, uq, up, brow, bcol = out[9 * l:9 * l + 9]
        deg = indptr[cur_seeds + 1] - indptr[cur_seeds]
        assert torch.equal(sub[1:] - sub[:-1], deg.clamp_max(K))           # min(deg, K) per column
        assert torch.equal(indices[sel], rows)                              # every edge exists ...
        col_g = cur_seeds[cols]
        assert bool(((sel >= indptr[col_g]) & (sel < indptr[col_g + 1])).all())   # ... in its column
        key = cols * nnz + sel
        assert bool((key[1:] != key[:-1]).all()) and bool((cols[1:] >= cols[:-1]).all())
        assert torch.unique(key).numel() == key.numel()                     # no duplicate edge in a column
        assert torch.equal(eptr, sub[cur_ptr])
        r_uq, r_up, r_row, r_col, r_eptr = ref.batch_coo_relabel(cur_seeds, cur_ptr, col_g, rows, eptr)
        assert torch.equal(r_up, up) and torch.equal(r_uq, uq)
        assert torch.equal(r_row, brow) and torch.equal(r_col, bcol)
        cur_seeds, cur_ptr = uq, up
    assert rows.numel() > 15_000_000      # the last layer really has the benchmark's size
    del out, indptr, indices
    torch.cuda.empty_cache()


def test_one_large_minibatch_relabel_equals_reference(gsb, ref):
    """Unique / relabel of ONE minibatch of 6.5 M items (a whole layer relabelled at once, as the
    non-batch samplers do): more buckets than the scatter pass's shared histogram holds, so its
    per-item atomic path runs; a few ids repeated tens of thousands of times fill their buckets'
    regions and go through the overflow list.  Bit-exact against the reference's
    TensorUniqueCUDA / TensorRelabelCUDA (src/cuda/unique_reindex.cu:174-199)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(31)
    n = 3_000_000
    seeds = torch.randint(0, n, (1_500_000,), generator=g, device="cuda")
    rows = torch.randint(0, n, (5_000_000,), generator=g, device="cuda")
    hubs = torch.randint(0, n, (12,), generator=g, device="cuda")
    at = torch.randint(0, rows.numel(), (400_000,), generator=g, device="cuda")
    rows[at] = hubs[torch.randint(0, 12, (at.numel(),), generator=g, device="cuda")]
    cols = torch.sort(torch.randint(0, seeds.numel(), (rows.numel(),), generator=g, device="cuda")).values
    A = gsb.Graph(n, seeds.numel())
    A._CAPI_LoadCOO(rows, cols, False, True)
    no_map = torch.empty(0, dtype=torch.int64, device="cuda")
    assert torch.equal(A._CAPI_GetValidNodes(seeds, no_map), ref.tensor_unique(torch.cat([seeds, rows])))
    r_uq, (r_col, r_row) = ref.tensor_relabel([seeds, rows], [seeds[cols], rows])
    uq, new_row, new_col, _ = A._CAPI_GraphRelabel(seeds, no_map)
    assert torch.equal(uq, r_uq) and torch.equal(new_row, r_row) and torch.equal(new_col, r_col)


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_sort_columns_equals_reference_and_oracle(gsb, ref, oracle, idx_dtype):
    """Per-column sort (Graph::SortCSCIndices): bit-exact against the reference's SortIndicesCUDA
    (src/cuda/sort_indices.cu:11-37, a CUB segmented radix sort; int64 only) and against the
    restated SortIndicesCPU, over every kernel path: empty and one-entry columns, columns of up
    to 256 entries (warp), up to 4096 (CTA), longer ones (range partition), a long column whose
    ids crowd into a narrow range (the in-place network), and duplicate ids."""
    rng = np.random.default_rng(21)
    n = 60000
    degs = np.concatenate([rng.integers(0, 80, 3000), [0, 1, 2, 255, 256, 257, 4095, 4096, 4097, 20000, 70000, 9000],
                           rng.integers(200, 3000, 40)])
    indptr = np.concatenate([[0], np.cumsum(degs)]).astype(np.int64)
    indices = rng.integers(0, n, indptr[-1]).astype(np.int64)
    crowded = int(np.flatnonzero(degs == 9000)[0])
    indices[indptr[crowded]:indptr[crowded + 1]] = rng.integers(500, 520, 9000)       # 20 distinct values
    indices[indptr[crowded]] = n - 1                                                 # ... and one far away
    g = gsb.Graph(n, degs.size)
    g._CAPI_LoadCSC(cuda(indptr), cuda(indices, idx_dtype))
    g._CAPI_SortCSCIndices()
    got = host(g._CAPI_GetCSCIndices()).astype(np.int64)
    assert np.array_equal(got, oracle.sort_indices(indptr, indices))
    assert np.array_equal(got, host(ref.sort_indices(cuda(indptr), cuda(indices))))
    assert g._CAPI_GetCSCIndices().dtype == idx_dtype


def test_fused_edge_operators_against_reference_kernels(gsb, ref, graph):
    """The fused edge operators of the PASS / AS-GCN / LADIES samplers against the reference's own
    fused kernels: two u-op-v maps in one pass (FUSED_COO_U_OP_V, FUSED_CSC_U_OP_V), sum of e^2
    and sum of e / u per node (ESquareSum*, EDivUSum*); 1e-5 relative."""
    indptr, indices = graph
    n, E = indptr.size - 1, indices.size
    rng = np.random.default_rng(14)
    ip, ix = cuda(indptr), cuda(indices)
    col = torch.repeat_interleave(torch.arange(n, device="cuda"), ip[1:] - ip[:-1])
    A = new_graph(gsb, indptr, indices)
    tol = dict(rtol=1e-5, atol=1e-6)
    for shape in ((n, 1), (n, 6)):
        u1, v1, u2, v2 = (cuda(rng.random(shape) + 0.5, torch.float32) for _ in range(4))
        for op in ("mul", "add", "div", "sub"):
            want1, want2 = (torch.zeros(E, shape[1], device="cuda") for _ in range(2))
            ref.fused_u_op_v_coo(op, ix, col, u1, v1, want1, u2, v2, want2)
            for fmt in (gsb._COO, gsb._CSC):
                got1, got2 = (torch.full((E, shape[1]), -1.0, device="cuda") for _ in range(2))
                A._CAPI_FusedUOPV(op, u1, v1, got1, u2, v2, got2, fmt)
                assert np.allclose(host(got1), host(want1), **tol) and np.allclose(host(got2), host(want2), **tol)
        wc1, wc2 = (torch.zeros(E, shape[1], device="cuda") for _ in range(2))
        ref.fused_u_op_v_csc("mul", ip, ix, u1, v1, wc1, u2, v2, wc2)
        g1, g2 = (torch.zeros(E, shape[1], device="cuda") for _ in range(2))
        A._CAPI_FusedUOPV("mul", u1, v1, g1, u2, v2, g2, gsb._CSC)
        assert np.allclose(host(g1), host(wc1), **tol) and np.allclose(host(g2), host(wc2), **tol)
    # fused reductions (scalar edge weights, the samplers' case)
    w = cuda(rng.random((E, 1)) + 0.05, torch.float32)
    node = cuda(rng.random((n, 1)) + 0.5, torch.float32)
    aux = lambda: torch.zeros(n, 1, dtype=torch.int64, device="cuda")  # noqa: E731
    dummy = torch.zeros(1, 1, device="cuda")
    # sums of positive fp32 terms in different orders: each side is held to the fp64 sum of the
    # same terms (1e-5 relative; 4 * sqrt(terms) * 2^-24 where rounding alone can exceed that)
    terms = np.diff(indptr)
    bound = np.maximum(1e-5, 4 * np.sqrt(terms) * 2.0 ** -24)
    col_h, w64, node64 = host(col), host(w)[:, 0].astype(np.float64), host(node)[:, 0].astype(np.float64)
    cases = (("e_square_sum_csc", "copy_rhs", dummy, "_CAPI_FusedESquareSum", None,
              np.bincount(col_h, weights=w64 ** 2, minlength=n)),
             ("e_div_u_sum_csc", "div", node, "_CAPI_FusedEDivUSum", node,
              np.bincount(col_h, weights=w64 / node64[indices], minlength=n)))
    for ref_name, op, ref_u, our_name, our_u, want64 in cases:
        theirs = torch.zeros(n, 1, device="cuda")
        getattr(ref, ref_name)(op, "sum", ip, ix, ref_u, w, theirs, aux(), aux())
        ours = torch.zeros(n, 1, device="cuda")
        getattr(A, our_name)(op, "sum", our_u, w, ours, None, None, 0, gsb._CSC)
        for side in (ours, theirs):
            assert np.all(np.abs(host(side)[:, 0].astype(np.float64) - want64) <= bound * want64 + 1e-7), ref_name
