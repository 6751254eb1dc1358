"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle on
the same seeded inputs.  Deterministic stages and the counter-based sampler are compared bit
for bit; the sampler is additionally compared statistically with the reference's reservoir
sampler (oracle.sample_ref)."""
import numpy as np
import pytest
import torch

from tests import abi

pytestmark = pytest.mark.gpu


def dev(a, dtype=torch.int64):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).cuda()


def host(t):
    return t.cpu().numpy()


def rand_csc(rng, n, avg, heavy=0):
    deg = rng.poisson(avg, n)
    deg[rng.integers(0, n, max(n // 10, 1))] = 0
    if heavy:
        deg[rng.integers(0, n, heavy)] = rng.integers(200, 3000, heavy)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n, indptr[-1]).astype(np.int64)
    return indptr, indices


@pytest.fixture(scope="module")
def graph():
    rng = np.random.default_rng(11)
    return rand_csc(rng, 5000, 14, heavy=20)


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
@pytest.mark.parametrize("K,replace", [(1, False), (5, False), (15, False), (25, False), (40, False),
                                       (4, True), (33, True)])
def test_fused_sampling_bit_exact(oracle, graph, idx_dtype, K, replace):
    indptr, indices = graph
    rng = np.random.default_rng(K)
    seeds = rng.integers(0, indptr.size - 1, 3000)            # with duplicates
    sub, rows, cols, sel, err = abi.sample_cols(dev(indptr), dev(indices, idx_dtype), dev(seeds), K,
                                                replace, seed=1234, stream=3)
    assert err == 0
    esub, erows, ecols, esel = oracle.sample_spec(indptr, indices, seeds, K, replace, 1234, 3)
    assert np.array_equal(host(sub), esub)
    assert np.array_equal(host(sel), esel)
    assert np.array_equal(host(rows), erows)
    assert np.array_equal(host(cols), ecols)


def test_plain_sampling_and_edge_cases(oracle, graph):
    indptr, indices = graph
    d_ip, d_ix = dev(indptr), dev(indices)
    # seeds == None: every column of the operand
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, None, 7, False, 5, 0)
    esub, erows, ecols, esel = oracle.sample_spec(indptr, indices, None, 7, False, 5, 0)
    assert err == 0 and np.array_equal(host(sub), esub) and np.array_equal(host(sel), esel)
    # no seeds at all
    empty = torch.empty(0, dtype=torch.int64, device="cuda")
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, empty, 7, False, 5, 0)
    assert err == 0 and host(sub).tolist() == [0] and rows.numel() == 0
    # only empty columns
    zero_cols = np.flatnonzero(np.diff(indptr) == 0)[:50]
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, dev(zero_cols), 7, False, 5, 0)
    assert err == 0 and int(sub[-1]) == 0 and not host(sub).any()
    # device-side live count smaller than the launch bound
    seeds = np.arange(1000)
    live = torch.tensor([333], dtype=torch.int64, device="cuda")
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, dev(seeds), 6, False, 8, 1, d_S=live)
    esub, erows, _, esel = oracle.sample_spec(indptr, indices, seeds[:333], 6, False, 8, 1)
    assert err == 0 and np.array_equal(host(sub)[:334], esub) and np.array_equal(host(sel), esel)
    # capacity too small is reported, not overrun
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, dev(seeds), 6, False, 8, 1, E_cap=100)
    assert err & 8


def test_reference_fixture_through_abi(oracle):
    # tests/test_colwise_sampling.cc:7-23 and test_colwise_slicing.cc:7-21 of the reference
    indptr = np.arange(21) * 5
    indices = np.arange(100)
    sub, rows, cols, sel, err = abi.sample_cols(dev(indptr), dev(indices), None, 6, False, 7777, 0)
    assert host(sub).tolist() == indptr.tolist() and host(rows).tolist() == indices.tolist()
    for fan in (6, 4):
        sub, rows, cols, sel, err = abi.sample_cols(dev(indptr), dev(indices), None, fan, True, 7777, 0)
        assert host(sub).tolist() == (np.arange(21) * fan).tolist()
        assert rows.numel() == 20 * fan and host(rows).tolist() != indices.tolist()
        assert np.all(host(rows) // 5 == host(cols))
    sub, rows, cols, sel, err = abi.slice_cols(dev(indptr), dev(indices), dev(np.arange(3)))
    assert host(sub).tolist() == [0, 5, 10, 15] and host(rows).tolist() == list(range(15))


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_slicing_bit_exact(oracle, graph, idx_dtype):
    indptr, indices = graph
    rng = np.random.default_rng(3)
    seeds = rng.integers(0, indptr.size - 1, 2000)
    sub, rows, cols, sel, err = abi.slice_cols(dev(indptr), dev(indices, idx_dtype), dev(seeds))
    esub, erows, ecols, esel = oracle.slice_cols(indptr, indices, seeds)
    assert err == 0
    for a, b in ((sub, esub), (rows, erows), (cols, ecols), (sel, esel)):
        assert np.array_equal(host(a), b)
    bptr = np.array([0, 100, 100, 900, 2000])
    sub, rows, cols, sel, err = abi.slice_cols(dev(indptr), dev(indices, idx_dtype), dev(seeds),
                                               dev(bptr), 5000)
    _, erows, _, _ = oracle.slice_cols(indptr, indices, seeds, bptr, 5000)
    assert np.array_equal(host(rows), erows)


def _relabel_case(rng, B, max_seeds, max_edges, nid):
    ns = rng.integers(1, max_seeds, B)
    ne = rng.integers(0, max_edges, B)
    ns[B // 2] = 0
    ne[B // 2] = 0
    if B > 3:
        ne[1] = 0
    sp = np.concatenate([[0], np.cumsum(ns)])
    ep = np.concatenate([[0], np.cumsum(ne)])
    seeds = rng.integers(0, nid, sp[-1])
    rows = rng.integers(0, nid, ep[-1])
    col_local = np.concatenate([rng.integers(sp[b], sp[b + 1], ne[b]) if ns[b] else
                                np.empty(0, np.int64) for b in range(B)] + [np.empty(0, np.int64)])
    col_local = np.sort(col_local).astype(np.int64)   # column-sorted COO like the sampler emits
    return seeds, sp, rows, col_local, ep


@pytest.mark.parametrize("B,max_seeds,max_edges,nid", [(1, 50, 400, 100), (7, 300, 5000, 1000),
                                                        (32, 1200, 20000, 200000), (3, 5, 3, 10)])
def test_batch_relabel_bit_exact(oracle, B, max_seeds, max_edges, nid):
    rng = np.random.default_rng(B)
    seeds, sp, rows, col_local, ep = _relabel_case(rng, B, max_seeds, max_edges, nid)
    uq, up, orow, ocol, err = abi.batch_relabel(dev(seeds), dev(sp), dev(rows), dev(col_local), dev(ep))
    assert err == 0
    euq, eup, eorow, eocol = oracle.batch_coo_relabel(seeds, sp, seeds[col_local], rows, ep)
    assert np.array_equal(host(up), eup)
    assert np.array_equal(host(uq), euq)
    assert np.array_equal(host(orow), eorow)
    assert np.array_equal(host(ocol), eocol)
    # node lists only (all_nodes)
    uq2, up2, _, _, err = abi.batch_relabel(dev(seeds), dev(sp), dev(rows), None, dev(ep), want_edges=False)
    assert err == 0 and np.array_equal(host(uq2), euq) and np.array_equal(host(up2), eup)


def test_relabel_reports_bad_ids():
    seeds = dev([1, 2, 3])
    rows = dev([5, 2 ** 33, -4])
    uq, up, orow, ocol, err = abi.batch_relabel(seeds, dev([0, 3]), rows, dev([0, 1, 2]), dev([0, 3]))
    assert err & 16
    # a stated bound: ids at or above it are reported and relabelled to -1, the rest is exact
    rows = dev([5, 9, 2, 10, 7])
    uq, up, orow, ocol, err = abi.batch_relabel(seeds, dev([0, 3]), rows, dev([0, 0, 1, 2, 2]), dev([0, 5]),
                                                id_bound=10)
    assert err & 16
    assert host(uq).tolist() == [1, 2, 3, 5, 9, 7] and host(orow).tolist() == [3, 4, 1, -1, 5]
    assert host(ocol).tolist() == [0, 0, 1, 2, 2]


def _bucket_of(ids, nbk):
    """The relabel stage's bucket of an id (csrc/gsb_relabel.cu: hash32, then scaled to [0, nbk))."""
    k = np.asarray(ids, dtype=np.uint64) & np.uint64(0xFFFFFFFF)
    m = np.uint64(0xFFFFFFFF)
    k ^= k >> np.uint64(16); k = (k * np.uint64(0x85ebca6b)) & m
    k ^= k >> np.uint64(13); k = (k * np.uint64(0xc2b2ae35)) & m
    k ^= k >> np.uint64(16)
    return (k * np.uint64(nbk)) >> np.uint64(32)


def test_batch_relabel_ids_crowding_into_one_bucket(oracle):
    """Ids chosen so that all of them hash into ONE of the minibatch's three buckets: 10 300
    mostly distinct ids in a bucket whose region holds 4096 entries and whose shared table holds
    8192 -- the rest goes through the overflow list, and the CTA falls back to its table in global
    memory.  A second minibatch of ordinary ids follows."""
    rng = np.random.default_rng(77)
    pool = rng.integers(0, 2 ** 31 - 5, 200_000)
    crowd = pool[_bucket_of(pool, 3) == 0]
    assert crowd.size >= 11_000
    ns = np.array([100, 300]); ne = np.array([10_300, 5_000])       # 10 400 items -> 3 buckets
    sp = np.concatenate([[0], np.cumsum(ns)]); ep = np.concatenate([[0], np.cumsum(ne)])
    seeds = np.concatenate([crowd[:100], rng.integers(0, 50_000, 300)])
    rows = np.concatenate([rng.permutation(crowd[50:10_350]), rng.integers(0, 50_000, 5_000)])   # 10 300 distinct
    col_local = np.sort(np.concatenate([rng.integers(0, 100, 10_300), rng.integers(100, 400, 5_000)])).astype(np.int64)
    uq, up, orow, ocol, err = abi.batch_relabel(dev(seeds), dev(sp), dev(rows), dev(col_local), dev(ep))
    assert err == 0
    euq, eup, eorow, eocol = oracle.batch_coo_relabel(seeds, sp, seeds[col_local], rows, ep)
    assert np.array_equal(host(up), eup) and np.array_equal(host(uq), euq)
    assert np.array_equal(host(orow), eorow) and np.array_equal(host(ocol), eocol)
    assert eup[1] > 8192      # more distinct ids than the shared table has slots


@pytest.mark.parametrize("case", ["streamed_buckets", "table_overflow", "hub", "two_big"])
def test_batch_relabel_large_minibatches(oracle, case):
    """Minibatches far larger than a sampler produces: several thousand buckets per minibatch
    (more than the scatter pass's shared histogram holds: its per-item path), and one id
    repeated hundreds of thousands of times (overflow list)."""
    rng = np.random.default_rng(len(case))
    if case == "streamed_buckets":      # 1452 buckets, ids repeat about twice
        sizes, nid = [(1000, 5_200_000)], 3_000_000
    elif case == "table_overflow":      # 2665 buckets of mostly distinct ids
        sizes, nid = [(50_000, 9_500_000)], 2 ** 31 - 5
    elif case == "hub":
        sizes, nid = [(100, 400_000), (50, 30_000)], 50_000
    else:
        sizes, nid = [(20_000, 1_500_000), (0, 0), (30_000, 2_500_000)], 400_000
    ns = np.array([s for s, _ in sizes]); ne = np.array([e for _, e in sizes])
    sp = np.concatenate([[0], np.cumsum(ns)]); ep = np.concatenate([[0], np.cumsum(ne)])
    seeds = rng.integers(0, nid, sp[-1])
    rows = rng.integers(0, nid, ep[-1])
    if case == "hub":
        rows[rng.random(rows.size) < 0.9] = 4242
    col_local = np.sort(np.concatenate([rng.integers(sp[b], sp[b + 1], ne[b]) if ns[b] else
                                        np.empty(0, np.int64) for b in range(len(sizes))])).astype(np.int64)
    uq, up, orow, ocol, err = abi.batch_relabel(dev(seeds), dev(sp), dev(rows), dev(col_local), dev(ep))
    assert err == 0
    euq, eup, eorow, eocol = oracle.batch_coo_relabel(seeds, sp, seeds[col_local], rows, ep)
    assert np.array_equal(host(up), eup)
    assert np.array_equal(host(uq), euq)
    assert np.array_equal(host(orow), eorow)
    assert np.array_equal(host(ocol), eocol)


def test_sampler_statistics_vs_reference(oracle):
    """Per-edge inclusion frequencies of the CUDA sampler against (a) the exact value K/deg and
    (b) the reference's reservoir sampler, chi-square at p > 0.01."""
    from scipy import stats

    deg, K, S = 37, 10, 64000
    indptr = np.array([0, deg, deg + 3])
    indices = np.arange(deg + 3)
    seeds = np.zeros(S, np.int64)
    _, rows, cols, _, err = abi.sample_cols(dev(indptr), dev(indices), dev(seeds), K, False, 99, 0)
    assert err == 0
    rows, cols = host(rows), host(cols)
    for i in range(0, S, 997):                              # distinct picks per column
        assert np.unique(rows[cols == i]).size == K
    mine = np.bincount(rows, minlength=deg).astype(float)
    n = S
    # inclusion counts of a uniform K-subset: variance n*p*(1-p), covariance gives (deg-1) dof
    p = K / deg
    chi2 = ((mine - n * p) ** 2 / (n * p * (1 - p))).sum() * (deg - 1) / deg
    assert stats.chi2.sf(chi2, deg - 1) > 0.01
    _, rrows, rcols, _ = oracle.sample_ref(indptr, indices, seeds, K, False)
    keep = (rcols % 32) == 0            # the reference's 32 rows per block repeat one sample
    ref = np.bincount(rrows[keep], minlength=deg).astype(float)
    m = keep.sum() / K
    pooled = (mine + ref) / (n + m)
    chi2 = (((mine - n * pooled) ** 2) / (n * pooled * (1 - p)) +
            ((ref - m * pooled) ** 2) / (m * pooled * (1 - p))).sum() * (deg - 1) / deg
    assert stats.chi2.sf(chi2, deg - 1) > 0.01


def test_weighted_sampling_invariants_and_statistics(oracle, graph):
    from scipy import stats

    indptr, indices = graph
    rng = np.random.default_rng(8)
    probs = rng.random(indices.size).astype(np.float32) + 0.05
    seeds = rng.integers(0, indptr.size - 1, 1500)
    d_p = dev(probs, torch.float32)
    for K in (3, 20, 48):
        sub, rows, cols, sel, err = abi.sample_cols(dev(indptr), dev(indices), dev(seeds), K, False,
                                                    5, 0, probs=d_p)
        assert err == 0
        sub, rows, cols, sel = map(host, (sub, rows, cols, sel))
        degs = indptr[seeds + 1] - indptr[seeds]
        assert np.array_equal(np.diff(sub), np.minimum(degs, K))
        assert np.array_equal(rows, indices[sel])
        assert np.all((sel >= indptr[seeds[cols]]) & (sel < indptr[seeds[cols] + 1]))
        for i in range(0, seeds.size, 37):
            s = sel[sub[i]:sub[i + 1]]
            assert np.unique(s).size == s.size
    # one column, K = 1: inclusion probability of edge e must be p_e / sum(p)
    deg, S = 12, 40000
    w = np.array([1, 2, 3, 4, 5, 6, 1, 1, 2, 2, 8, 0.5], np.float32)
    ip = np.array([0, deg])
    _, rows, _, _, err = abi.sample_cols(dev(ip), dev(np.arange(deg)), dev(np.zeros(S, np.int64)), 1,
                                         False, 17, 0, probs=dev(w, torch.float32))
    cnt = np.bincount(host(rows), minlength=deg)
    assert stats.chisquare(cnt, S * w.astype(np.float64) / w.astype(np.float64).sum()).pvalue > 0.01
    # with replacement: K independent draws from the same distribution
    _, rows, _, _, err = abi.sample_cols(dev(ip), dev(np.arange(deg)), dev(np.zeros(4000, np.int64)),
                                         8, True, 21, 0, probs=dev(w, torch.float32))
    cnt = np.bincount(host(rows), minlength=deg)
    assert rows.numel() == 32000 and stats.chisquare(cnt, 32000 * w.astype(np.float64) / w.astype(np.float64).sum()).pvalue > 0.01


@pytest.mark.parametrize("K", [1, 7, 32, 40])
def test_weighted_sampling_bit_exact_on_every_kernel_path(oracle, K):
    """Short columns (thread per column), medium ones (warp, cached or recomputed keys) and a hub
    (CTA per column) draw the same winners as the oracle; columns with fewer positive weights
    than K fill up with zero-weight entries from the lowest positions."""
    rng = np.random.default_rng(100 + K)
    degs = np.concatenate([rng.integers(0, 60, 300), rng.integers(200, 1500, 12), [6000, 9000, 257, 256, K, K + 1]])
    indptr = np.concatenate([[0], np.cumsum(degs)]).astype(np.int64)
    n = degs.size
    indices = rng.integers(0, n, indptr[-1]).astype(np.int64)
    probs = (rng.random(indptr[-1]) + 0.05).astype(np.float32)
    probs[rng.random(probs.size) < 0.2] = 0.0
    z = int(np.flatnonzero(degs == 9000)[0])
    probs[indptr[z]:indptr[z + 1]] = 0.0                  # a hub with no positive weight at all
    probs[indptr[z] + 4321] = 1.0                          # ... except one entry
    seeds = rng.permutation(n)
    want = oracle.sample_probs_spec(indptr, indices, probs, seeds, K, False, seed=9, stream=2)
    sub, rows, cols, sel, err = abi.sample_cols(dev(indptr), dev(indices), dev(seeds), K, False, 9, 2,
                                                probs=dev(probs, torch.float32))
    assert err == 0
    sub, rows, cols, sel = map(host, (sub, rows, cols, sel))
    assert np.array_equal(sub, want[0]) and np.array_equal(cols, want[2])
    assert np.array_equal(rows, indices[sel])
    # the library writes a column's winners in column order, the oracle in its own: same SET
    col_of = np.repeat(np.arange(seeds.size), np.diff(sub))
    assert np.all(np.diff(sel)[np.diff(col_of) == 0] > 0)
    assert np.array_equal(sel, want[3][np.lexsort((want[3], col_of))])


def test_edge_positions_beyond_2_pow_31(oracle):
    """A CSC with int32 row ids and more than 2^31 entries (8.8 GB): edge positions are 64-bit
    all the way.  indices[pos] is a closed-form function of pos written in chunks, so a sampled
    (position, row id) pair can be checked without a host copy of the graph.  Seeds whose
    columns start above 2^31 must yield positions above 2^31, row ids equal to f(position),
    min(deg, K) distinct positions per column, and a relabel that is bit-exact against the
    oracle on the sampled edges; the same through the torch class and the whole-sampler call."""
    import gsampler_b200 as gsb

    deg, ncols, K = 1000, 2_200_000, 10
    nnz = deg * ncols
    assert nnz > 2 ** 31
    mul, mod = 2654435761, 2_199_997          # f(pos) = (pos * mul mod 2^40) mod `mod` < ncols

    def f(pos):
        return ((pos * mul) & ((1 << 40) - 1)) % mod

    indptr = torch.arange(ncols + 1, dtype=torch.int64, device="cuda") * deg
    indices = torch.empty(nnz, dtype=torch.int32, device="cuda")
    step = 1 << 27
    for a in range(0, nnz, step):
        b = min(a + step, nnz)
        indices[a:b] = f(torch.arange(a, b, dtype=torch.int64, device="cuda")).to(torch.int32)
    rng = np.random.default_rng(31)
    first_high = (2 ** 31) // deg + 1                      # first column that starts above 2^31
    seeds = np.concatenate([rng.integers(first_high, ncols, 3000), rng.integers(0, first_high, 1000),
                            [ncols - 1, first_high - 1, first_high]]).astype(np.int64)
    B = 4
    sp = np.array([0, 1000, 1000, 3200, seeds.size], dtype=np.int64)
    sub, rows, cols, sel, err = abi.sample_cols(indptr, indices, dev(seeds), K, False, seed=77, stream=1)
    assert err == 0
    sub_h, rows_h, cols_h, sel_h = map(host, (sub, rows, cols, sel))
    assert np.array_equal(np.diff(sub_h), np.full(seeds.size, K))
    assert np.array_equal(rows_h, f(sel_h))
    col_g = seeds[cols_h]
    assert np.all((sel_h >= col_g * deg) & (sel_h < (col_g + 1) * deg))
    high = col_g >= first_high
    assert high.sum() >= 3000 * K and np.all(sel_h[high] >= 2 ** 31)
    per_col = np.sort(sel_h.reshape(seeds.size, K), axis=1)
    assert np.all(per_col[:, 1:] != per_col[:, :-1])
    # the counter-based draws do not depend on where the column lies: same in-column offsets
    # as the oracle's sampler on a one-column stand-in of the same degree
    esub, _, _, esel = oracle.sample_spec(np.array([0, deg]), np.arange(deg), np.zeros(seeds.size, np.int64),
                                          K, False, 77, 1)
    assert np.array_equal(sel_h - col_g * deg, esel)
    # relabel of the sampled edges, per minibatch, against the oracle
    ep = sub_h[sp]
    uq, up, orow, ocol, err = abi.batch_relabel(dev(seeds), dev(sp), rows, cols, dev(ep), id_bound=ncols)
    assert err == 0
    euq, eup, eorow, eocol = oracle.batch_coo_relabel(seeds, sp, col_g, rows_h, ep)
    assert np.array_equal(host(up), eup) and np.array_equal(host(uq), euq)
    assert np.array_equal(host(orow), eorow) and np.array_equal(host(ocol), eocol)
    # the torch class and the whole-sampler call on the same graph
    A = gsb.Graph(ncols, ncols)
    A._CAPI_LoadCSC(indptr, indices)
    A._CAPI_SetSeed(3)
    out = A._CAPI_BatchGraphSAGE(dev(seeds), dev(sp), [K, 4])
    cur = dev(seeds)
    for l in range(2):
        sub2, rows2, cols2, sel2, eptr2, uq2, up2, brow2, bcol2 = out[9 * l:9 * l + 9]
        assert torch.equal(rows2, f(sel2))
        lo = cur[cols2] * deg
        assert bool(((sel2 >= lo) & (sel2 < lo + deg)).all())
        assert int((sel2 >= 2 ** 31).sum()) > 0
        assert torch.equal(uq2[brow2 + up2[torch.bucketize(torch.arange(rows2.numel(), device="cuda"), eptr2[1:], right=True)]], rows2)
        cur = uq2
    del A, out, indices, indptr
    torch.cuda.empty_cache()


def test_out_of_range_seeds_are_reported_not_read(oracle, graph):
    """A seed that is not a column of the graph -- negative, or at or beyond the column count --
    sets the BAD_INPUT bit and counts as an empty column; the offsets array is not read for it,
    so nothing faults.  The valid seeds of the same call are sampled as usual."""
    indptr, indices = graph
    n = indptr.size - 1
    rng = np.random.default_rng(77)
    good = rng.integers(0, n, 500)
    seeds = good.copy()
    bad_at = np.array([3, 77, 140, 499])
    seeds[bad_at] = [n, -1, 2 ** 40, n + 12345]
    d_ip, d_ix = dev(indptr), dev(indices)
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, dev(seeds), 6, False, seed=5, stream=2)
    assert err & 16
    esub, erows, ecols, esel = oracle.sample_spec(indptr, indices, good, 6, False, 5, 2)
    cnt, ecnt = np.diff(host(sub)), np.diff(esub)
    assert np.all(cnt[bad_at] == 0)
    keep = np.ones(seeds.size, bool); keep[bad_at] = False
    assert np.array_equal(cnt[keep], ecnt[keep])
    live = ~np.isin(ecols, bad_at)                      # the oracle's edges without the bad columns
    assert np.array_equal(host(sel), esel[live]) and np.array_equal(host(rows), erows[live])
    assert np.array_equal(host(cols), ecols[live])
    # the slicing count pass and the weighted sampler share the check
    ssub, srows, scols, ssel, err = abi.slice_cols(d_ip, d_ix, dev(seeds))
    assert err & 16 and np.all(np.diff(host(ssub))[bad_at] == 0)
    probs = dev(rng.random(indices.size) + 0.1, torch.float32)
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, dev(seeds), 4, False, 5, 0, probs=probs)
    assert err & 16 and np.all(np.diff(host(sub))[bad_at] == 0)
    # a graph with fewer columns than rows: a row id that is not a column cannot be a seed
    sub, rows, cols, sel, err = abi.sample_cols(d_ip, d_ix, dev(good), 6, False, 5, 2, num_cols=n // 2)
    assert err & 16 and np.all(np.diff(host(sub))[good >= n // 2] == 0)
