"""GPU tests of the host layer (torch.classes.gs_classes.Graph) and of the Python surface
(Matrix / BatchMatrix / compile) against the CPU oracle, on the CPU-baseline configuration:
R-MAT graph, 100 000 nodes / 2 000 000 drawn edges, 2-layer GraphSAGE, fanouts [25, 10]."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def host(t):
    return t.cpu().numpy()


def cuda(a):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=torch.int64).cuda()


@pytest.fixture(scope="module")
def rmat():
    from gsampler_b200 import synth

    return synth.rmat_csc(100000, 2000000, seed=42)


@pytest.fixture(scope="module")
def fx():
    with open(os.path.join(HERE, "golden", "reference_fixtures.json")) as f:
        return json.load(f)


def new_graph(gsb, indptr, indices, seed=4242, idx_dtype=torch.int64):
    n = indptr.size - 1
    g = gsb.Graph(n, n)
    g._CAPI_LoadCSC(torch.as_tensor(indptr).cuda(), torch.as_tensor(indices).to(idx_dtype).cuda())
    g._CAPI_SetSeed(seed)
    return g


def test_reference_gtest_fixtures(gsb, fx):
    c = fx["colwise_slicing"]
    A = new_graph(gsb, np.asarray(c["indptr"]), np.asarray(c["indices"]))
    sub, _ = A._CAPI_Slicing(torch.tensor(c["cols"]).cuda(), 1, gsb._CSC, gsb._CSC)
    assert host(sub._CAPI_GetCSCIndptr()).tolist() == c["expect_indptr"]
    assert host(sub._CAPI_GetCSCIndices()).tolist() == c["expect_indices"]
    c = fx["colwise_sampling"]
    sub, _ = A._CAPI_Sampling(1, c["copy_all"]["fanout"], False, gsb._CSC, gsb._CSC)
    assert host(sub._CAPI_GetCSCIndptr()).tolist() == c["copy_all"]["expect_indptr"]
    assert host(sub._CAPI_GetCSCIndices()).tolist() == c["copy_all"]["expect_indices"]
    for case in c["replace"]:
        sub, _ = A._CAPI_Sampling(1, case["fanout"], True, gsb._CSC, gsb._CSC)
        assert host(sub._CAPI_GetCSCIndptr()).tolist() == case["expect_indptr"]
        ids = host(sub._CAPI_GetCSCIndices())
        assert ids.size == 20 * case["fanout"] and ids.tolist() != c["indices"]
        assert np.unique(ids).size <= 100
    c = fx["rowwise_slicing"]
    A = new_graph(gsb, np.asarray(c["indptr"]), np.asarray(c["indices"]))
    sub, _ = A._CAPI_Slicing(torch.tensor(c["rows"]).cuda(), 0, gsb._CSR, gsb._CSR)
    assert sub._CAPI_GetCSRIndptr().numel() == c["expect_csr_indptr_numel"]
    assert host(sub._CAPI_GetCSRIndices()).tolist() == c["expect_csr_indices"]


def _seeds(n_nodes, nb=4, bs=1024, seed=0):
    rng = np.random.default_rng(seed)
    seeds = rng.permutation(n_nodes)[:nb * bs].astype(np.int64)
    ptr = np.arange(nb + 1, dtype=np.int64) * bs
    return seeds, ptr


def _compare_layer(layer, sub, rows, cols, sel, uq, up, brow, bcol):
    assert np.array_equal(host(sub), layer["sub_indptr"])
    assert np.array_equal(host(sel), layer["select"])
    assert np.array_equal(host(rows), layer["rows"])
    assert np.array_equal(host(cols), layer["cols"])
    assert np.array_equal(host(up), layer["unique_ptr"])
    assert np.array_equal(host(uq), layer["unique"])
    assert np.array_equal(host(brow), layer["block_row"])
    assert np.array_equal(host(bcol), layer["block_col"])


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_native_graphsage_pipeline_bit_exact(gsb, oracle, rmat, idx_dtype):
    indptr, indices = rmat
    seeds, ptr = _seeds(indptr.size - 1)
    want = oracle.graphsage_batch(indptr, indices, seeds, ptr, [25, 10], seed=4242)
    A = new_graph(gsb, indptr, indices, idx_dtype=idx_dtype)
    out = A._CAPI_BatchGraphSAGE(torch.as_tensor(seeds).cuda(), torch.as_tensor(ptr).cuda(), [25, 10])
    counts = out[-1].numpy()
    for l, layer in enumerate(want):
        sub, rows, cols, sel, eptr, uq, up, brow, bcol = out[9 * l:9 * l + 9]
        _compare_layer(layer, sub, rows, cols, sel, uq, up, brow, bcol)
        assert np.array_equal(host(eptr), layer["edge_ptr"])
        assert counts[3 * l:3 * l + 3].tolist() == [layer["seeds"].size, layer["rows"].size,
                                                    layer["unique"].size]


def test_preallocated_sampler_cuda_graph_replay(gsb, oracle, rmat):
    """The pre-allocated pipeline recorded into a CUDA graph and replayed on a full and on a
    shorter super-batch: bit-exact against the oracle both times."""
    indptr, indices = rmat
    n = indptr.size - 1
    rng = np.random.default_rng(12)
    smp = gsb.GraphSAGESampler(torch.as_tensor(indptr).cuda(), torch.as_tensor(indices).cuda(), 4, 2048,
                               [10, 5], seed=321)
    smp.capture()
    for sizes in ([512, 512, 512, 512], [300, 0, 77, 0]):
        ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        seeds = rng.permutation(n)[:ptr[-1]].astype(np.int64)
        smp.replay(torch.as_tensor(seeds).cuda(), torch.as_tensor(ptr).cuda())
        counts = smp.counts()
        want = oracle.graphsage_batch(indptr, indices, seeds, ptr, [10, 5], seed=321)
        for l, layer in enumerate(want):
            S, E, U = counts[l]
            assert (S, E, U) == (layer["seeds"].size, layer["rows"].size, layer["unique"].size)
            L = smp.layers[l]
            assert np.array_equal(host(L["rows"][:E]), layer["rows"])
            assert np.array_equal(host(L["unique"][:U]), layer["unique"])
            assert np.array_equal(host(L["block_row"][:E]), layer["block_row"])
            assert np.array_equal(host(L["block_col"][:E]), layer["block_col"])
    assert smp.replayed_launches > 0


def test_graphsage_async_two_in_flight(gsb, rmat):
    """The enqueue-only form gives the same tensors as the synchronous one, also with two
    super-batches in flight on two streams."""
    indptr, indices = rmat
    seeds, ptr = _seeds(indptr.size - 1)
    A = new_graph(gsb, indptr, indices)
    bm = gsb.BatchMatrix()
    bm.load_from_matrix(gsb.Matrix(A), False)
    sd, pd = torch.as_tensor(seeds).cuda(), torch.as_tensor(ptr).cuda()
    A._CAPI_SetSeed(77)
    want = [bm.graphsage(sd, pd, [10, 5]) for _ in range(2)]
    A._CAPI_SetSeed(77)
    torch.cuda.synchronize()
    futs = []
    for i in range(2):
        with torch.cuda.stream(torch.cuda.Stream()):
            futs.append(bm.graphsage_async(sd, pd, [10, 5]))
    got = [f.wait() for f in futs]
    torch.cuda.synchronize()
    for w, g in zip(want, got):
        assert len(w) == len(g)
        for a, b in zip(w, g):
            assert torch.equal(a.cpu(), b.cpu())


def test_batchmatrix_sampler_matches_oracle(gsb, oracle, rmat):
    """The reference's batch_graphsage_sampler (examples/graphsage/graphsage.py:20-27) written
    against this package's BatchMatrix."""
    indptr, indices = rmat
    seeds, ptr = _seeds(indptr.size - 1, nb=3, bs=512, seed=1)
    fanouts = [25, 10]
    want = oracle.graphsage_batch(indptr, indices, seeds, ptr, fanouts, seed=4242)

    def sampler(A, seeds, seeds_ptr, fanouts):
        ret = []
        for k in fanouts:
            subA = A[:, seeds::seeds_ptr]
            sampleA = subA.individual_sampling(k, None, False)
            seeds, seeds_ptr = sampleA.all_nodes()
            ret.append(sampleA.to_dgl_block())
        return ret

    m = gsb.Matrix(new_graph(gsb, indptr, indices))
    bm = gsb.BatchMatrix()
    bm.load_from_matrix(m, False)
    fn = gsb.jit.compile(func=sampler, args=(bm, torch.as_tensor(seeds).cuda(),
                                            torch.as_tensor(ptr).cuda(), fanouts))
    blocks = fn(bm, torch.as_tensor(seeds).cuda(), torch.as_tensor(ptr).cuda(), fanouts)
    for l, layer in enumerate(want):
        assert len(blocks[l]) == 3
        for b, blk in enumerate(blocks[l]):
            e0, e1 = layer["edge_ptr"][b], layer["edge_ptr"][b + 1]
            u0, u1 = layer["unique_ptr"][b], layer["unique_ptr"][b + 1]
            assert np.array_equal(host(blk.row), layer["block_row"][e0:e1])
            assert np.array_equal(host(blk.col), layer["block_col"][e0:e1])
            assert np.array_equal(host(blk.srcdata["_ID"]), layer["unique"][u0:u1])
            assert blk.num_src_nodes() == u1 - u0
            assert blk.num_dst_nodes() == layer["seeds_ptr"][b + 1] - layer["seeds_ptr"][b]


def test_batch_blocks_in_csc_form(gsb, oracle, rmat):
    """to_dgl_block(block_format="csc"): per minibatch the offsets over its seed slots and the
    relabelled row ids -- the CSC block build (src/cuda/batch/batch_relabel.cu:215-321 in gSampler
    prepares the same arrays).  Expanding the offsets gives back the COO block, and both equal the
    oracle's relabel of the sampled edges."""
    indptr, indices = rmat
    seeds, ptr = _seeds(indptr.size - 1, nb=4, bs=300, seed=9)
    ptr[2] = ptr[1]                                             # an empty minibatch
    m = gsb.Matrix(new_graph(gsb, indptr, indices))
    bm = gsb.BatchMatrix()
    bm.load_from_matrix(m, False)
    d_seeds, d_ptr = torch.as_tensor(seeds).cuda(), torch.as_tensor(ptr).cuda()
    cur_seeds, cur_ptr = seeds, ptr
    for K in (7, 3):
        sample = bm[:, d_seeds::d_ptr].individual_sampling(K, None, False)
        coo = sample.to_dgl_block()
        csc = sample.to_dgl_block(block_format="csc")
        sub = sample._graph
        rows_g, cols = host(sub._CAPI_GetCOORows()), host(sub._CAPI_GetCOOCols())
        eptr = host(sub._CAPI_GetEdgeBptr())
        euq, eup, erow, ecol = oracle.batch_coo_relabel(cur_seeds, cur_ptr, cur_seeds[cols], rows_g, eptr)
        assert len(coo) == len(csc) == ptr.size - 1
        for b, (a, c) in enumerate(zip(coo, csc)):
            ns = int(cur_ptr[b + 1] - cur_ptr[b])
            ip = host(c.indptr)
            assert ip.size == ns + 1 and ip[0] == 0 and c.num_dst_nodes() == ns
            assert np.array_equal(np.repeat(np.arange(ns), np.diff(ip)), host(a.col))   # seeds are distinct here
            assert np.array_equal(host(c.row), host(a.row)) and c.col is None
            assert np.array_equal(host(c.row), erow[eptr[b]:eptr[b + 1]])
            assert np.array_equal(host(c.srcdata["_ID"]), euq[eup[b]:eup[b + 1]])
        d_seeds, d_ptr = sample.all_nodes()
        cur_seeds, cur_ptr = host(d_seeds), host(d_ptr)


def test_matrix_sampler_matches_oracle(gsb, oracle, rmat):
    """Single-minibatch graphsage_sampler (examples/graphsage/graphsage.py:7-17): slice, sample,
    all_nodes, to_dgl_block -- both the fused (lazy slice) and the unfused order of calls."""
    indptr, indices = rmat
    rng = np.random.default_rng(3)
    seeds0 = rng.integers(0, indptr.size - 1, 1024).astype(np.int64)   # duplicates allowed
    fanouts = [25, 10]
    want = oracle.graphsage_batch(indptr, indices, seeds0, np.array([0, 1024]), fanouts, seed=4242)
    for fused in (True, False):
        m = gsb.Matrix(new_graph(gsb, indptr, indices))
        seeds = torch.as_tensor(seeds0).cuda()
        for l, K in enumerate(fanouts):
            subA = m[:, seeds]
            if not fused:
                assert subA.num_edges() >= 0            # touching the graph materialises the slice
            sampleA = subA.individual_sampling(K, None, False)
            seeds = sampleA.all_nodes()
            blk = sampleA.to_dgl_block()
            layer = want[l]
            assert np.array_equal(host(seeds), layer["unique"])
            if fused:
                # unfused sampling draws with slot = column of the slice and the same stream
                # counter, so both orders give the same picks
                pass
            assert np.array_equal(host(blk.row), layer["block_row"])
            assert np.array_equal(host(blk.col), layer["block_col"])
            assert blk.num_dst_nodes() == layer["seeds"].size


def test_graph_accessors_and_formats(gsb, oracle):
    rng = np.random.default_rng(5)
    deg = rng.poisson(5, 300)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, 300, indptr[-1]).astype(np.int64)
    A = new_graph(gsb, indptr, indices)
    assert (A._CAPI_GetNumRows(), A._CAPI_GetNumCols(), A._CAPI_GetNumEdges()) == (300, 300, indptr[-1])
    assert np.array_equal(host(A._CAPI_GetCOOCols()), oracle.csc2coo(indptr))
    assert np.array_equal(host(A._CAPI_GetCOORows()), indices)
    ip, ids, perm = oracle.coo2csc(indices, oracle.csc2coo(indptr), 300)
    assert np.array_equal(host(A._CAPI_GetCSRIndptr()), ip)
    assert np.array_equal(host(A._CAPI_GetCSRIndices()), ids)
    assert np.array_equal(host(A._CAPI_GetCSREids()), perm)
    # slicing with encoding: per-minibatch compacted rows
    seeds = torch.as_tensor(rng.integers(0, 300, 40)).cuda()
    ptr = torch.tensor([0, 10, 40]).cuda()
    sub, _ = A._CAPI_BatchColSlicing(seeds, ptr, True)
    rows, row_ptr = sub._CAPI_BatchGetRows()
    esub, erows, _, _ = oracle.slice_cols(indptr, indices, host(seeds), host(ptr), 300)
    uq, cp = oracle.compact(erows)
    bp, dec = oracle.batch_offsets(uq, 2, 300)
    assert np.array_equal(host(rows), dec) and np.array_equal(host(row_ptr), bp)
    assert np.array_equal(host(sub._CAPI_GetCSCIndices()), cp)
    counts = sub._CAPI_BatchGetColCounts()
    assert counts == [10, 30]


def test_unsorted_coo_to_csc_and_csr_is_the_stable_grouping(gsb):
    """An unsorted COO turned into CSC and CSR by the library's counting sort (histogram, scan,
    scatter, per-segment sort by original position): offsets, ids and the edge-id permutation equal
    a stable sort by key (what the reference's radix sort of (key, position) pairs gives,
    src/cuda/format_transform.cu:66-86, 108-142).  Empty segments, a segment of 40 000 entries
    (the long-column sort path) and segments of a few thousand are present."""
    rng = np.random.default_rng(12)
    n, nnz = 50000, 1_500_000
    row = rng.integers(0, n, nnz)
    col = rng.integers(0, n, nnz)
    col[rng.choice(nnz, 40000, replace=False)] = 7          # one hub column
    col[col == 11] = 12                                      # an empty column
    row[rng.choice(nnz, 3000, replace=False)] = 123          # a mid-size row
    g = gsb.Graph(n, n)
    g._CAPI_LoadCOO(cuda(row), cuda(col), False, False)
    for key, val, ip_fn, id_fn, e_fn in ((col, row, g._CAPI_GetCSCIndptr, g._CAPI_GetCSCIndices, g._CAPI_GetCSCEids),
                                         (row, col, g._CAPI_GetCSRIndptr, g._CAPI_GetCSRIndices, g._CAPI_GetCSREids)):
        perm = np.argsort(key, kind="stable")
        want_ip = np.concatenate([[0], np.cumsum(np.bincount(key, minlength=n))])
        assert np.array_equal(host(ip_fn()), want_ip)
        assert np.array_equal(host(id_fn()), val[perm])
        assert np.array_equal(host(e_fn()), perm)
    gsb.check_async_errors()


def test_short_row_id_map_is_an_exception(gsb, rmat):
    """A row-id map shorter than the row ids it is indexed with is reported as an exception (the
    gather is bounds-checked on the device), and the context stays usable."""
    indptr, indices = rmat
    A = new_graph(gsb, indptr, indices)
    seeds = torch.arange(0, 64, device="cuda")
    sub, _ = A._CAPI_SlicingSampling(1, seeds, 5, False, gsb._CSC, gsb._COO)
    short_map = torch.arange(0, 10, device="cuda")
    with pytest.raises(RuntimeError):
        sub._CAPI_GetValidNodes(seeds, short_map)
    with pytest.raises(RuntimeError):
        sub._CAPI_GraphRelabel(seeds, short_map)
    ok = sub._CAPI_GetValidNodes(seeds, torch.empty(0, dtype=torch.int64, device="cuda"))
    assert ok.numel() >= 64


def test_errors_are_exceptions(gsb):
    A = gsb.Graph(4, 4)
    A._CAPI_LoadCSC(torch.tensor([0, 1, 2, 3, 4]).cuda(), torch.tensor([0, 1, 2, 3]).cuda())
    with pytest.raises(RuntimeError):
        A._CAPI_Slicing(torch.tensor([0, 1]), 1, gsb._CSC, gsb._CSC)        # CPU tensor
    with pytest.raises(RuntimeError):
        A._CAPI_Sampling(1, 0, False, gsb._CSC, gsb._CSC)                    # fanout 0
    with pytest.raises(RuntimeError):
        A._CAPI_Sampling(0, 2, False, gsb._CSC, gsb._CSC)                    # axis / format mismatch
