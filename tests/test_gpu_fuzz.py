"""Randomised shapes of the whole layered sampler against the CPU oracle: small graphs with
isolated nodes and hubs, minibatches of uneven sizes (empty ones included), repeated seeds,
1 to 4 layers, fanouts from 1 up, 32-bit and 64-bit row ids -- through the torch class
(`_CAPI_BatchGraphSAGE`) and through the pre-allocated pipeline (`GraphSAGESampler`), which takes
its own 32-bit copy of the row ids."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def host(t):
    return t.cpu().numpy()


def _graph(rng):
    n = int(rng.integers(5, 3000))
    deg = rng.poisson(rng.uniform(0.5, 20), n)
    deg[rng.integers(0, n, max(1, n // 10))] = 0                       # isolated columns
    if n > 50:
        deg[rng.integers(0, n, 3)] = rng.integers(n // 2, n, 3)        # hubs
    deg = np.minimum(deg, n)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg] +
                             [np.empty(0, np.int64)]).astype(np.int64)
    return n, indptr, indices


@pytest.mark.parametrize("case", range(24))
def test_random_super_batches_bit_exact(gsb, oracle, case):
    rng = np.random.default_rng(1000 + case)
    n, indptr, indices = _graph(rng)
    B = int(rng.integers(1, 9))
    sizes = rng.integers(0, 60, B)
    if case % 5 == 0:
        sizes[rng.integers(0, B)] = 0                                   # an empty minibatch
    ptr = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    seeds = rng.integers(0, n, ptr[-1]).astype(np.int64)                # repeats allowed
    fanouts = [int(k) for k in rng.integers(1, 12, int(rng.integers(1, 5)))]
    idx_dtype = torch.int32 if case % 2 else torch.int64
    want = oracle.graphsage_batch(indptr, indices, seeds, ptr, fanouts, seed=77, stream_base=0)

    A = gsb.Graph(n, n)
    A._CAPI_LoadCSC(torch.as_tensor(indptr).cuda(), torch.as_tensor(indices).to(idx_dtype).cuda())
    A._CAPI_SetSeed(77)
    out = A._CAPI_BatchGraphSAGE(torch.as_tensor(seeds).cuda(), torch.as_tensor(ptr).cuda(), fanouts)
    sampler = gsb.GraphSAGESampler(torch.as_tensor(indptr).cuda(), torch.as_tensor(indices).to(idx_dtype).cuda(),
                                   B, max(1, int(ptr[-1])), fanouts, seed=77)
    sampler.sample(torch.as_tensor(seeds).cuda(), torch.as_tensor(ptr).cuda())
    counts = sampler.counts()
    for l, layer in enumerate(want):
        sub, rows, cols, sel, eptr, uq, up, brow, bcol = out[9 * l:9 * l + 9]
        S, E, U = layer["seeds"].size, layer["rows"].size, layer["unique"].size
        assert counts[l] == [S, E, U]
        t = sampler.layers[l]
        for name, got_a, got_b in (("sub_indptr", sub, t["sub_indptr"][:S + 1]), ("rows", rows, t["rows"][:E]),
                                   ("cols", cols, t["cols"][:E]), ("select", sel, t["sel"][:E]),
                                   ("edge_ptr", eptr, t["edge_ptr"]), ("unique", uq, t["unique"][:U]),
                                   ("unique_ptr", up, t["unique_ptr"]), ("block_row", brow, t["block_row"][:E]),
                                   ("block_col", bcol, t["block_col"][:E])):
            assert np.array_equal(host(got_a), layer[name]), (case, l, name, "torch class")
            assert np.array_equal(host(got_b), layer[name]), (case, l, name, "pipeline")
