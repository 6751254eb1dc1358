"""The allocation-free sampling entry point (``gsb_sample_cols_noalloc``).

Some users of the library cannot call ``cudaMalloc``: code that lives inside another
application's memory budget and only receives input and output buffers, or threads that must
keep away from the allocator because allocating and freeing synchronise the whole device.
For them the sampling kernel's scratch words sit in a fixed array inside the library.  This
test calls that entry point through the C ABI twice in a row (the second call finds the first
call's words in the shared array) and requires bit-identical results with the regular entry
point, which gets a fresh workspace each time.  It is collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import abi

pytestmark = pytest.mark.gpu


def _noalloc(indptr, indices, seeds, K, replace, seed, stream):
    L = abi.lib()
    S = seeds.numel()
    o = dict(dtype=torch.int64, device=indptr.device)
    sub = torch.full((S + 1,), -7, **o)
    rows, cols, sel = (torch.full((S * K,), -7, **o) for _ in range(3))
    n_edges = torch.zeros(1, **o)
    err = torch.zeros(1, dtype=torch.int32, device=indptr.device)
    dt = abi.I32 if indices.dtype == torch.int32 else abi.I64
    rc = L.gsb_sample_cols_noalloc(abi.ptr(indptr), abi.ptr(indices), dt, abi.i64(indptr.numel() - 1),
                                   abi.ptr(seeds), abi.i64(S), None, abi.i64(K), int(replace), C.c_uint64(seed),
                                   C.c_uint32(stream), abi.ptr(sub), abi.ptr(rows), abi.ptr(cols),
                                   abi.ptr(sel), abi.i64(S * K), abi.ptr(n_edges), abi.ptr(err),
                                   C.c_void_p(torch.cuda.current_stream().cuda_stream))
    abi.check(rc, "gsb_sample_cols_noalloc")
    torch.cuda.synchronize()
    E = int(n_edges[0])
    return sub, rows[:E], cols[:E], sel[:E], int(err[0])


def test_noalloc_matches_regular_entry_point_twice():
    rng = np.random.default_rng(123)
    n = 4000
    deg = rng.poisson(20, n)
    deg[::7] = 0
    indptr = torch.as_tensor(np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)).cuda()
    indices = torch.as_tensor(rng.integers(0, n, int(deg.sum())).astype(np.int64)).cuda()
    # first call: many tiles; second call: fewer tiles, other fanout -> stale words beyond its
    # own range stay in the shared array and must not matter
    for S, K, replace, idx in ((3000, 7, False, indices), (700, 12, False, indices.to(torch.int32)),
                               (900, 5, True, indices)):
        seeds = torch.as_tensor(rng.integers(0, n, S).astype(np.int64)).cuda()
        got = _noalloc(indptr, idx, seeds, K, replace, seed=2718, stream=S)
        want = abi.sample_cols(indptr, idx, seeds, K, replace, seed=2718, stream=S)
        assert got[4] == 0 and want[4] == 0
        for a, b in zip(got[:4], want[:4]):
            assert torch.equal(a, b)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    L = abi.lib()
    L.gsb_sample_cols_noalloc_max_columns.restype = C.c_int64
    limit = L.gsb_sample_cols_noalloc_max_columns(abi.i64(15))
    assert limit == 65536 * 256
    rc = L.gsb_sample_cols_noalloc(None, None, 1, abi.i64(1), None, abi.i64(limit + 1), None, abi.i64(15), 0,
                                   C.c_uint64(0), C.c_uint32(0), None, None, None, None,
                                   abi.i64(0), None, None, None)
    assert rc == 5
    assert b"fixed scratch" in L.gsb_status_string(rc)
