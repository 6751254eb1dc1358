"""Seeded synthetic graphs with the shapes of the benchmark configurations.

The public datasets gSampler measures on (Reddit, ogbn-products, ogbn-papers100M) are not
redistributable with this repository; these generators produce graphs with the same node /
edge counts and a comparable degree skew:

* :func:`rmat_csc`      R-MAT (a,b,c,d) recursive quadrant sampling, self-loops added,
                        duplicate edges removed -- numpy, deterministic on any machine.
* :func:`powerlaw_csc`  undirected graph whose degree sequence follows a capped power law,
                        returned symmetrised as a CSC with sorted columns -- torch, runs on the
                        GPU for the large shapes.
"""
from __future__ import annotations

import numpy as np
import torch


def coo_to_csc_numpy(row: np.ndarray, col: np.ndarray, num_nodes: int):
    order = np.lexsort((row, col))
    row, col = row[order], col[order]
    indptr = np.zeros(num_nodes + 1, dtype=np.int64)
    np.add.at(indptr, col + 1, 1)
    np.cumsum(indptr, out=indptr)
    return indptr, row.astype(np.int64)


def rmat_csc(num_nodes: int, num_edges: int, abcd=(0.57, 0.19, 0.19, 0.05), seed: int = 42,
             self_loops: bool = True, dedupe: bool = True):
    """R-MAT graph as CSC (int64 indptr / indices), columns sorted.

    ``num_edges`` directed edges are drawn (endpoints outside [0, num_nodes) are redrawn),
    then self-loops are added and duplicates dropped."""
    rng = np.random.default_rng(seed)
    scale = int(np.ceil(np.log2(max(num_nodes, 2))))
    a, b, c, d = abcd
    rows = np.empty(0, np.int64)
    cols = np.empty(0, np.int64)
    while rows.size < num_edges:
        n = int((num_edges - rows.size) * 1.7) + 1024
        r = np.zeros(n, np.int64)
        cc = np.zeros(n, np.int64)
        for _ in range(scale):
            q = rng.random(n)
            right = (q >= a) & (q < a + b) | (q >= a + b + c)   # quadrants b, d: column bit set
            down = q >= a + b                                    # quadrants c, d: row bit set
            r = (r << 1) | down
            cc = (cc << 1) | right
        ok = (r < num_nodes) & (cc < num_nodes)
        rows = np.concatenate([rows, r[ok]])
        cols = np.concatenate([cols, cc[ok]])
    rows, cols = rows[:num_edges], cols[:num_edges]
    if self_loops:
        loop = np.arange(num_nodes, dtype=np.int64)
        rows = np.concatenate([rows, loop])
        cols = np.concatenate([cols, loop])
    if dedupe:
        key = np.unique(cols * num_nodes + rows)
        cols, rows = key // num_nodes, key % num_nodes
    return coo_to_csc_numpy(rows, cols, num_nodes)


def powerlaw_csc(num_nodes: int, num_directed_edges: int, exponent: float = 2.1,
                 max_degree: int = 20000, seed: int = 0, device="cpu",
                 index_dtype=torch.int64):
    """Symmetric graph with exactly ``num_directed_edges`` directed edges (an even number),
    no self-loops, no duplicates; "out-degrees" (stubs per node) follow a power law with the
    given exponent, capped at ``max_degree``; partners are uniform.  Returns
    (indptr int64, indices ``index_dtype``) on ``device`` with sorted columns."""
    assert num_directed_edges % 2 == 0
    target_pairs = num_directed_edges // 2
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    dev = torch.device(device)
    u = torch.rand(num_nodes, generator=gen, device=dev, dtype=torch.float64)
    raw = (1.0 - u).clamp_min(1e-12).pow(-1.0 / (exponent - 1.0)).clamp_max(float(max_degree))
    keys = torch.empty(0, dtype=torch.int64, device=dev)
    want = int(target_pairs * 1.04) + 16
    while keys.numel() < target_pairs:
        scale = want / float(raw.sum())
        for _ in range(8):  # rescale so that the capped degrees still sum to `want`
            scale *= want / float((raw * scale).clamp_max(float(max_degree)).sum())
        deg = torch.floor((raw * scale).clamp_max(float(max_degree)) +
                          torch.rand(num_nodes, generator=gen, device=dev,
                                     dtype=torch.float64)).to(torch.int64)
        src = torch.repeat_interleave(torch.arange(num_nodes, device=dev), deg)
        dst = torch.randint(0, num_nodes, (src.numel(),), generator=gen, device=dev)
        keep = src != dst
        lo, hi = torch.minimum(src, dst)[keep], torch.maximum(src, dst)[keep]
        keys = torch.unique(torch.cat([keys, lo * num_nodes + hi]))
        want = int(want * 1.05)
        del src, dst, keep, lo, hi
    if keys.numel() > target_pairs:
        perm = torch.randperm(keys.numel(), generator=gen, device=dev)[:target_pairs]
        keys = keys[perm]
    lo, hi = keys // num_nodes, keys % num_nodes
    del keys
    col = torch.cat([lo, hi])
    row = torch.cat([hi, lo])
    del lo, hi
    order = torch.argsort(col * num_nodes + row)
    row, col = row[order], col[order]
    del order
    indptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=dev)
    indptr[1:] = torch.cumsum(torch.bincount(col, minlength=num_nodes), 0)
    return indptr, row.to(index_dtype)


def seed_batches(num_seeds: int, num_nodes: int, batch: int, seed: int, device="cpu"):
    """``num_seeds`` distinct training seeds (a seeded permutation prefix) and the list of
    minibatch boundaries: returns (seeds int64, ptr int64 with steps of ``batch``)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    seeds = torch.randperm(num_nodes, generator=gen)[:num_seeds].to(torch.int64)
    ptr = torch.arange(0, num_seeds + batch, batch, dtype=torch.int64).clamp_max(num_seeds)
    if ptr[-1] == ptr[-2] and ptr.numel() > 2:
        ptr = ptr[:-1]
    return seeds.to(device), ptr.to(device)


def powerlaw_csc_large(num_nodes: int, num_directed_edges: int, exponent: float = 2.1,
                       max_degree: int = 100000, seed: int = 0, device="cuda", chunk: int = 1 << 28):
    """Memory-lean variant of :func:`powerlaw_csc` for billions of edges (int32 indices, int64
    offsets): same construction -- power-law stub counts, uniform partners, no self-loops, no
    duplicate pairs, symmetric -- but the CSC is assembled from two sorts of the undirected
    pairs instead of a sort of all directed edges.  For a column c the neighbours below c are
    the ``lo`` ends of the pairs with ``hi == c`` and the neighbours above c are the ``hi`` ends
    of the pairs with ``lo == c``; listing the first group (sorted by lo) before the second
    (sorted by hi) gives a sorted column without any further sort.  The number of edges is
    close to, not exactly, ``num_directed_edges`` (duplicates are dropped, the surplus is thinned
    at random).  Returns (indptr int64, indices int32)."""
    assert num_nodes < (1 << 31)
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    target = num_directed_edges // 2
    want = int(target * 1.03) + 16
    u = torch.rand(num_nodes, generator=gen, device=dev, dtype=torch.float64)
    raw = (1.0 - u).clamp_min_(1e-12).pow_(-1.0 / (exponent - 1.0)).clamp_max_(float(max_degree))
    del u
    scale = want / float(raw.sum())
    for _ in range(8):
        scale *= want / float((raw * scale).clamp_max(float(max_degree)).sum())
    deg = torch.floor((raw * scale).clamp_max_(float(max_degree)) +
                      torch.rand(num_nodes, generator=gen, device=dev, dtype=torch.float64)).to(torch.int64)
    del raw
    src = torch.repeat_interleave(torch.arange(num_nodes, device=dev, dtype=torch.int32), deg)
    del deg
    dst = torch.randint(0, num_nodes, (src.numel(),), generator=gen, device=dev, dtype=torch.int32)
    lo, hi = torch.minimum(src, dst), torch.maximum(src, dst)
    del src, dst
    keep = lo != hi
    key = lo[keep].to(torch.int64) * num_nodes + hi[keep]
    del lo, hi, keep
    key = torch.unique_consecutive(torch.sort(key).values)
    if key.numel() > target:
        thin = torch.rand(key.numel(), generator=gen, device=dev) < (target / key.numel())
        key = key[thin]
        del thin
    m = key.numel()
    lo = torch.div(key, num_nodes, rounding_mode="floor").to(torch.int32)   # sorted by (lo, hi)
    hi = (key - lo.to(torch.int64) * num_nodes).to(torch.int32)
    key2 = torch.sort(hi.to(torch.int64) * num_nodes + lo).values           # sorted by (hi, lo)
    del key
    hi2 = torch.div(key2, num_nodes, rounding_mode="floor").to(torch.int32)
    lo2 = (key2 - hi2.to(torch.int64) * num_nodes).to(torch.int32)
    del key2
    cnt_lo = torch.bincount(lo, minlength=num_nodes)     # neighbours above c
    cnt_hi = torch.bincount(hi2, minlength=num_nodes)    # neighbours below c
    indptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=dev)
    indptr[1:] = torch.cumsum(cnt_lo + cnt_hi, 0)
    start_lo = torch.cumsum(cnt_lo, 0) - cnt_lo
    start_hi = torch.cumsum(cnt_hi, 0) - cnt_hi
    indices = torch.empty(2 * m, dtype=torch.int32, device=dev)
    for a in range(0, m, chunk):
        b = min(a + chunk, m)
        j = torch.arange(a, b, device=dev)
        c = hi2[a:b].to(torch.int64)                      # below-c group first
        indices[indptr[c] + (j - start_hi[c])] = lo2[a:b]
        c = lo[a:b].to(torch.int64)                       # then the above-c group
        indices[indptr[c] + cnt_hi[c] + (j - start_lo[c])] = hi[a:b]
        del j, c
    return indptr, indices
