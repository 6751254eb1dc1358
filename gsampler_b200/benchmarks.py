"""Secondary benchmarks of the operators next to the GraphSAGE path (``bench.py`` at the
repository root holds the headline one):

    python -m gsampler_b200.benchmarks ladies     # 2-layer LADIES, 4000 nodes/layer, 512 seeds,
                                                  # 232 965 nodes / 114.6 M weighted edges
    python -m gsampler_b200.benchmarks node2vec   # 1 M walkers x 80 steps, p=2, q=0.5,
                                                  # 2 449 029 nodes / 123.7 M edges
    python -m gsampler_b200.benchmarks limits     # uniform walks, COO row sums, uniform list sampling on
                                                  # a 1 M-node / 50 M-edge graph (a profiling shape)
    python -m gsampler_b200.benchmarks weighted   # weighted per-column sampling of a column slice, same
                                                  # 1 M-node graph: 400 000 columns, K = 10 and K = 5
    python -m gsampler_b200.benchmarks gather     # feature fetch: 4 M rows of 100 fp32 out of 2 449 029
    python -m gsampler_b200.benchmarks cfg5       # the same on the full 111 M nodes / 3.2 G edges (14 GB)
    python -m gsampler_b200.benchmarks cfg5s      # GraphSAGE [15,10,5] on an int32-index R-MAT-like
                                                  # power-law graph, 11.1 M nodes / 320 M edges

Each prints one JSON line with the metric, the per-kernel CUDA-event times collected by the
library's launch accounting, and the algorithmic GB/s of the dominant kernel.  Graphs are
seeded synthetic stand-ins with the shapes named above.
"""
from __future__ import annotations

import json
import sys
import time

import torch

import gsampler_b200 as gs
from gsampler_b200 import pipeline, synth

PEAK_GBS = 6535.4  # measured copy bandwidth of this pool's B200 (MEASURED_PEAKS.json)


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _kernel_table(timed):
    by = {}
    for name, tag, ms, cnt in timed:
        a = by.setdefault(name, [0.0, 0])
        a[0] += ms
        a[1] += cnt
    return {k: {"ms": round(v[0], 4), "launches": v[1]} for k, v in sorted(by.items())}


def ladies(steps=10, warmup=3):
    dev = torch.device("cuda")
    n, e, nseeds, K = 232965, 114615892, 512, 4000
    indptr, indices = synth.powerlaw_csc(n, e, exponent=2.1, max_degree=30000, seed=11, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    w = torch.rand(indices.numel(), generator=g, device=dev).clamp_min_(1e-3)
    A = gs.Graph(n, n)
    A._CAPI_LoadCSC(indptr, indices)
    m = gs.Matrix(A)
    m.edata["w"] = w
    # column-normalise once (the reference's P = D^-1/2 A D^-1/2 preprocessing is out of the loop)
    colsum = m.sum("w", axis=0)
    m = m.div("w", colsum.clamp_min(1e-12), axis=0)

    def layer_fn(A, seeds, fanouts):
        edges = 0
        for k in fanouts:
            subA = A[:, seeds]
            subA.edata["p"] = subA.edata["w"] ** 2
            prob = subA.sum("p", axis=1)
            sampleA, sel = subA.collective_sampling(k, prob, False)
            sampleA = sampleA.div("w", prob[sel], axis=1)
            out = sampleA.sum("w", axis=0)
            sampleA = sampleA.div("w", out, axis=0)
            seeds = sampleA.all_nodes()
            blk = sampleA.to_dgl_block(prefetch_edata={"w"})
            edges += blk.num_edges()
        return edges

    gen = torch.Generator()
    gen.manual_seed(1)
    batches = [torch.randperm(n, generator=gen)[:nseeds].to(dev) for _ in range(steps + warmup)]
    for i in range(warmup):
        layer_fn(m, batches[i], [K, K])
    torch.cuda.synchronize()
    e0, e1 = _events()
    e0.record()
    edges = 0
    for i in range(steps):
        edges += layer_fn(m, batches[warmup + i], [K, K])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    pipeline.timing_enable(True)
    for i in range(steps):
        layer_fn(m, batches[warmup + i], [K, K])
    timed = pipeline.timing_collect()
    pipeline.timing_enable(False)
    # the same layers through the single native call per layer
    def native_fn(A, seeds, fanouts):
        edges = 0
        for k in fanouts:
            blk, seeds, _ = A.ladies_layer(seeds, k)
            edges += blk.num_edges()
        return edges

    for i in range(warmup):
        native_fn(m, batches[i], [K, K])
    torch.cuda.synchronize()
    e0, e1 = _events()
    e0.record()
    n_edges = 0
    for i in range(steps):
        n_edges += native_fn(m, batches[warmup + i], [K, K])
    e1.record()
    torch.cuda.synchronize()
    native_ms = e0.elapsed_time(e1)
    print(json.dumps({"metric": "ladies_block_edges_per_sec", "value": edges / (ms / 1e3), "unit": "edges/s",
                      "native_layer_call": {"value": n_edges / (native_ms / 1e3), "ms_per_step": native_ms / steps,
                                            "edges_per_step": n_edges / steps},
                      "ms_per_step": ms / steps, "steps": steps, "edges_per_step": edges / steps,
                      "config": {"workload": "LADIES 2 layers x %d nodes, %d seeds, %d nodes / %d edges fp32 w"
                                 % (K, nseeds, n, int(indptr[-1]))},
                      "kernels": _kernel_table(timed)}))


def node2vec(steps=3, warmup=1, walkers=1000000, length=80):
    dev = torch.device("cuda")
    n, e = 2449029, 123718280
    indptr, indices = synth.powerlaw_csc(n, e, exponent=2.1, max_degree=20000, seed=2024, device=dev)
    A = gs.Graph(n, n)
    A._CAPI_LoadCSC(indptr, indices)
    A._CAPI_SortCSCIndices()     # generator output is already sorted; kept for the API contract
    gen = torch.Generator()
    gen.manual_seed(7)
    seeds = torch.randint(0, n, (walkers,), generator=gen).to(dev)
    out = {}
    for name, fn in (("node2vec", lambda: A._CAPI_Node2Vec(seeds, length, 2.0, 0.5)),
                     ("random_walk", lambda: A._CAPI_RandomWalk(seeds, length))):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            tr = fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        live = int((tr.reshape(length + 1, walkers)[1:] >= 0).sum())
        # compulsory bytes per taken step: indptr pair + one id + the trace entry
        alg = live * (16 + 8 + 8)
        out[name] = {"ms_per_call": ms, "steps_per_sec": live / (ms / 1e3),
                     "algorithmic_gbs": alg / (ms / 1e3) / 1e9, "frac_of_copy_peak": alg / (ms / 1e3) / 1e9 / PEAK_GBS,
                     "live_steps": live}
    print(json.dumps({"metric": "walk_steps_per_sec", "value": out["node2vec"]["steps_per_sec"],
                      "unit": "steps/s",
                      "config": {"workload": "%d walkers x %d steps, p=2 q=0.5, %d nodes / %d edges"
                                 % (walkers, length, n, int(indptr[-1]))}, **out}))


def limits(steps=3, warmup=2, n=1000000, e=50000000):
    """Operators whose rate is set by one hardware unit rather than by the algorithm: uniform
    walks (random 32-byte gathers), row sums over a COO in column order (one L2 reduction per
    edge), the fused pair of u-op-v maps (a streaming pass) and a uniform choice from one list
    (one Philox block per candidate).  Small enough for a profiler capture, larger than L2."""
    dev = torch.device("cuda")
    indptr, indices = synth.powerlaw_csc(n, e, exponent=2.1, max_degree=20000, seed=2024, device=dev)
    nnz = int(indptr[-1])
    A = gs.Graph(n, n)
    A._CAPI_LoadCSC(indptr, indices)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    walkers = torch.randint(0, n, (400000,), generator=gen, device=dev)
    M = gs.Matrix(A)
    M.edata["w"] = torch.rand(nnz, generator=gen, device=dev)
    M.sum("w", axis=1)   # builds the COO outside the timed calls
    u1, v1, u2, v2 = (torch.rand(n, 1, generator=gen, device=dev) + 0.5 for _ in range(4))
    o1, o2 = torch.empty(nnz, 1, device=dev), torch.empty(nnz, 1, device=dev)
    # the yardstick for a walk step: as many 8-byte gathers from random places of the row-id array
    # as the walks take steps, by the tensor library (it also reads the positions and writes the result)
    where = torch.randint(0, nnz, (400000 * 80,), generator=gen, device=dev)
    out = {}
    for name, fn, units in (("random_walk", lambda: A._CAPI_RandomWalk(walkers, 80), 400000 * 80),
                            ("library_gather_of_as_many_row_ids", lambda: torch.index_select(indices, 0, where), 400000 * 80),
                            ("coo_row_sums", lambda: M.sum("w", axis=1), nnz),
                            ("fused_u_op_v", lambda: A._CAPI_FusedUOPV("mul", u1, v1, o1, u2, v2, o2, gs._COO), nnz),
                            ("list_sampling_uniform", lambda: torch.ops.gs_ops._CAPI_ListSampling(n, 4000, False), n)):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[name] = {"ms_per_call": ms, "units_per_sec": units / (ms / 1e3)}
    print(json.dumps({"metric": "operator_ms", "config": {"workload": "%d nodes / %d edges" % (n, nnz)}, **out}))


def weighted(steps=3, warmup=2, n=1000000, e=50000000, columns=400000):
    """Weighted per-column sampling (`_CAPI_SamplingProbs` on a column slice with fp32 weights),
    with the per-kernel times of the library's launch accounting.  A profiling shape."""
    dev = torch.device("cuda")
    indptr, indices = synth.powerlaw_csc(n, e, exponent=2.1, max_degree=20000, seed=2024, device=dev)
    nnz = int(indptr[-1])
    A = gs.Graph(n, n)
    A._CAPI_LoadCSC(indptr, indices)
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    probs = torch.rand(nnz, generator=gen, device=dev) + 0.01
    seeds = torch.randint(0, n, (columns,), generator=gen, device=dev)
    sub, sel = A._CAPI_Slicing(seeds, 1, gs._CSC, gs._CSC)
    w = probs[sel]
    out = {}
    for K in (10, 5):
        fn = lambda: sub._CAPI_SamplingProbs(1, w, K, False, gs._CSC, gs._COO)  # noqa: E731
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        pipeline.timing_enable(True)
        for _ in range(steps):
            fn()
        timed = pipeline.timing_collect()
        pipeline.timing_enable(False)
        out["K=%d" % K] = {"ms_per_call": e0.elapsed_time(e1) / steps,
                           "kernels_ms": {name: round(ms / cnt, 4) for name, _, ms, cnt in timed}}
    print(json.dumps({"metric": "weighted_sampling_ms", "config": {"workload": "%d columns of %d nodes / %d edges"
                                                                   % (columns, n, nnz)}, **out}))


def gather(steps=10, warmup=3, rows=4000000, width=100):
    """Feature fetch for a sampled frontier: random rows of a [2 449 029, 100] fp32 table."""
    dev = torch.device("cuda")
    n = 2449029
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    feat = torch.rand(n, width, generator=g, device=dev)
    idx = torch.randint(0, n, (rows,), generator=g, device=dev)
    out = {}
    for name, src in (("device", feat), ("pinned_host", feat[:200000].cpu().pin_memory())):
        ix = idx if name == "device" else idx[:400000] % 200000
        for _ in range(warmup):
            gs.gather_rows(src, ix)
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            o = gs.gather_rows(src, ix)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        alg = ix.numel() * (8 + 2 * width * 4)       # index + row read + row write
        out[name] = {"ms_per_call": ms, "rows": ix.numel(), "algorithmic_gbs": alg / (ms / 1e3) / 1e9,
                     "frac_of_copy_peak": alg / (ms / 1e3) / 1e9 / PEAK_GBS}
        assert torch.equal(o[:1000], src[ix[:1000].cpu()].to(dev) if name != "device" else src[ix[:1000]])
    gs.check_async_errors()
    print(json.dumps({"metric": "gather_rows_gbs", "value": out["device"]["algorithmic_gbs"], "unit": "GB/s",
                      "config": {"workload": "%d rows x %d fp32 out of %d" % (rows, width, n)}, **out}))


def cfg5(steps=6, warmup=3):
    """The full-size configuration: 111 059 956 nodes / about 3.2 G directed edges."""
    cfg5s(steps, warmup, n=111059956, e=3200000000, large=True)


def cfg5s(steps=6, warmup=3, n=11105996, e=320000000, large=False):
    dev = torch.device("cuda")
    batch, sb = 1024, 64
    t_gen = time.time()
    if large:
        indptr, indices = synth.powerlaw_csc_large(n, e, exponent=2.1, max_degree=100000, seed=9, device=dev)
    else:
        indptr, indices = synth.powerlaw_csc(n, e, exponent=2.1, max_degree=100000, seed=9, device=dev,
                                             index_dtype=torch.int32)
    torch.cuda.synchronize()
    t_gen = time.time() - t_gen
    torch.cuda.empty_cache()
    fan = [15, 10, 5]
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    seeds_all = torch.randperm(n, generator=gen, device=dev)[:batch * sb * (steps + warmup)].contiguous()
    ptr = (torch.arange(sb + 1, dtype=torch.int64) * batch).to(dev)
    probe = pipeline.GraphSAGESampler(indptr, indices, sb, batch * sb, fan)
    probe.sample(seeds_all[:batch * sb], ptr)
    caps = [(int(S * 1.2) + 4096, int(E * 1.2) + 4096) for S, E, U in probe.counts()]
    caps[0] = (batch * sb, batch * sb * fan[0])
    del probe
    torch.cuda.empty_cache()
    smp = pipeline.GraphSAGESampler(indptr, indices, sb, batch * sb, fan, capacities=caps)
    counts = torch.zeros(steps + warmup, 9, dtype=torch.int64, device=dev)
    for i in range(warmup):
        smp.sample(seeds_all[i * batch * sb:(i + 1) * batch * sb], ptr, counts_out=counts[i])
    torch.cuda.synchronize()
    smp.check()
    e0, e1 = _events()
    e0.record()
    for i in range(warmup, warmup + steps):
        smp.sample(seeds_all[i * batch * sb:(i + 1) * batch * sb], ptr, counts_out=counts[i])
    e1.record()
    torch.cuda.synchronize()
    smp.check()
    ms = e0.elapsed_time(e1)
    c = counts[warmup:].cpu().view(steps, 3, 3)
    edges = int(c[:, :, 1].sum())
    print(json.dumps({"metric": "graphsage_sampled_edges_per_sec", "value": edges / (ms / 1e3), "unit": "edges/s",
                      "ms_per_step": ms / steps, "steps": steps,
                      "config": {"workload": "GraphSAGE [15,10,5], %d x %d seeds, %d nodes / %d edges, int32 indices"
                                 % (sb, batch, n, int(indptr[-1])),
                                 "graph_gb": (indices.numel() * 4 + indptr.numel() * 8) / 1e9,
                                 "graph_build_s": t_gen,
                                 "mean_SEU_per_layer": c.double().mean(0).tolist()}}))


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "node2vec"
    t0 = time.time()
    {"ladies": ladies, "node2vec": node2vec, "cfg5s": cfg5s, "cfg5": cfg5, "gather": gather,
     "limits": limits, "weighted": weighted}[which]()
    print("# %s finished in %.1f s" % (which, time.time() - t0), file=sys.stderr)
