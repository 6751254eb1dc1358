#!/usr/bin/env python
"""Benchmark of the sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--reps R] [--impl ours|reference]
                    [--workload cfg2|cfg3|cfg4|cfg5|medium|small]

Workloads (seeded synthetic graphs with the shapes of the benchmark configurations):

cfg2 (default)  3-layer GraphSAGE sampler, fanouts [15, 10, 5], uniform without replacement,
                minibatch 1024, 32 minibatches per step, power-law graph 2 449 029 nodes /
                123 718 280 directed edges (CSC int64 / int64), one epoch over 196 615 seeds.
                One step = one super-batch through all layers (fused slice + sample, then
                per-minibatch unique / relabel = block construction).  Every rank samples its
                own epoch (weak scaling).
cfg5            the same sampler at scale: 64 minibatches per step, 111 059 956 nodes / about
                3.2 G directed edges, int32 indices (13.7 GB per GPU); 1 207 179 seeds split
                evenly over the ranks (strong scaling).
cfg3            2-layer LADIES layer-wise sampler, 4000 nodes per layer, 512 seeds, 232 965
                nodes / 114 615 892 fp32-weighted edges.  One step = both layers.
cfg4            node2vec walks, 1 000 000 walkers x 80 steps, p = 2, q = 0.5, on the cfg2 graph.
                One step = one call producing the [81 x 1 000 000] trace.
medium / small  reduced GraphSAGE shapes for profiling and functional runs.

Prints ONE JSON line.  The timed region (K steps between two synchronised CUDA events, barrier on
both sides, max over ranks) is repeated R times; ``ms_per_step`` / ``value`` are the median
repetition, the spread is reported beside them.  ``value`` has its inputs resident in HBM and
pre-allocated outputs; ``e2e`` goes through the public Python API with the step's inputs coming
from pinned host memory and its result sizes read back.  ``--impl reference`` times the CPU port
of the reference's algorithms (oracle/) on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import gc
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "cfg2": dict(kind="sage", nodes=2449029, edges=123718280, train=196615, fanouts=[15, 10, 5], batch=1024,
                 super_batch=32, index_dtype="int64", max_degree=20000, scaling="weak", graph_seed=2024, streams=4),
    "cfg5": dict(kind="sage", nodes=111059956, edges=3200000000, train=1207179, fanouts=[15, 10, 5], batch=1024,
                 super_batch=64, index_dtype="int32", max_degree=100000, scaling="strong", graph_seed=9, large=True),
    # profiling shape: graph larger than L2, a few GB on the device, short kernels
    "medium": dict(kind="sage", nodes=1000000, edges=50000000, train=65536, fanouts=[15, 10, 5], batch=1024,
                   super_batch=16, index_dtype="int64", max_degree=20000, scaling="weak", graph_seed=2024),
    "small": dict(kind="sage", nodes=200000, edges=8000000, train=20480, fanouts=[15, 10, 5], batch=1024,
                  super_batch=8, index_dtype="int64", max_degree=5000, scaling="weak", graph_seed=2024),
    "cfg3": dict(kind="ladies", nodes=232965, edges=114615892, seeds=512, layer_nodes=4000, layers=2,
                 index_dtype="int64", max_degree=30000, scaling="weak", graph_seed=11),
    "cfg4": dict(kind="walk", nodes=2449029, edges=123718280, walkers=1000000, length=80, p=2.0, q=0.5,
                 index_dtype="int64", max_degree=20000, scaling="weak", graph_seed=2024),
}

# DRAM bytes (read + write) per sampled edge, from the `ncu --set full` capture of the "medium"
# case summarised under profiles/; the access pattern per unit is the same on the bench
# workload, so the traffic is scaled by the units of a launch / a step.
NCU_DRAM_BYTES_PER_EDGE = {"sample_tile": 75.6}
NCU_PATH_DRAM_BYTES_PER_EDGE = 119.3


# ----------------------------------------------------------------------------- helpers
def load_plain(name):
    """gsampler_b200/<name>.py loaded as a plain file (synth, shard: they need numpy and torch only):
    the reference arm must not load this repository's native libraries, which importing the package
    would do."""
    spec = importlib.util.spec_from_file_location("gsb_%s_standalone" % name, os.path.join(ROOT, "gsampler_b200", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_synth():
    return load_plain("synth")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_graph(cfg, device, synth):
    import torch

    if cfg.get("large"):
        return synth.powerlaw_csc_large(cfg["nodes"], cfg["edges"], exponent=2.1, max_degree=cfg["max_degree"],
                                        seed=cfg["graph_seed"], device=device)
    dt = torch.int32 if cfg["index_dtype"] == "int32" else torch.int64
    return synth.powerlaw_csc(cfg["nodes"], cfg["edges"], exponent=2.1, max_degree=cfg["max_degree"],
                              seed=cfg["graph_seed"], device=device, index_dtype=dt)


def sage_seed_list(cfg, rank, world, shard):
    """This rank's training seeds: its own epoch for a weak-scaling workload, its shard of the one
    global seed list (``shard`` = the gsampler_b200.shard module) for a strong-scaling one."""
    import torch

    g = torch.Generator()
    if cfg["scaling"] == "strong":
        g.manual_seed(7)
        seeds = torch.randperm(cfg["nodes"], generator=g)[:cfg["train"]].to(torch.int64)
        return shard.shard_seeds(seeds, rank, world).contiguous()
    g.manual_seed(7 + rank)
    return torch.randperm(cfg["nodes"], generator=g)[:cfg["train"]].to(torch.int64)


def sage_bytes(S, E, U, w_idx=8):
    """Compulsory bytes of one GraphSAGE layer: fused slice + sample reads 8S seeds + 16S offsets +
    w_idx * E gathered ids and writes 8(S+1) + 24E; unique / relabel reads 8S + 16E and writes
    8U + 16E."""
    return 8 * S + 16 * S + w_idx * E + 8 * (S + 1) + 24 * E, 8 * S + 16 * E + 8 * U + 16 * E


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        super().__init__(daemon=True)
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                self.rows.append([x.strip() for x in line.split(",")])
        except Exception:
            pass

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        self.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU side (oracle port)
def cpu_threads():
    """All host cores for the OpenMP port (a launcher such as torchrun pins OMP_NUM_THREADS to 1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(n)
    os.environ["GS_ORACLE_THREADS"] = str(n)  # read by the oracle when it loads: OpenMP may be initialised already
    return n


def cpu_sage(cfg, indptr_np, indices_np, steps, warmup, minibatches):
    """The CPU port (reference reservoir sampler + batch relabel) on `minibatches` minibatches per
    step.  Returns (edges/s, sample description, threads, ms per step)."""
    from oracle import gs_oracle

    gs_oracle.build()
    rng = np.random.default_rng(7)
    n = cfg["batch"] * minibatches
    ptr = np.arange(minibatches + 1, dtype=np.int64) * cfg["batch"]
    total_edges, total_t = 0, 0.0
    for i in range(warmup + steps):
        seeds = rng.permutation(cfg["nodes"])[:n].astype(np.int64)
        t0 = time.perf_counter()
        layers = gs_oracle.graphsage_batch(indptr_np, indices_np, seeds, ptr, cfg["fanouts"], seed=i, sampler="ref")
        dt = time.perf_counter() - t0
        if i >= warmup:
            total_t += dt
            total_edges += sum(int(L["rows"].size) for L in layers)
    desc = "%d steps x %d minibatches of %d seeds, %d layers, oracle reference-sampler + batch relabel" % (
        steps, minibatches, cfg["batch"], len(cfg["fanouts"]))
    return total_edges / total_t, desc, gs_oracle.num_threads(), total_t / steps * 1e3


def cpu_cfg1():
    """The CPU baseline protocol on configuration 1: R-MAT 100 000 nodes / 2 000 000 edges (seed 42,
    self-loops, no duplicates), 2 layers [25, 10], 20 minibatches x 1024 seeds of a seed-0
    permutation; one warm-up, best of 5."""
    from oracle import gs_oracle

    synth = load_synth()
    gs_oracle.build()
    indptr, indices = synth.rmat_csc(100000, 2000000, seed=42)
    seeds = np.random.default_rng(0).permutation(100000)[:20 * 1024].astype(np.int64)
    ptr = np.arange(21, dtype=np.int64) * 1024
    best, edges = None, 0
    for i in range(6):
        t0 = time.perf_counter()
        layers = gs_oracle.graphsage_batch(indptr, indices, seeds, ptr, [25, 10], seed=i, sampler="ref")
        dt = time.perf_counter() - t0
        edges = sum(int(L["rows"].size) for L in layers)
        if i >= 1:
            best = dt if best is None else min(best, dt)
    S = [int(L["sub_indptr"].size - 1) for L in layers]
    E = [int(L["rows"].size) for L in layers]
    U = [int(L["unique"].size) for L in layers]
    alg = sum(sum(sage_bytes(s, e, u)) for s, e, u in zip(S, E, U))
    return {"value": edges / best, "unit": "edges/s", "cores": gs_oracle.num_threads(), "kind": "port",
            "sample": "cfg1: R-MAT 100000 nodes / %d edges, fanouts [25, 10], 20 x 1024 seeds, 1 warm-up + best of 5"
                      % int(indptr[-1]), "seconds": best, "algorithmic_gbs": alg / best / 1e9}


def cpu_sort_indices(indptr_np, indices_np, max_edges=20_000_000):
    """The one CPU routine the reference owns on this path -- SortIndicesCPU, an OpenMP parallel
    for over columns with a qsort each (src/cpu/sort_indices.cc:27-48 in gSampler, the node2vec
    preprocessing of a graph kept in host memory) -- timed as restated in oracle/ on the leading
    columns of the bench graph with their row ids shuffled."""
    from oracle import gs_oracle

    ncols = max(int(np.searchsorted(indptr_np, max_edges, side="right")) - 1, 1)
    ip = np.ascontiguousarray(indptr_np[:ncols + 1])
    idx = np.random.default_rng(11).permutation(indices_np[:ip[-1]])
    t0 = time.perf_counter()
    out = gs_oracle.sort_indices(ip, idx)
    dt = time.perf_counter() - t0
    assert out.size == idx.size
    return {"what": "SortIndicesCPU algorithm (per-column qsort under OpenMP)", "columns": ncols,
            "edges": int(ip[-1]), "seconds": dt, "edges_per_sec": float(ip[-1]) / dt, "cores": gs_oracle.num_threads()}


def cpu_ladies(cfg, indptr, indices, w, steps, warmup):
    """LADIES layers composed from the oracle's operators (column slice, row sums of w^2, weighted
    list sampling, row slice, the two renormalisations, relabel)."""
    from oracle import gs_oracle as o

    o.build()
    n, K = cfg["nodes"], cfg["layer_nodes"]
    rng = np.random.default_rng(1)
    edges, total = 0, 0.0
    for i in range(warmup + steps):
        seeds = rng.permutation(n)[:cfg["seeds"]].astype(np.int64)
        t0 = time.perf_counter()
        step_edges = 0
        for l in range(cfg["layers"]):
            sip, srows, scols, ssel = o.slice_cols(indptr, indices, seeds)
            p = o.edge_sum(srows, scols, w[ssel], 0, n, square=True)
            sel = o.list_sample_probs_spec(p, K, seed=i, stream=l)
            csr_ip, csr_cols, perm = o.coo2csc(srows, scols, n)
            rip, rcols, rloc, rsel = o.slice_cols(csr_ip, csr_cols, sel)
            ew = w[ssel][perm][rsel]
            w1 = o.edge_op_node(rloc, ew, p[sel], "div")
            colsum = o.edge_sum(rloc, rcols, w1, 2, seeds.size)
            o.edge_op_node(rcols, w1, colsum, "div")
            frontier, _, _ = o.relabel(seeds, sel[rloc], rcols)
            step_edges += rloc.size
            seeds = frontier
        dt = time.perf_counter() - t0
        if i >= warmup:
            total += dt
            edges += step_edges
    return edges / total, "%d steps of the %d-layer LADIES recipe composed from the oracle's operators" % (
        steps, cfg["layers"]), o.num_threads(), total / steps * 1e3


def cpu_walk(cfg, indptr, indices, steps, warmup, walkers):
    from oracle import gs_oracle as o

    o.build()
    rng = np.random.default_rng(7)
    live, total = 0, 0.0
    for i in range(warmup + steps):
        seeds = rng.integers(0, cfg["nodes"], walkers).astype(np.int64)
        t0 = time.perf_counter()
        tr = o.node2vec_spec(indptr, indices, seeds, cfg["length"], cfg["p"], cfg["q"], seed=i)
        dt = time.perf_counter() - t0
        if i >= warmup:
            total += dt
            live += int((np.asarray(tr).reshape(cfg["length"] + 1, walkers)[1:] >= 0).sum())
    return live / total, "%d calls of %d walkers x %d steps (oracle node2vec)" % (steps, walkers, cfg["length"]), \
        o.num_threads(), total / steps * 1e3


def reference_gpu_sage(cfg, indptr, indices, batches, steps, warmup):
    """The reference's own CUDA kernels (oracle/_ref/gs_ref.so, built from the reference tree by
    oracle/build_ref.py) on the same super-batches on this GPU: per layer
    FusedCSCColSlicingSamplingCUDA, edge_ptr = sub_indptr[seeds_ptr], BatchCOORelabelCUDA once
    (the reference's Python pipeline runs the relabel twice per layer).  None when the file has
    not been built or the graph is beyond its int64 / 2^31 limits."""
    import torch

    from oracle import build_ref

    ref = build_ref.load()
    if ref is None or not indptr.is_cuda or indices.numel() >= 2 ** 31:
        return None
    indices = indices.to(torch.int64)
    batches = [(s.to(indptr.device), p.to(indptr.device)) for s, p in batches]

    def step(seeds, ptr):
        edges = 0
        for K in cfg["fanouts"]:
            sub_indptr, col, rows, _ = ref.fused_slice_sample(indptr, indices, K, seeds, False, True)
            uq, up, _, _, _ = ref.batch_coo_relabel(seeds, ptr, seeds[col], rows, sub_indptr[ptr])
            edges += rows.numel()
            seeds, ptr = uq, up
        return edges

    for i in range(warmup):
        step(*batches[i % len(batches)])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    edges = 0
    for i in range(steps):
        edges += step(*batches[(warmup + i) % len(batches)])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    return {"value": edges / (ms / 1e3), "unit": "edges/s", "ms_per_step": ms / steps, "steps": steps,
            "what": "the reference's CUDA kernels compiled unmodified for sm_100a, one relabel per layer, "
                    "device-resident inputs, CUDA-event time"}


def run_reference(args, cfg, rank, world):
    """The reference arm: rank 0 alone, all host cores, the workload's own graph, seeds and step
    shape; this repository's native libraries are not loaded."""
    if rank != 0:
        return
    import torch

    threads = cpu_threads()
    synth = load_synth()
    device = "cuda" if torch.cuda.is_available() else "cpu"
    indptr, indices = make_graph(cfg, device, synth)
    extra = {}
    if cfg["kind"] == "sage":
        ref_gpu = None
        if device == "cuda":
            shard = load_plain("shard")
            batches = shard.super_batches(sage_seed_list(cfg, 0, 1, shard), cfg["batch"], cfg["super_batch"])
            ref_gpu = reference_gpu_sage(cfg, indptr, indices, batches, args.steps, args.warmup)
        indptr_np, indices_np = indptr.cpu().numpy(), indices.cpu().numpy().astype(np.int64)
        del indptr, indices
        # the arm's own step shape (super_batch minibatches per step); at most 32 so that a run of
        # K + W steps stays within minutes on the largest workload
        eps, desc, cores, ms = cpu_sage(cfg, indptr_np, indices_np, args.steps, args.warmup,
                                        min(cfg["super_batch"], 32))
        metric, unit = "graphsage_sampled_edges_per_sec", "edges/s"
        if ref_gpu is not None:
            extra["reference_gpu"] = ref_gpu
    elif cfg["kind"] == "ladies":
        g = torch.Generator(device=device)
        g.manual_seed(5)
        w = torch.rand(indices.numel(), generator=g, device=device).clamp_min_(1e-3).cpu().numpy()
        eps, desc, cores, ms = cpu_ladies(cfg, indptr.cpu().numpy(), indices.cpu().numpy().astype(np.int64), w,
                                          args.steps, args.warmup)
        metric, unit = "ladies_block_edges_per_sec", "edges/s"
    else:
        eps, desc, cores, ms = cpu_walk(cfg, indptr.cpu().numpy(), indices.cpu().numpy().astype(np.int64),
                                        args.steps, args.warmup, walkers=cfg["walkers"] // 10)
        metric, unit = "walk_steps_per_sec", "steps/s"
    line = {
        "impl": "reference", "metric": metric, "value": eps, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": cfg["scaling"], "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": {"workload": args.workload, **{k: v for k, v in cfg.items() if k not in ("kind", "large")},
                   "note": "the reference has no CPU sampler; this is the CPU port of its algorithms (oracle/) "
                           "on all host cores of rank 0's machine, %d threads" % threads},
        "cpu_baseline": {"value": eps, "unit": unit, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": eps, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    line.update(extra)
    print(json.dumps(line))


# ----------------------------------------------------------------------------- workloads (GPU arm)
class SageWorkload(object):
    metric, unit = "graphsage_sampled_edges_per_sec", "edges/s"

    def __init__(self, cfg, dev, rank, world, nstreams):
        import torch

        import gsampler_b200 as gs
        from gsampler_b200 import pipeline, shard, synth

        self.cfg, self.dev, self.gs, self.pipeline, self.torch = cfg, dev, gs, pipeline, torch
        self.L = len(cfg["fanouts"])
        t0 = time.time()
        self.indptr, self.indices = make_graph(cfg, dev, synth)
        torch.cuda.synchronize()
        self.graph_build_s = time.time() - t0
        torch.cuda.empty_cache()
        seeds = sage_seed_list(cfg, rank, world, shard)
        self.batches_host = shard.super_batches(seeds, cfg["batch"], cfg["super_batch"])
        self.batches_dev = [(s.to(dev), p.to(dev)) for s, p in self.batches_host]
        self.batches_pin = [(s.pin_memory(), p.pin_memory()) for s, p in self.batches_host]
        self.nb = len(self.batches_dev)
        max_seeds = cfg["batch"] * cfg["super_batch"]
        # capacities from a measured dry run (the worst case would be ~4x larger); an overflow
        # raises the sampler's error word, which is checked after every timed region
        probe = pipeline.GraphSAGESampler(self.indptr, self.indices, cfg["super_batch"], max_seeds, cfg["fanouts"])
        caps = None
        for s, p in self.batches_dev[:8]:
            probe.sample(s, p)
            cur = [(int(S * 1.15) + 4096, int(E * 1.15) + 4096) for S, E, U in probe.counts()]
            caps = cur if caps is None else [(max(a[0], b[0]), max(a[1], b[1])) for a, b in zip(caps, cur)]
        caps[0] = (max_seeds, max_seeds * cfg["fanouts"][0])
        del probe
        torch.cuda.empty_cache()
        # Super-batches are independent: `nstreams` of them are in flight at once, each with its own
        # pre-allocated sampler on its own CUDA stream, so that the latency-bound relabel passes of
        # one overlap the bandwidth-bound sampling pass of another.
        self.nstreams = nstreams
        self.samplers = [pipeline.GraphSAGESampler(self.indptr, self.indices, cfg["super_batch"], max_seeds,
                                                   cfg["fanouts"], capacities=caps) for _ in range(nstreams)]
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(nstreams)]
        self.counts = None

    def alloc_counts(self, n):
        self.counts = self.torch.zeros(n, 3 * self.L, dtype=self.torch.int64, device=self.dev)

    def step(self, i, row, overlapped=True):
        s, p = self.batches_dev[i % self.nb]
        if not overlapped:
            self.samplers[0].sample(s, p, counts_out=self.counts[row])
            return
        k = i % self.nstreams
        with self.torch.cuda.stream(self.streams[k]):
            self.samplers[k].sample(s, p, counts_out=self.counts[row])

    def fork(self):
        cur = self.torch.cuda.current_stream(self.dev)
        for st in self.streams:
            st.wait_stream(cur)

    def join(self):
        cur = self.torch.cuda.current_stream(self.dev)
        for st in self.streams:
            cur.wait_stream(st)

    def check(self):
        for sm in self.samplers:
            sm.check()

    def units(self, rows):
        c = self.counts[rows].cpu().numpy().reshape(-1, self.L, 3)
        return int(c[:, :, 1].sum()), c

    def e2e_setup(self):
        gs, cfg = self.gs, self.cfg
        A = gs.Graph(cfg["nodes"], cfg["nodes"])
        A._CAPI_LoadCSC(self.indptr, self.indices)
        self.bm = gs.BatchMatrix()
        self.bm.load_from_matrix(gs.Matrix(A), False)
        self.e2e_streams = [self.torch.cuda.Stream(self.dev) for _ in range(self.nstreams)]

    def e2e_run(self, first, count):
        """Like a data loader with a prefetch depth of `streams`: the next super-batches are copied in
        and enqueued (each on its own stream) before the host waits for the sizes of the oldest one
        in flight.  Every step copies its own seeds from pinned host memory and reads its own result
        sizes back."""
        torch, L = self.torch, self.L
        depth = len(self.e2e_streams)
        edges, nin, nout, pending = 0, 0, 0, []
        for k in range(count + depth - 1):
            if k < count:
                s, p = self.batches_pin[(first + k) % self.nb]
                with torch.cuda.stream(self.e2e_streams[k % depth]):
                    sd, pd = s.to(self.dev, non_blocking=True), p.to(self.dev, non_blocking=True)
                    pending.append((self.bm.graphsage_async(sd, pd, self.cfg["fanouts"]), s.numel() * 8 + p.numel() * 8))
            if k >= depth - 1 and pending:
                fut, nbytes = pending.pop(0)
                cnt = fut.wait()[-1]
                edges += int(cnt.view(L, 3)[:, 1].sum())
                nin += nbytes
                nout += (3 * L + 1) * 8
        return edges, nin, nout

    e2e_api = "BatchMatrix.graphsage_async (one native call per super-batch, as many in flight as `streams`)"

    def describe(self, c_host, world):
        cfg = self.cfg
        return {"graph": "power-law, %d nodes, %d directed edges, CSC int64/%s" % (
                    cfg["nodes"], int(self.indptr[-1]), cfg["index_dtype"]),
                "graph_gb": (self.indices.numel() * self.indices.element_size() + self.indptr.numel() * 8) / 1e9,
                "graph_build_s": round(self.graph_build_s, 2),
                "fanouts": cfg["fanouts"], "batch": cfg["batch"], "super_batch": cfg["super_batch"],
                "train_seeds": cfg["train"], "seeds_this_rank": int(sum(s.numel() for s, _ in self.batches_host)),
                "super_batches_per_epoch_this_rank": self.nb,
                "parallelism": ("replica x%d, own epoch per rank" if cfg["scaling"] == "weak" else
                                "replica x%d, one seed list split by gsampler_b200.shard.shard_seeds") % world,
                "l2": "inputs_larger_than_l2 (graph indices %.1f GB)" % (
                    self.indices.numel() * self.indices.element_size() / 1e9),
                "mean_SEU_per_layer": [[float(c_host[:, l, j].mean()) for j in range(3)] for l in range(self.L)],
                "capacities": "measured x1.15", "streams": self.nstreams,
                "row_ids_read_from": ("a 32-bit copy made when the sampler is built (inputs and outputs stay int64)"
                                      if cfg["index_dtype"] == "int64" else "the int32 array itself")}

    def roofline(self, timed, c_host, elapsed_s, steps, peak, peak_kind):
        w_idx = 4 if self.cfg["index_dtype"] == "int32" else 8
        by = {(name, tag): (ms, cnt) for name, tag, ms, cnt in timed}
        total_ms = sum(v[0] for v in by.values())
        (dname, dtag), (dms, dcnt) = max(by.items(), key=lambda kv: kv[1][0])
        S, E, U = (c_host[:, dtag, j].astype(np.float64) for j in range(3))
        per_launch = {
            # the sampling kernel also writes the block's column ids (8E): 32E written, not 24E
            "sample_tile": (8 * S + 16 * S + w_idx * E + 8 * (S + 1) + 32 * E).mean(),
            "relabel_pcount": (8 * (S + E)).mean(), "relabel_scatter": (8 * (S + E)).mean(),
            "relabel_dedupe": (8 * (S + E)).mean(), "relabel_mark": (4 * (S + E)).mean(),
            # one pass over the items: min_idx (4) and the ids of first occurrences (8U) in, node
            # list (8U) and relabelled rows (8E) out
            "relabel_emit": (4 * (S + E) + 16 * U + 8 * E).mean(),
        }.get(dname, 0.0)
        dur_s = dms / dcnt / 1e3
        achieved = per_launch / dur_s / 1e9 if dur_s > 0 else 0.0
        path_bytes = 0.0
        for l in range(self.L):
            f, b = sage_bytes(c_host[:, l, 0].sum(), c_host[:, l, 1].sum(), c_host[:, l, 2].sum(), w_idx)
            path_bytes += f + b
        path_gbs = path_bytes / elapsed_s / 1e9
        edges = float(c_host[:, :, 1].sum())
        per = NCU_DRAM_BYTES_PER_EDGE.get(dname)
        roof = {"bound": "hbm", "kernel": "%s[layer %d]" % (dname, dtag), "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "traffic": None if per is None else per * float(E.mean()),
                "peak_kind": peak_kind, "share_of_kernel_time": dms / total_ms, "avg_launch_ms": dms / dcnt,
                "algorithmic_bytes_per_launch": per_launch}
        path = {"algorithmic_gb_per_step": path_bytes / steps / 1e9, "achieved": path_gbs, "unit": "GB/s",
                "frac": path_gbs / peak, "peak_kind": peak_kind,
                "dram_traffic_gbs": NCU_PATH_DRAM_BYTES_PER_EDGE * edges / elapsed_s / 1e9,
                "dram_traffic_frac": NCU_PATH_DRAM_BYTES_PER_EDGE * edges / elapsed_s / 1e9 / peak}
        return roof, path

    def cpu_baseline(self):
        indptr_np = self.indptr.cpu().numpy()
        indices_np = self.indices.cpu().numpy().astype(np.int64)
        eps, desc, cores, _ = cpu_sage(self.cfg, indptr_np, indices_np, steps=3, warmup=1, minibatches=4)
        return {"value": eps, "unit": "edges/s", "cores": cores, "kind": "port", "sample": desc,
                "reference_cpu_code": cpu_sort_indices(indptr_np, indices_np)}


class LadiesWorkload(object):
    metric, unit = "ladies_block_edges_per_sec", "edges/s"

    def __init__(self, cfg, dev, rank, world, nstreams):
        import torch

        import gsampler_b200 as gs
        from gsampler_b200 import pipeline, synth

        self.cfg, self.dev, self.gs, self.pipeline, self.torch = cfg, dev, gs, pipeline, torch
        t0 = time.time()
        self.indptr, self.indices = make_graph(cfg, dev, synth)
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        self.w = torch.rand(self.indices.numel(), generator=g, device=dev).clamp_min_(1e-3)
        torch.cuda.synchronize()
        self.graph_build_s = time.time() - t0
        A = gs.Graph(cfg["nodes"], cfg["nodes"])
        A._CAPI_LoadCSC(self.indptr, self.indices)
        m = gs.Matrix(A)
        m.edata["w"] = self.w
        # column-normalise once (the preprocessing P = A D^-1 of the recipe, outside the loop)
        self.m = m.div("w", m.sum("w", axis=0).clamp_min(1e-12), axis=0)
        gen = torch.Generator()
        gen.manual_seed(1 + rank)
        self.batches_host = [torch.randperm(cfg["nodes"], generator=gen)[:cfg["seeds"]].to(torch.int64)
                             for _ in range(16)]
        self.batches_dev = [s.to(dev) for s in self.batches_host]
        self.batches_pin = [s.pin_memory() for s in self.batches_host]
        self.nb = len(self.batches_dev)
        self.nstreams = 1
        self.stats = []

    def alloc_counts(self, n):
        self.stats = [None] * n

    def _sample(self, seeds):
        """Both layers; returns [(slice edges, candidate rows, block edges, seeds)] per layer."""
        out = []
        for _ in range(self.cfg["layers"]):
            S = seeds.numel()
            blk, seeds, picked = self.m.ladies_layer(seeds, self.cfg["layer_nodes"])
            out.append((S, blk.num_edges(), int(seeds.numel())))
        return out

    def step(self, i, row, overlapped=True):
        self.stats[row] = self._sample(self.batches_dev[i % self.nb])

    def fork(self):
        pass

    def join(self):
        pass

    def check(self):
        self.gs.check_async_errors()

    def units(self, rows):
        sel = [self.stats[r] for r in (range(*rows.indices(len(self.stats))) if isinstance(rows, slice) else rows)]
        return sum(e for st in sel for _, e, _ in st), sel

    def e2e_setup(self):
        pass

    def e2e_run(self, first, count):
        edges, nin, nout = 0, 0, 0
        for k in range(count):
            s = self.batches_pin[(first + k) % self.nb]
            st = self._sample(s.to(self.dev, non_blocking=True))     # block sizes are read back per layer
            edges += sum(e for _, e, _ in st)
            nin += s.numel() * 8
            nout += 2 * 8 * self.cfg["layers"]
        return edges, nin, nout

    e2e_api = "Matrix.ladies_layer (one native call per layer; two size read-backs per layer)"

    def describe(self, sel, world):
        cfg = self.cfg
        return {"graph": "power-law, %d nodes, %d directed fp32-weighted edges, CSC int64/int64" % (
                    cfg["nodes"], int(self.indptr[-1])),
                "graph_build_s": round(self.graph_build_s, 2), "seeds": cfg["seeds"], "layer_nodes": cfg["layer_nodes"],
                "layers": cfg["layers"], "parallelism": "replica x%d" % world,
                "l2": "inputs_larger_than_l2 (indices + weights %.1f GB)" % (self.indices.numel() * 12 / 1e9),
                "mean_block_edges_per_step": float(np.mean([sum(e for _, e, _ in st) for st in sel]))}

    def roofline(self, timed, sel, elapsed_s, steps, peak, peak_kind):
        """Compulsory bytes of a layer with S seeds, E_s sliced edges, R rows, K picks, E kept edges:
        slice 8S + 16S + 8E_s + 8(S+1) + 24E_s; row sums of w^2: 4E_s + 8E_s + 4R; weighted list
        sampling 4R + 8K; row filter 8E_s + 24E; two renormalisations 2(4E + 8E + 4E) and the column
        sums 4E + 8E + 4S; relabel 8S + 16E + 8U + 16E.  E_s is not read back by the native call: the
        mean column degree times S stands in for it."""
        by = {}
        for name, tag, ms, cnt in timed:
            a = by.setdefault(name, [0.0, 0])
            a[0] += ms
            a[1] += cnt
        total_ms = sum(v[0] for v in by.values())
        dname, (dms, dcnt) = max(by.items(), key=lambda kv: kv[1][0])
        R, K = self.cfg["nodes"], self.cfg["layer_nodes"]
        deg = float(self.indptr[-1]) / self.cfg["nodes"]
        path = 0.0
        for st in sel:
            for S, E, U in st:
                Es = S * deg
                path += (40 * S + 32 * Es) + (12 * Es + 4 * R) + (4 * R + 8 * K) + (8 * Es + 24 * E) + \
                        (32 * E + 12 * E + 4 * S) + (8 * S + 32 * E + 8 * U)
        gbs = path / elapsed_s / 1e9
        roof = {"bound": "hbm", "kernel": dname, "achieved": None, "peak": peak, "unit": "GB/s", "frac": None,
                "traffic": None, "peak_kind": peak_kind, "share_of_kernel_time": dms / total_ms,
                "avg_launch_ms": dms / dcnt,
                "note": "per-kernel bytes are not separated for this workload; see roofline_path"}
        return roof, {"algorithmic_gb_per_step": path / steps / 1e9, "achieved": gbs, "unit": "GB/s",
                      "frac": gbs / peak, "peak_kind": peak_kind,
                      "kernel_ms_per_step": total_ms / steps}

    def cpu_baseline(self):
        eps, desc, cores, _ = cpu_ladies(self.cfg, self.indptr.cpu().numpy(), self.indices.cpu().numpy(),
                                         self.w.cpu().numpy(), steps=2, warmup=1)
        return {"value": eps, "unit": "edges/s", "cores": cores, "kind": "port", "sample": desc}


class WalkWorkload(object):
    metric, unit = "walk_steps_per_sec", "steps/s"

    def __init__(self, cfg, dev, rank, world, nstreams):
        import torch

        import gsampler_b200 as gs
        from gsampler_b200 import pipeline, synth

        self.cfg, self.dev, self.gs, self.pipeline, self.torch = cfg, dev, gs, pipeline, torch
        t0 = time.time()
        self.indptr, self.indices = make_graph(cfg, dev, synth)
        torch.cuda.synchronize()
        self.graph_build_s = time.time() - t0
        self.A = gs.Graph(cfg["nodes"], cfg["nodes"])
        self.A._CAPI_LoadCSC(self.indptr, self.indices)   # the generator's columns are sorted
        gen = torch.Generator()
        gen.manual_seed(7 + rank)
        self.batches_host = [torch.randint(0, cfg["nodes"], (cfg["walkers"],), generator=gen) for _ in range(4)]
        self.batches_dev = [s.to(dev) for s in self.batches_host]
        self.batches_pin = [s.pin_memory() for s in self.batches_host]
        self.nb = 4
        self.nstreams = 1
        # Steps actually taken per call.  The graph is symmetric, so a walk only fails to move when
        # its start node has no neighbour at all: walkers with a neighbour x length, known before
        # the walk and checked against a real trace here.
        deg = self.indptr[1:] - self.indptr[:-1]
        self.batch_live = [int((deg[s] > 0).sum()) * cfg["length"] for s in self.batches_dev]
        tr = self._walk(self.batches_dev[0])
        assert int((tr.view(-1)[cfg["walkers"]:] >= 0).sum()) == self.batch_live[0]
        del tr
        self.live = None

    def alloc_counts(self, n):
        self.live = np.zeros(n, dtype=np.int64)

    def _walk(self, seeds, row=None):
        c = self.cfg
        return self.A._CAPI_Node2Vec(seeds, c["length"], c["p"], c["q"])

    def step(self, i, row, overlapped=True):
        self._walk(self.batches_dev[i % self.nb])
        self.live[row] = self.batch_live[i % self.nb]

    def fork(self):
        pass

    def join(self):
        pass

    def check(self):
        self.gs.check_async_errors()

    def units(self, rows):
        v = self.live[rows]
        return int(v.sum()), v

    def e2e_setup(self):
        pass

    def e2e_run(self, first, count):
        live, nin, nout = 0, 0, 0
        for k in range(count):
            s = self.batches_pin[(first + k) % self.nb]
            tr = self._walk(s.to(self.dev, non_blocking=True))
            live += int((tr.view(-1)[self.cfg["walkers"]:] >= 0).sum())     # the step's result summary
            nin += s.numel() * 8
            nout += 8
        return live, nin, nout

    e2e_api = "Graph._CAPI_Node2Vec (the trace stays on the device; the count of taken steps is read back)"

    def describe(self, v, world):
        cfg = self.cfg
        return {"graph": "power-law, %d nodes, %d directed edges, sorted columns, CSC int64/int64" % (
                    cfg["nodes"], int(self.indptr[-1])),
                "graph_build_s": round(self.graph_build_s, 2), "walkers": cfg["walkers"], "length": cfg["length"],
                "p": cfg["p"], "q": cfg["q"], "parallelism": "replica x%d" % world,
                "l2": "inputs_larger_than_l2 (graph indices %.1f GB)" % (self.indices.numel() * 8 / 1e9),
                "trace_bytes_per_step": cfg["walkers"] * (cfg["length"] + 1) * 8}

    def roofline(self, timed, v, elapsed_s, steps, peak, peak_kind):
        """Compulsory bytes per taken step: the offsets pair (16), one row id (8), the trace entry (8)."""
        by = {}
        for name, tag, ms, cnt in timed:
            a = by.setdefault(name, [0.0, 0])
            a[0] += ms
            a[1] += cnt
        total_ms = sum(x[0] for x in by.values())
        dms, dcnt = by.get("walk", (0.0, 1))
        alg_launch = float(np.mean(v)) * 32
        dur = dms / max(dcnt, 1) / 1e3
        achieved = alg_launch / dur / 1e9 if dur > 0 else 0.0
        gbs = float(np.sum(v)) * 32 / elapsed_s / 1e9
        roof = {"bound": "hbm", "kernel": "node2vec_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                "share_of_kernel_time": dms / total_ms if total_ms else None, "avg_launch_ms": dms / max(dcnt, 1),
                "algorithmic_bytes_per_launch": alg_launch}
        return roof, {"algorithmic_gb_per_step": float(np.sum(v)) * 32 / steps / 1e9, "achieved": gbs,
                      "unit": "GB/s", "frac": gbs / peak, "peak_kind": peak_kind}

    def cpu_baseline(self):
        eps, desc, cores, _ = cpu_walk(self.cfg, self.indptr.cpu().numpy(), self.indices.cpu().numpy(),
                                       steps=2, warmup=1, walkers=self.cfg["walkers"] // 10)
        return {"value": eps, "unit": "steps/s", "cores": cores, "kind": "port", "sample": desc}


KINDS = {"sage": SageWorkload, "ladies": LadiesWorkload, "walk": WalkWorkload}


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=14)
    ap.add_argument("--warmup", type=int, default=7)
    ap.add_argument("--reps", type=int, default=int(os.environ.get("GSB_REPS", "15")),
                    help="repetitions of the timed K-step region (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=os.environ.get("GSB_WORKLOAD", "cfg2"), choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--streams", type=int, default=int(os.environ.get("GSB_STREAMS", "0")),
                    help="independent super-batches in flight, each on its own CUDA stream (default: the "
                         "workload's own setting -- 4 for cfg2, 2 elsewhere: the 64-minibatch super-batches "
                         "of cfg5 run slower with 4 in flight, 2.75 against 2.58 ms per step)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU fallback "
                         "(use --impl reference for the CPU port)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    json_fd = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL writes its version banner to stdout when the first communicator is made: until the
        # result line is printed, file descriptor 1 points at stderr, so that stdout carries the
        # one JSON line and nothing else
        sys.stdout.flush()
        json_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)

    from gsampler_b200 import pipeline

    wl = KINDS[cfg["kind"]](cfg, dev, rank, world, args.streams if args.streams > 0 else cfg.get("streams", 2))
    K, W, R = args.steps, args.warmup, max(1, args.reps)
    wl.alloc_counts(W + K * R + K)

    wl.fork()
    for w in range(W):
        wl.step(w, w)
    wl.join()
    torch.cuda.synchronize()
    wl.check()

    clocks = ClockSampler(local_rank)
    clocks.start()
    time.sleep(0.3)
    launches0 = pipeline.kernel_launches()
    rep_ms = []
    for r in range(R):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        wl.fork()
        for k in range(K):
            wl.step(W + r * K + k, W + r * K + k)
        wl.join()
        ev1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        rep_ms.append(ev0.elapsed_time(ev1))
    launches = (pipeline.kernel_launches() - launches0) // R
    wl.check()
    rep_units = [wl.units(slice(W + r * K, W + (r + 1) * K))[0] for r in range(R)]

    # ---- per-kernel durations of K steps (CUDA events around every launch; one stream, no
    # overlap: a kernel's duration is then its own)
    pipeline.timing_enable(True)
    base = W + K * R
    for k in range(K):
        wl.step(W + k, base + k, overlapped=False)
    timed = pipeline.timing_collect()
    pipeline.timing_enable(False)
    clocks.stop()
    _, detail = wl.units(slice(base, base + K))

    # ---- end to end through the public API: pinned host inputs -> result sizes on the host
    wl.e2e_setup()
    wl.e2e_run(0, max(W, 3))
    torch.cuda.synchronize()
    gc.collect()
    gc.disable()          # a collection inside a ~20 ms timed region would be most of it
    e2e_ms, e2e_units, h2d, d2h = [], [], 0, 0
    for r in range(R):
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        u, h2d, d2h = wl.e2e_run(W + r * K, K)
        torch.cuda.synchronize()
        e2e_ms.append((time.perf_counter() - t0) * 1e3)   # host clock around copies, launches and reads
        e2e_units.append(u)
    gc.enable()

    # ---- reduce over ranks: per repetition the slowest rank's time and the summed units
    rep_ms_local = list(rep_ms)
    if world > 1:
        t = torch.tensor([rep_ms, e2e_ms], dtype=torch.float64, device=dev)
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        per_rank = torch.stack(gathered)                       # [world, 2, R]
        rep_ms, e2e_ms = per_rank[:, 0].max(0).values.tolist(), per_rank[:, 1].max(0).values.tolist()
        rank_medians = per_rank[:, 0].median(1).values.tolist()
        n = torch.tensor([rep_units, e2e_units], dtype=torch.int64, device=dev)
        dist.all_reduce(n, op=dist.ReduceOp.SUM)
        rep_units, e2e_units = n[0].tolist(), n[1].tolist()
        ln = torch.tensor([launches], dtype=torch.int64, device=dev)
        dist.all_reduce(ln, op=dist.ReduceOp.SUM)
        launches = int(ln[0])
    else:
        rank_medians = [float(np.median(rep_ms))]

    if rank == 0:
        peak, peak_kind = load_peaks()
        rates = [u / (ms / 1e3) for u, ms in zip(rep_units, rep_ms)]
        mid = int(np.argsort(rep_ms)[len(rep_ms) // 2])          # the median repetition
        e2e_rates = [u / (ms / 1e3) for u, ms in zip(e2e_units, e2e_ms)]
        e_mid = int(np.argsort(e2e_ms)[len(e2e_ms) // 2])
        # rooflines use rank 0's own median time and the per-kernel run's counts
        elapsed_local_s = float(np.median(rep_ms_local)) / 1e3
        roof, path = wl.roofline(timed, detail, elapsed_local_s, K, peak, peak_kind)
        by = {}
        for name, tag, ms, cnt in timed:
            by["%s[%d]" % (name, tag)] = {"ms": round(ms, 4), "launches": cnt}
        line = {
            "metric": wl.metric, "value": rates[mid], "unit": wl.unit, "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": rep_ms[mid] / K,
            "higher_is_better": True, "scaling": cfg["scaling"], "vs_baseline": None,
            "dtype": "int64" if cfg["kind"] != "ladies" else "int64+f32", "data": "synthetic",
            # the workload's defining keys first (the reference arm prints the same ones), then what
            # this arm measured about it
            "config": {"workload": args.workload, **{k: v for k, v in cfg.items() if k not in ("kind", "large")},
                       **wl.describe(detail, world)},
            "repeats": {"n": R, "what": "the K-step timed region repeated; value / ms_per_step are the median repetition",
                        "ms_per_step": {"min": min(rep_ms) / K, "median": rep_ms[mid] / K, "max": max(rep_ms) / K},
                        "value": {"min": min(rates), "median": rates[mid], "max": max(rates)},
                        "rank_median_ms_per_step": [m / K for m in rank_medians]},
            "e2e": {"value": e2e_rates[e_mid], "unit": wl.unit,
                    "h2d_bytes_per_step": h2d // K, "d2h_bytes_per_step": d2h // K, "api": wl.e2e_api,
                    "repeats": {"n": R, "min": min(e2e_rates), "median": e2e_rates[e_mid], "max": max(e2e_rates)}},
            "gpu_launches": launches,
            "roofline": roof, "roofline_path": path, "kernels": dict(sorted(by.items())),
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            cpu_threads()
            line["cpu_baseline"] = wl.cpu_baseline()
            if cfg["kind"] == "sage":
                line["cpu_baseline"]["cfg1"] = cpu_cfg1()
        if json_fd is None:
            print(json.dumps(line))
        else:
            sys.stdout.flush()
            os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
