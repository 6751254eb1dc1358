"""Operator-by-operator timing of this library against the reference's OWN CUDA kernels (the
tier-2 oracle ``oracle/_ref/gs_ref.so``, the reference's kernel files compiled unmodified for
sm_100a by ``oracle/build_ref.py``) on one GPU and the same inputs.

    python oracle/ref_op_times.py [--reps 5] > table.json

Both sides run with device-resident inputs, allocate their own outputs and include their own size
read-backs; time is CUDA-event time per call, mean of `reps` calls after 2 warm-up calls.  This
library is called through its reference-facing boundary (``gs_classes.Graph`` / ``gs_ops``), the
reference through its kernel entry points (so the reference's ``gs::Graph`` host layer is NOT
charged to it).  Where this library caches a result on the graph object (formats, relabel), a
fresh object is made inside the timed call and the producing operator is timed with it on both
sides ("FSS+RL" = fused sampling followed by relabel).  Not a test: results are printed, one JSON
line per operator; equality of the results is what tests/test_gpu_reference.py checks."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
import gsampler_b200 as gsb  # noqa: E402
from gsampler_b200 import synth  # noqa: E402
from oracle import build_ref  # noqa: E402


def timed(fn, reps):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        out = fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps, out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    ref = build_ref.load()
    if ref is None:
        print(json.dumps({"unavailable": "oracle/_ref/gs_ref.so not built"}))
        return
    dev = torch.device("cuda")
    cfg = bench.WORKLOADS["cfg2"]
    indptr, indices = bench.make_graph(cfg, dev, synth)
    n, E = cfg["nodes"], int(indptr[-1])
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    rnd = lambda hi, k: torch.randint(0, hi, (k,), generator=gen, device=dev)  # noqa: E731
    no_map = torch.empty(0, dtype=torch.int64, device=dev)
    CSC, COO = gsb._CSC, gsb._COO

    def graph():
        g = gsb.Graph(n, n)
        g._CAPI_LoadCSC(indptr, indices)
        return g

    A = graph()
    rows_out = []

    def row(op, what, ours, theirs):
        ms_o, _ = timed(ours, args.reps)
        ms_r, _ = timed(theirs, args.reps)
        rows_out.append({"op": op, "workload": what, "ms": round(ms_o, 4), "reference_ms": round(ms_r, 4),
                         "speedup": round(ms_r / ms_o, 2)})
        print(json.dumps(rows_out[-1]), flush=True)

    # ---- SL / BSL: column slicing
    S = 400000
    seeds = rnd(n, S)
    ptr = (torch.arange(33, device=dev) * (S // 32)).to(torch.int64)
    row("SL", "A[:, 400 000 random columns] (20 M entries), CSC+COO out",
        lambda: A._CAPI_Slicing(seeds, 1, CSC, CSC + COO),
        lambda: ref.slice_cols(indptr, indices, seeds, True))
    row("BSL", "the same as 32 minibatches (no encoding)",
        lambda: A._CAPI_BatchColSlicing(seeds, ptr, False),
        lambda: ref.batch_slice_cols(indptr, indices, seeds, ptr, True, False, 0))

    # ---- FSS / SA: uniform sampling
    S3 = 3700000
    seeds3 = rnd(n, S3)
    row("FSS", "fused slice+sample, 3.7 M columns, K=5",
        lambda: A._CAPI_SlicingSampling(1, seeds3, 5, False, CSC, COO),
        lambda: ref.fused_slice_sample(indptr, indices, 5, seeds3, False, True))
    row("FSS", "fused slice+sample, 400 000 columns, K=10",
        lambda: A._CAPI_SlicingSampling(1, seeds, 10, False, CSC, COO),
        lambda: ref.fused_slice_sample(indptr, indices, 10, seeds, False, True))
    sub, _ = A._CAPI_Slicing(seeds, 1, CSC, CSC)
    s_indptr, s_indices = sub._CAPI_GetCSCIndptr(), sub._CAPI_GetCSCIndices()
    row("SA", "sampling of an already sliced matrix (400 000 columns, 20 M entries), K=10",
        lambda: sub._CAPI_Sampling(1, 10, False, CSC, COO),
        lambda: ref.sample_cols(s_indptr, s_indices, 10, False, True))

    # ---- SAP: weighted per-column sampling of the slice
    probs = torch.rand(E, generator=gen, device=dev) + 0.01
    M = gsb.Matrix(graph())
    M.edata["w"] = probs

    def ours_sap():
        g = graph()
        s, sel = g._CAPI_Slicing(seeds, 1, CSC, CSC)
        return s._CAPI_SamplingProbs(1, probs[sel], 10, False, CSC, COO)

    def ref_sap():
        ip, _, r, sel = ref.slice_cols(indptr, indices, seeds, True)
        return ref.sample_cols_probs(ip, r, probs[sel], 10, False, True)

    row("SL+SAP", "column slice, weights of the slice, weighted sampling K=10 (400 000 columns)", ours_sap, ref_sap)

    # ---- UQ / RL / BRL on a sampled layer (3.7 M columns, K=5: about 18 M edges)
    def ours_fss_then(f):
        def run():
            s, _ = graph()._CAPI_SlicingSampling(1, seeds3, 5, False, CSC, COO)
            return f(s)
        return run

    def ref_fss_then(f):
        def run():
            ip, col, r, _ = ref.fused_slice_sample(indptr, indices, 5, seeds3, False, True)
            return f(ip, col, r)
        return run

    row("FSS+UQ", "sampling as above, then unique(cat(seeds, rows)) in first-occurrence order",
        ours_fss_then(lambda s: s._CAPI_GetValidNodes(seeds3, no_map)),
        ref_fss_then(lambda ip, col, r: ref.tensor_unique(torch.cat([seeds3, r]))))
    row("FSS+RL", "sampling as above, then unique + relabelled COO",
        ours_fss_then(lambda s: s._CAPI_GraphRelabel(seeds3, no_map)),
        ref_fss_then(lambda ip, col, r: ref.tensor_relabel([seeds3, r], [seeds3[col], r])))
    ptr3 = (torch.arange(33, device=dev) * (S3 // 32)).to(torch.int64)
    ptr3[-1] = S3

    def ours_brl():
        s, _ = graph()._CAPI_BatchFusedSlicingSampling(seeds3, ptr3, 5, False)
        return s._CAPI_BatchGraphRelabel(seeds3, no_map)

    def ref_brl():
        ip, col, r, _ = ref.fused_slice_sample(indptr, indices, 5, seeds3, False, True)
        return ref.batch_coo_relabel(seeds3, ptr3, seeds3[col], r, ip[ptr3])

    row("BFSS+BRL", "32 minibatches: fused sampling, then per-minibatch unique + relabel", ours_brl, ref_brl)

    # ---- LS: collective sampling
    p_nodes = torch.rand(n, generator=gen, device=dev)
    row("LS", "weighted choice of 4000 of 2 449 029 items without replacement",
        lambda: torch.ops.gs_ops._CAPI_ListSamplingWithProbs(p_nodes, 4000, False),
        lambda: ref.list_sampling_probs(p_nodes, 4000, False))
    rng_ptr = (torch.arange(33, device=dev) * (n // 32)).to(torch.int64)
    rng_ptr[-1] = n
    row("LS (batch)", "the same in 32 segments, 4000 picks each",
        lambda: torch.ops.gs_ops._CAPI_BatchListSamplingWithProbs(p_nodes, 4000, False, rng_ptr),
        lambda: ref.batch_list_sampling_probs(p_nodes, 4000, False, rng_ptr))
    row("LS (uniform)", "uniform choice of 4000 of 2 449 029 without replacement",
        lambda: torch.ops.gs_ops._CAPI_ListSampling(n, 4000, False),
        lambda: ref.list_sampling(n, 4000, False))

    # ---- RS: row slicing
    keep = torch.randperm(n, generator=gen, device=dev)[:n // 4]
    row("RS", "rows: keep 612 257 of 2 449 029 row ids over the whole CSC (123.7 M entries)",
        lambda: A._CAPI_Slicing(keep, 0, CSC, CSC),
        lambda: ref.slice_rows_on_indices(indptr, indices, keep, False))
    ncol, nrow = 512, 4000
    cols = rnd(n, 32 * ncol)
    rws = torch.cat([torch.randperm(n, generator=gen, device=dev)[:nrow] for _ in range(32)])
    cptr = (torch.arange(33, device=dev) * ncol).to(torch.int64)
    rptr = (torch.arange(33, device=dev) * nrow).to(torch.int64)
    row("RS (fused col+row, batch)", "32 minibatches of 512 columns x 4000 kept rows",
        lambda: A._CAPI_BatchColRowSlcing(cols, cptr, rws, rptr),
        lambda: ref.batch_col_row_slicing(indptr, indices, cols, cptr, rws, rptr, n))

    # ---- SPMM / SDDMM on scalar edge weights of the whole graph
    col_of_edge = torch.repeat_interleave(torch.arange(n, device=dev), indptr[1:] - indptr[:-1])
    dummy = torch.zeros(1, 1, device=dev)
    aux = torch.zeros(n, 1, dtype=torch.int64, device=dev)
    w2 = probs[:, None].contiguous()

    def ref_spmm_csc():
        out = torch.zeros(n, 1, device=dev)
        ref.spmm_csc("copy_rhs", "sum", indptr, indices, dummy, w2, out, aux, aux)
        return out

    def ref_spmm_coo():
        out = torch.zeros(n, 1, device=dev)
        ref.spmm_coo("copy_rhs", "sum", indices, col_of_edge, dummy, w2, out, 2, aux, aux)
        return out

    M.sum("w", axis=1)  # COO made once, outside the timed calls, as col_of_edge is for the reference
    row("SPMM", "column sums of 123.7 M fp32 edge weights (CSC)", lambda: M.sum("w", axis=0), ref_spmm_csc)
    row("SPMM", "row sums of the same (COO, atomics on both sides)", lambda: M.sum("w", axis=1), ref_spmm_coo)
    node = torch.rand(n, 1, generator=gen, device=dev) + 0.5
    node1 = node[:, 0].contiguous()

    def ref_sddmm():
        out = torch.zeros(E, 1, device=dev)
        ref.sddmm_coo("mul", indices, col_of_edge, w2, node, out, 1, 0)
        return out

    row("SDDMM", "edge weight x value of the row node, 123.7 M edges",
        lambda: gsb.ops.gsddmm(M, "mul", probs, node1, "e", "u"), ref_sddmm)

    # ---- RW / N2V
    walkers = rnd(n, 1000000)
    row("RW", "1 M uniform walks x 80 steps", lambda: A._CAPI_RandomWalk(walkers, 80),
        lambda: ref.random_walk(walkers, 80, indices, indptr))
    row("N2V", "1 M node2vec walks x 80 steps, p=2, q=0.5 (sorted columns)",
        lambda: A._CAPI_Node2Vec(walkers, 80, 2.0, 0.5),
        lambda: ref.node2vec(walkers, 80, indices, indptr, 2.0, 0.5))

    # ---- fused edge operators of the PASS / AS-GCN / LADIES samplers (scalar per-node values)
    u1, v1, u2, v2 = (torch.rand(n, 1, generator=gen, device=dev) + 0.5 for _ in range(4))
    o1, o2 = torch.empty(E, 1, device=dev), torch.empty(E, 1, device=dev)
    row("FUSED_U_OP_V", "two u-mul-v maps over 123.7 M edges in one pass (COO)",
        lambda: A._CAPI_FusedUOPV("mul", u1, v1, o1, u2, v2, o2, COO),
        lambda: ref.fused_u_op_v_coo("mul", indices, col_of_edge, u1, v1, o1, u2, v2, o2))

    def ours_e2():
        out = torch.zeros(n, 1, device=dev)
        A._CAPI_FusedESquareSum("copy_rhs", "sum", None, w2, out, None, None, 0, CSC)
        return out

    def ref_e2():
        out = torch.zeros(n, 1, device=dev)
        ref.e_square_sum_csc("copy_rhs", "sum", indptr, indices, dummy, w2, out, aux, aux)
        return out

    row("E_SQUARE_SUM", "per-column sum of squared edge weights, 123.7 M edges (CSC)", ours_e2, ref_e2)

    def ours_edu():
        out = torch.zeros(n, 1, device=dev)
        A._CAPI_FusedEDivUSum("div", "sum", node, w2, out, None, None, 0, CSC)
        return out

    def ref_edu():
        out = torch.zeros(n, 1, device=dev)
        ref.e_div_u_sum_csc("div", "sum", indptr, indices, node, w2, out, aux, aux)
        return out

    row("E_DIV_U_SUM", "per-column sum of edge weight / value of the row node (CSC)", ours_edu, ref_edu)

    # ---- SORT: per-column sort of the whole graph (once-per-graph preprocessing), shuffled columns
    shuffled = indices[torch.randperm(E, generator=gen, device=dev)]  # columns keep their lengths, not their order

    def ours_sort():
        g = gsb.Graph(n, n)
        g._CAPI_LoadCSC(indptr, shuffled)
        g._CAPI_SortCSCIndices()
        return g

    row("SORT", "every column of 123.7 M randomly ordered row ids sorted (copy included on both sides)",
        ours_sort, lambda: ref.sort_indices(indptr, shuffled))
    print(json.dumps({"graph": "cfg2: %d nodes / %d edges, int64" % (n, E), "reps": args.reps,
                      "rows": len(rows_out)}))


if __name__ == "__main__":
    main()
