"""``gsampler_b200.jit``: tracing and graph rewriting, checked on the structure of the rewritten
trace (no GPU needed: nothing is executed; what the compiled samplers compute is checked on the
GPU in test_gpu_jit.py).  The samplers are the ones gSampler's examples compile
(examples/graphsage/graphsage.py:7-27, examples/ladies/ladies.py:7-21 there)."""
from typing import List

import pytest
import torch

import gsampler_b200 as gs
from gsampler_b200.jit import passes


def graphsage_sampler(A, seeds, fanouts: List):
    input_node = seeds
    ret = []
    for K in fanouts:
        subA = A[:, seeds]
        sampleA = subA.individual_sampling(K, None, False)
        seeds = sampleA.all_nodes()
        ret.append(sampleA.to_dgl_block())
    return input_node, seeds, ret


def batch_graphsage_sampler(A, seeds, seeds_ptr, fanouts):
    ret = []
    for k in fanouts:
        subA = A[:, seeds::seeds_ptr]
        sampleA = subA.individual_sampling(k, None, False)
        seeds, seeds_ptr = sampleA.all_nodes()
        ret.append(sampleA.to_dgl_block())
    return ret


def ladies_sampler(A, seeds, fanouts: List):
    input_node = seeds
    ret = []
    for K in fanouts:
        subA = A[:, seeds]
        subA.edata["p"] = subA.edata["w"] ** 2
        prob = subA.sum("p", axis=1)
        sampleA, select_index = subA.collective_sampling(K, prob, False)
        sampleA = sampleA.div("w", prob[select_index], axis=1)
        out = sampleA.sum("w", axis=0)
        sampleA = sampleA.div("w", out, axis=0)
        seeds = sampleA.all_nodes()
        ret.append(sampleA.to_dgl_block(prefetch_edata={"w"}))
    return input_node, seeds, ret


def two_edge_maps(A, seeds, hu, hv):
    """Two u*v edge maps over one slice (the attention scores of the PASS sampler)."""
    subA = A[:, seeds]
    a = gs.ops.gsddmm(subA, "mul", hu, hv, "u", "v")
    b = gs.ops.gsddmm(subA, "mul", hv, hu, "u", "v")
    return a + b


def targets(gm):
    return [str(n.target) for n in gm.graph.nodes if n.op == "call_method"]


@pytest.fixture()
def matrix():
    m = gs.Matrix(gs.Graph(100, 100))
    m.edata["w"] = torch.rand(10)
    return m


def test_graphsage_trace_is_fused(matrix):
    seeds = torch.arange(10)
    raw = gs.jit.compile(graphsage_sampler, (matrix, seeds, [5, 3]), try_compact=False, format_select=False,
                         pipeline=())
    t = targets(raw.gm)
    # the trace holds the elementary operators ...
    assert t.count("_CAPI_Slicing") == 2 and t.count("_CAPI_Sampling") == 2
    assert t.count("_CAPI_GetValidNodes") == 2 and t.count("_CAPI_GraphRelabel") == 2
    c = gs.jit.compile(graphsage_sampler, (matrix, seeds, [5, 3]), try_compact=False, format_select=False)
    t = targets(c.gm)
    # ... and the passes leave one fused sampling call and one relabel per layer
    assert t.count("_CAPI_SlicingSampling") == 2 and "_CAPI_Slicing" not in t and "_CAPI_Sampling" not in t
    assert "_CAPI_GetValidNodes" not in t and t.count("_CAPI_GraphRelabel") == 2
    fused = [n for n in c.gm.graph.nodes if n.target == "_CAPI_SlicingSampling"]
    assert [n.args[3] for n in fused] == [5, 3] and all(n.args[1] == 1 and n.args[4] is False for n in fused)


def test_edge_data_follows_the_fused_index(matrix):
    def sampler(A, seeds):
        s = A[:, seeds].individual_sampling(4, None, False)
        return s.edata["w"], s.all_nodes()

    c = gs.jit.compile(sampler, (matrix, torch.arange(10)), try_compact=False, format_select=False)
    assert "_CAPI_SlicingSampling" in targets(c.gm)
    gathers = [n for n in c.gm.graph.nodes if getattr(n.target, "__name__", "") == "data_index"]
    assert len(gathers) == 1                                     # data[slice_index][sample_index] -> data[fused_index]
    idx = gathers[0].args[1]
    assert idx.args[0].target == "_CAPI_SlicingSampling" and idx.args[1] == 1
    assert gathers[0].args[0].op == "get_attr"                   # the parent's edge data, a trace constant


def test_slice_used_elsewhere_is_not_fused(matrix):
    def sampler(A, seeds):
        sub = A[:, seeds]
        return sub.individual_sampling(4, None, False).all_nodes(), sub.num_edges()

    c = gs.jit.compile(sampler, (matrix, torch.arange(10)), try_compact=False, format_select=False)
    t = targets(c.gm)
    assert "_CAPI_Slicing" in t and "_CAPI_Sampling" in t and "_CAPI_SlicingSampling" not in t


def test_batch_graphsage_becomes_one_native_call(matrix):
    bm = gs.BatchMatrix()
    bm.load_from_matrix(matrix, False)
    args = (bm, torch.arange(10), torch.tensor([0, 4, 10]), [5, 3, 2])
    no_whole = tuple(p for p in passes.DEFAULT_PIPELINE if p is not passes.fuse_graphsage_layers)
    c = gs.jit.compile(batch_graphsage_sampler, args, pipeline=no_whole)
    t = targets(c.gm)
    assert t.count("_CAPI_BatchFusedSlicingSampling") == 3 and t.count("_CAPI_BatchGraphRelabel") == 3
    assert "_CAPI_BatchColSlicing" not in t and "_CAPI_BatchRowSampling" not in t
    assert "_CAPI_BatchGetValidNodes" not in t
    c = gs.jit.compile(batch_graphsage_sampler, args)
    t = targets(c.gm)
    assert t == ["_CAPI_BatchGraphSAGE"]                         # the only graph operator left
    whole = next(n for n in c.gm.graph.nodes if n.target == "_CAPI_BatchGraphSAGE")
    assert whole.args[3] == [5, 3, 2]
    views = [n for n in c.gm.graph.nodes if getattr(n.target, "__name__", "") == "graphsage_layer_view"]
    assert [n.args[1] for n in views] == [0, 1, 2]


def test_replacement_sampling_is_not_folded_into_the_whole_call(matrix):
    def sampler(A, seeds, ptr):
        out = []
        for k in (4, 2):
            s = A[:, seeds::ptr].individual_sampling(k, None, True)
            seeds, ptr = s.all_nodes()
            out.append(s.to_dgl_block())
        return out

    bm = gs.BatchMatrix()
    bm.load_from_matrix(matrix, False)
    c = gs.jit.compile(sampler, (bm, torch.arange(10), torch.tensor([0, 10])))
    t = targets(c.gm)
    assert "_CAPI_BatchGraphSAGE" not in t and t.count("_CAPI_BatchFusedSlicingSampling") == 2


def test_ladies_trace_square_sum_fused(matrix):
    c = gs.jit.compile(ladies_sampler, (matrix, torch.arange(10), [5, 3]), try_compact=False, format_select=False)
    t = targets(c.gm)
    assert t.count("_CAPI_FusedESquareSum") == 2 and t.count("_CAPI_SpMM") == 2     # row sums fused, column sums kept
    assert not any(n.op == "call_function" and getattr(n.target, "__name__", "") == "pow" for n in c.gm.graph.nodes)
    assert t.count("_CAPI_SDDMM") == 4 and "_CAPI_GetValidNodes" not in t and t.count("_CAPI_GraphRelabel") == 2


def test_two_edge_maps_merge(matrix):
    hu, hv = torch.rand(100), torch.rand(100)
    c = gs.jit.compile(two_edge_maps, (matrix, torch.arange(10), hu, hv), try_compact=False, format_select=False)
    t = targets(c.gm)
    assert t.count("_CAPI_FusedUOPV") == 1 and "_CAPI_SDDMM" not in t
    fused = next(n for n in c.gm.graph.nodes if n.target == "_CAPI_FusedUOPV")
    order = list(c.gm.graph.nodes)
    for a in fused.args:                                         # everything it reads is computed before it
        if isinstance(a, torch.fx.Node):
            assert order.index(a) < order.index(fused)
    for n in order:                                              # and both outputs are only read after it
        if getattr(n.target, "__name__", "") == "sddmm_finish":
            assert order.index(n) > order.index(fused)


def test_random_draws_are_not_common_subexpressions(matrix):
    def sampler(A, seeds):
        sub = A[:, seeds]
        a = sub.individual_sampling(3, None, False).all_nodes()
        b = sub.individual_sampling(3, None, False).all_nodes()
        return a, b

    c = gs.jit.compile(sampler, (matrix, torch.arange(10)), try_compact=False, format_select=False)
    assert targets(c.gm).count("_CAPI_Sampling") == 2


def test_format_selection_and_compaction_follow_the_timer(matrix):
    """Selection is driven by measurements; here a scripted timer stands in for the GPU."""
    seeds = torch.arange(10)
    seen = []

    def fake_timer(run, iters):
        seen.append(iters)
        return [5.0, 1.0, 3.0, 4.0, 9.0, 8.0, 7.0, 6.0][(len(seen) - 1) % 8]

    c = gs.jit.compile(graphsage_sampler, (matrix, seeds, [5, 3]), try_compact=False, format_select=True,
                       timer=fake_timer)
    # two sub-graph-free operators on the caller's graph: one plan, formats taken from the table
    fused = [n for n in c.gm.graph.nodes if n.target == "_CAPI_SlicingSampling"]
    assert all(n.args[5] == gs._CSC and n.args[6] == gs._CSC | gs._COO for n in fused)
    seen.clear()
    c = gs.jit.compile(ladies_sampler, (matrix, seeds, [5]), try_compact=False, format_select=True, timer=fake_timer)
    timings = c.report["format_seconds"][0]
    assert len(timings) == 4 and min(t for t in timings if t is not None) == 1.0    # 2 free graphs -> 4 plans
    row_slice = [n for n in c.gm.graph.nodes if n.target == "_CAPI_Slicing" and n.args[2] == 0][0]
    assert row_slice.args[3] in (gs._CSR, gs._COO, gs._CSC)
    # compaction: both variants are built and timed, the faster one is kept
    order = iter([2.0, 1.0])
    c = gs.jit.compile(graphsage_sampler, (matrix, seeds, [5]), try_compact=True, format_select=False,
                       timer=lambda run, iters: next(order))
    assert c.report["compact_seconds"] == {True: 2.0, False: 1.0}
    assert "_CAPI_Compact" not in targets(c.gm)
    order = iter([1.0, 2.0])
    c = gs.jit.compile(graphsage_sampler, (matrix, seeds, [5]), try_compact=True, format_select=False,
                       timer=lambda run, iters: next(order))
    assert "_CAPI_Compact" in targets(c.gm)
