"""Graph rewriting passes over a traced sampler.

They do what gSampler's ``optimize.py`` passes do (python/gs/jit/optimize.py: cse :102-121,
dce :44-99, merge_relabel_and_all_indices :124-179, fuse_slicing_and_sampling :182-277,
batch_fuse_slicing_and_sampling :280-325, fuse_ESqure_and_SumReduce :328-369,
merge_fused_u_mul_v :377-425) on this package's traces, plus two rewrites gSampler does not
have: the batch form of the relabel merge and ``fuse_graphsage_layers``, which turns a whole
multi-layer GraphSAGE super-batch sampler into ONE native call.

A pass takes and returns a ``torch.fx.GraphModule``; it never changes what the sampler returns.
"""
from __future__ import annotations

import operator
from typing import Dict, List, Optional

import torch
import torch.fx as fx

# methods of gs_classes.Graph that write into a caller-provided tensor: they have no users in the
# graph but must stay, and two of them are never "the same computation"
IN_PLACE = {"_CAPI_SDDMM", "_CAPI_SpMM", "_CAPI_FusedUOPV", "_CAPI_FusedESquareSum", "_CAPI_FusedEDivUSum"}
# operators that draw random numbers: two textually equal calls are two different draws
RANDOM = {"_CAPI_Sampling", "_CAPI_SamplingProbs", "_CAPI_SlicingSampling", "_CAPI_BatchRowSampling",
          "_CAPI_BatchRowSamplingProbs", "_CAPI_BatchFusedSlicingSampling", "_CAPI_RandomWalk",
          "_CAPI_Node2Vec", "_CAPI_BatchGraphSAGE", "_CAPI_LadiesLayer"}
RANDOM_FUNCTIONS = ("_CAPI_ListSampling", "_CAPI_ListSamplingWithProbs", "_CAPI_BatchListSampling",
                    "_CAPI_BatchListSamplingWithProbs")
# leaf helpers that allocate an output which an in-place operator then fills
ALLOCATING = ("spmm_prepare", "sddmm_prepare")


def _name(node: fx.Node) -> str:
    t = node.target
    return t if isinstance(t, str) else getattr(t, "__name__", str(t))


def _is_random(node: fx.Node) -> bool:
    n = _name(node)
    return (node.op == "call_method" and n in RANDOM) or any(r in str(node.target) for r in RANDOM_FUNCTIONS)


def _finish(gm: fx.GraphModule) -> fx.GraphModule:
    gm.graph.lint()
    gm.recompile()
    return gm


def _item(graph: fx.Graph, src: fx.Node, i: int) -> fx.Node:
    return graph.call_function(operator.getitem, args=(src, i))


def _items_of(node: fx.Node) -> Dict[int, List[fx.Node]]:
    """users of `node` that are `node[i]`, by i"""
    out: Dict[int, List[fx.Node]] = {}
    for u in node.users:
        if u.op == "call_function" and u.target is operator.getitem and u.args[0] is node and isinstance(u.args[1], int):
            out.setdefault(u.args[1], []).append(u)
    return out


# ------------------------------------------------------------------ clean-up passes
def eliminate_dead_code(gm: fx.GraphModule) -> fx.GraphModule:
    """Removes nodes nothing depends on.  In-place operators stay (their effect is the tensor
    they fill), and so does everything they read."""
    for node in reversed(list(gm.graph.nodes)):
        if node.op in ("placeholder", "output"):
            continue
        if node.op == "call_method" and node.target in IN_PLACE:
            continue
        if len(node.users) == 0:
            gm.graph.erase_node(node)
    return _finish(gm)


def eliminate_common_subexpressions(gm: fx.GraphModule) -> fx.GraphModule:
    """Two nodes with the same target and the same arguments compute the same value -- unless
    they draw random numbers, fill a tensor in place, or allocate the tensor that gets filled."""
    seen: Dict[str, fx.Node] = {}
    for node in list(gm.graph.nodes):
        if node.op in ("placeholder", "output", "get_attr"):
            continue
        if _is_random(node) or (node.op == "call_method" and node.target in IN_PLACE):
            continue
        if _name(node) in ALLOCATING:
            continue
        key = "%s|%s|%r|%r" % (node.op, node.target, node.args, node.kwargs)
        first = seen.get(key)
        if first is None:
            seen[key] = node
        else:
            node.replace_all_uses_with(first)
            gm.graph.erase_node(node)
    return _finish(gm)


# ------------------------------------------------------------------ relabel + node list
def merge_relabel_with_node_list(gm: fx.GraphModule) -> fx.GraphModule:
    """``all_nodes()`` and ``to_dgl_block()`` on the same matrix both relabel the same edges:
    ``_CAPI_GetValidNodes(g, a, b)`` becomes item 0 of ``_CAPI_GraphRelabel(g, a, b)``, and
    ``_CAPI_BatchGetValidNodes`` items 0 / 1 of ``_CAPI_BatchGraphRelabel``."""
    pairs = (("_CAPI_GetValidNodes", "_CAPI_GraphRelabel", False),
             ("_CAPI_BatchGetValidNodes", "_CAPI_BatchGraphRelabel", True))
    gm = eliminate_common_subexpressions(gm)
    for nodes_name, relabel_name, batch in pairs:
        for node in list(gm.graph.nodes):
            if node.op != "call_method" or node.target != nodes_name:
                continue
            # (looked up afresh every time: an earlier merge rewrites the arguments of later calls)
            rel = next((r for r in gm.graph.nodes if r.op == "call_method" and r.target == relabel_name
                        and tuple(r.args[:3]) == tuple(node.args[:3])), None)
            if rel is None:
                continue
            # the relabel must come first: move it in front of the node-list call when needed
            if _comes_after(gm.graph, rel, node):
                node.prepend(rel)
            with gm.graph.inserting_after(rel):
                if batch:
                    ptr = _item(gm.graph, rel, 1)
                    ids = _item(gm.graph, rel, 0)
                    for i, users in _items_of(node).items():
                        for u in users:
                            u.replace_all_uses_with(ids if i == 0 else ptr)
                else:
                    node.replace_all_uses_with(_item(gm.graph, rel, 0))
    return eliminate_dead_code(gm)


def _comes_after(graph: fx.Graph, a: fx.Node, b: fx.Node) -> bool:
    for n in graph.nodes:
        if n is a:
            return False
        if n is b:
            return True
    return False


# ------------------------------------------------------------------ slicing + sampling
def _edge_data_users(index_node: Optional[fx.Node]):
    """For the edge index of a slice: [(data_index node, [lookups of it by a later index])] or
    None when the index is used in a way the fusion cannot follow."""
    if index_node is None:
        return []
    out = []
    for u in index_node.users:
        if u.op == "call_function" and _name(u) == "data_index" and u.args[1] is index_node:
            out.append(u)
        else:
            return None
    return out


def fuse_slicing_and_sampling(gm: fx.GraphModule) -> fx.GraphModule:
    """``A[:, seeds]`` followed by uniform per-column sampling of the slice is one kernel:
    ``_CAPI_Slicing(g, seeds, axis, f, o)[0]._CAPI_Sampling(axis, K, replace, f2, o2)`` ->
    ``g._CAPI_SlicingSampling(axis, seeds, K, replace, f2, o2)``.  The fused operator returns edge
    positions in ``g``, so edge data that went ``data[slice_index][sample_index]`` becomes
    ``data[fused_index]``.  Only done when the slice itself is used for nothing else."""
    for samp in list(gm.graph.nodes):
        if samp.op != "call_method" or samp.target != "_CAPI_Sampling":
            continue
        sub = samp.args[0]
        if not (sub.op == "call_function" and sub.target is operator.getitem and sub.args[1] == 0):
            continue
        sl = sub.args[0]
        if sl.op != "call_method" or sl.target != "_CAPI_Slicing" or sl.args[2] != samp.args[1]:
            continue
        if len(sub.users) != 1:
            continue
        sl_items, samp_items = _items_of(sl), _items_of(samp)
        if len(sl_items.get(0, [])) != 1 or len(sl_items.get(1, [])) > 1 or len(samp_items.get(1, [])) > 1:
            continue
        sl_index = sl_items.get(1, [None])[0]
        samp_index = samp_items.get(1, [None])[0]
        gathers = _edge_data_users(sl_index)
        if gathers is None:
            continue
        ok = True
        for gnode in gathers:   # every sliced edge array must only be looked up by the sampling index
            for u in gnode.users:
                if not (_name(u) == "data_index" and u.args[0] is gnode and u.args[1] is samp_index):
                    ok = False
        if not ok:
            continue
        with gm.graph.inserting_before(samp):
            fused = gm.graph.call_method("_CAPI_SlicingSampling",
                                         args=(sl.args[0], sl.args[2], sl.args[1], samp.args[2], samp.args[3],
                                               samp.args[4], samp.args[5]))
            fused_graph, fused_index = _item(gm.graph, fused, 0), _item(gm.graph, fused, 1)
            for gnode in gathers:
                for u in list(gnode.users):
                    u.replace_all_uses_with(gm.graph.call_function(u.target, args=(gnode.args[0], fused_index)))
        for u in samp_items.get(0, []):
            u.replace_all_uses_with(fused_graph)
        if samp_index is not None:
            samp_index.replace_all_uses_with(fused_index)
    return eliminate_dead_code(gm)


def fuse_batch_slicing_and_sampling(gm: fx.GraphModule) -> fx.GraphModule:
    """The super-batch form: ``_CAPI_BatchColSlicing(g, seeds, ptr, False)[0]
    ._CAPI_BatchRowSampling(K, replace)`` -> ``g._CAPI_BatchFusedSlicingSampling(seeds, ptr, K,
    replace)`` (not with row-id encoding, whose slice renames the rows)."""
    for samp in list(gm.graph.nodes):
        if samp.op != "call_method" or samp.target != "_CAPI_BatchRowSampling":
            continue
        sub = samp.args[0]
        if not (sub.op == "call_function" and sub.target is operator.getitem and sub.args[1] == 0):
            continue
        sl = sub.args[0]
        if sl.op != "call_method" or sl.target != "_CAPI_BatchColSlicing" or sl.args[3] is not False:
            continue
        if len(sub.users) != 1:
            continue
        sl_items, samp_items = _items_of(sl), _items_of(samp)
        if len(sl_items.get(1, [])) > 1 or len(samp_items.get(1, [])) > 1:
            continue
        sl_index = sl_items.get(1, [None])[0]
        samp_index = samp_items.get(1, [None])[0]
        gathers = _edge_data_users(sl_index)
        if gathers is None or any(not (_name(u) == "data_index" and u.args[1] is samp_index)
                                  for gnode in gathers for u in gnode.users):
            continue
        with gm.graph.inserting_before(samp):
            fused = gm.graph.call_method("_CAPI_BatchFusedSlicingSampling",
                                         args=(sl.args[0], sl.args[1], sl.args[2], samp.args[1], samp.args[2]))
            fused_graph, fused_index = _item(gm.graph, fused, 0), _item(gm.graph, fused, 1)
            for gnode in gathers:
                for u in list(gnode.users):
                    u.replace_all_uses_with(gm.graph.call_function(u.target, args=(gnode.args[0], fused_index)))
        for u in samp_items.get(0, []):
            u.replace_all_uses_with(fused_graph)
        if samp_index is not None:
            samp_index.replace_all_uses_with(fused_index)
    return eliminate_dead_code(gm)


# ------------------------------------------------------------------ edge maps
def fuse_square_and_sum(gm: fx.GraphModule) -> fx.GraphModule:
    """``sum(e ** 2)`` per node: the square moves into the reduction
    (``_CAPI_SpMM(copy_rhs, sum, e ** 2)`` -> ``_CAPI_FusedESquareSum(copy_rhs, sum, e)``), when the
    squared array feeds nothing but that sum."""
    for node in list(gm.graph.nodes):
        if not (node.op == "call_function" and node.target is operator.pow and node.args[1] == 2):
            continue
        users = list(node.users)
        if len(users) != 1 or _name(users[0]) != "spmm_prepare":
            continue
        prep = users[0]
        if prep.args[2] != "copy_rhs" or prep.args[3] != "sum" or prep.args[5] is not node:
            continue
        spmm = [u for i in _items_of(prep).values() for g in i for u in g.users
                if u.op == "call_method" and u.target == "_CAPI_SpMM"]
        if len(set(spmm)) != 1:
            continue
        spmm = spmm[0]
        prep.update_arg(5, node.args[0])
        with gm.graph.inserting_before(spmm):
            gm.graph.call_method("_CAPI_FusedESquareSum", args=tuple(spmm.args))
        gm.graph.erase_node(spmm)
    return eliminate_dead_code(gm)


def merge_u_op_v(gm: fx.GraphModule) -> fx.GraphModule:
    """Two edge maps ``op(u[row], v[col])`` with the same operator over the same graph read the
    endpoints once: a pair of ``_CAPI_SDDMM(g, op, l, r, out, 0, 2, f)`` -> ``_CAPI_FusedUOPV``."""
    groups: Dict[tuple, List[fx.Node]] = {}
    for node in gm.graph.nodes:
        if node.op == "call_method" and node.target == "_CAPI_SDDMM" and node.args[5] == 0 and node.args[6] == 2:
            prep = node.args[1].args[0] if isinstance(node.args[1], fx.Node) and node.args[1].args else None
            op = prep.args[1] if prep is not None and _name(prep) == "sddmm_prepare" else node.args[1]
            if isinstance(op, str):
                groups.setdefault((node.args[0], op, node.args[7]), []).append(node)
    for (g, op, fmt), nodes in groups.items():
        if len(nodes) != 2:
            continue
        first, second = nodes
        # everything the second call reads must exist before the fused call, which takes the
        # second call's place
        with gm.graph.inserting_before(second):
            gm.graph.call_method("_CAPI_FusedUOPV", args=(g, first.args[1], first.args[2], first.args[3], first.args[4],
                                                          second.args[2], second.args[3], second.args[4], fmt))
        # users of the first output (its finish leaf) ran between the two calls: move them behind
        out1 = first.args[4]
        later = [u for u in out1.users if u is not first and _comes_after(gm.graph, u, first) and
                 not _comes_after(gm.graph, u, second)]
        for u in later:
            _move_after(gm.graph, u, second)
        gm.graph.erase_node(first)
        gm.graph.erase_node(second)
    return eliminate_dead_code(gm)


def _move_after(graph: fx.Graph, node: fx.Node, anchor: fx.Node) -> None:
    """Moves `node` and, transitively, its users that lie before `anchor`, behind `anchor`."""
    order = {n: i for i, n in enumerate(graph.nodes)}
    todo = [node]
    moved = []
    while todo:
        n = todo.pop()
        if n in moved or order[n] > order[anchor]:
            continue
        moved.append(n)
        todo.extend(n.users)
    moved.sort(key=lambda n: order[n])
    at = anchor
    for n in moved:
        at.append(n)
        at = n


# ------------------------------------------------------------------ whole GraphSAGE sampler
def graphsage_layer_view(out, layer: int):
    """What ``_CAPI_BatchGraphRelabel`` returns for layer ``layer`` of a ``_CAPI_BatchGraphSAGE``
    result: (node lists, their offsets, block rows, block cols, edge ids (none), edge offsets)."""
    t = out[9 * layer:9 * layer + 9]
    return t[5], t[6], t[7], t[8], None, t[4]


def ptr_counts(ptr):
    """Segment sizes of an offset tensor as a list of ints (one host read)."""
    return (ptr[1:] - ptr[:-1]).tolist()


torch.fx.wrap("graphsage_layer_view")
torch.fx.wrap("ptr_counts")


def fuse_graphsage_layers(gm: fx.GraphModule) -> fx.GraphModule:
    """A super-batch GraphSAGE sampler -- per layer ``A[:, seeds::ptr]``, uniform sampling without
    replacement, ``all_nodes``, ``to_dgl_block``, the node lists being the next layer's seeds -- is
    a chain ``_CAPI_BatchFusedSlicingSampling(g, seeds, ptr, K, False)`` ->
    ``_CAPI_BatchGraphRelabel(sub, seeds, <empty>)`` whose items 0 / 1 feed the next layer's call
    on the same ``g``.  The whole chain becomes ONE ``g._CAPI_BatchGraphSAGE(seeds, ptr, [K...])``:
    every layer's kernels are enqueued without a host round trip in between, and the relabel
    results are views of its output.  Run after the slicing/sampling fusion and the relabel merge."""
    graph = gm.graph

    def layer_of(samp: fx.Node):
        """(relabel node, sub-graph node, edge-index node or None) when `samp` heads a fusable layer"""
        if samp.op != "call_method" or samp.target != "_CAPI_BatchFusedSlicingSampling" or samp.args[4] is not False:
            return None
        items = _items_of(samp)
        if len(items.get(0, [])) != 1 or len(items.get(1, [])) > 1:
            return None
        sub = items[0][0]
        rel = None
        for u in sub.users:
            if (u.op == "call_method" and u.target == "_CAPI_BatchGraphRelabel" and u.args[1] is samp.args[1]
                    and isinstance(u.args[2], fx.Node) and _name(u.args[2]) == "null_ids"):
                rel = u if rel is None else rel
            elif (u.op == "call_method" and u.target == "_CAPI_BatchGetColCounts") or _name(u) == "null_ids":
                pass
            else:
                return None
        if rel is None:
            return None
        return rel, sub, items.get(1, [None])[0]

    heads = [n for n in graph.nodes if layer_of(n) is not None]
    used = set()
    for head in heads:
        if head in used:
            continue
        chain = [head]
        while True:
            rel = layer_of(chain[-1])[0]
            rel_items = _items_of(rel)
            nxt = [u for g0 in rel_items.get(0, []) for u in g0.users
                   if layer_of(u) is not None and u.args[0] is head.args[0] and u.args[1] is g0 and
                   any(u.args[2] is g1 for g1 in rel_items.get(1, []))]
            if len(nxt) != 1:
                break
            chain.append(nxt[0])
        if len(chain) < 2:
            continue
        used.update(chain)
        fanouts = [int(c.args[3]) for c in chain]
        with graph.inserting_before(head):
            whole = graph.call_method("_CAPI_BatchGraphSAGE", args=(head.args[0], head.args[1], head.args[2], fanouts))
            layer_ptr = head.args[2]
            for l, samp in enumerate(chain):
                rel, sub, index = layer_of(samp)
                view = graph.call_function(graphsage_layer_view, args=(whole, l))
                if index is not None:
                    index.replace_all_uses_with(_item(graph, whole, 9 * l + 3))
                for u in list(sub.users):
                    if u.op == "call_method" and u.target == "_CAPI_BatchGetColCounts":
                        u.replace_all_uses_with(graph.call_function(ptr_counts, args=(layer_ptr,)))
                rel.replace_all_uses_with(view)
                layer_ptr = _item(graph, whole, 9 * l + 6)
    return eliminate_dead_code(gm)


DEFAULT_PIPELINE = (eliminate_common_subexpressions, eliminate_dead_code, merge_relabel_with_node_list,
                    fuse_slicing_and_sampling, fuse_batch_slicing_and_sampling, fuse_square_and_sum,
                    merge_u_op_v, fuse_graphsage_layers, eliminate_dead_code)


def optimize(gm: fx.GraphModule, pipeline=DEFAULT_PIPELINE) -> fx.GraphModule:
    for p in pipeline:
        gm = p(gm)
    return gm
