"""Generalised SDDMM: ``out[e] = op(lhs[sel_l(e)], rhs[sel_r(e)])`` with the operands taken
from source nodes (u), edges (e) or destination nodes (v) (wrapper with the behaviour of
python/gs/ops/sddmm.py:103-110 in gSampler)."""
import torch

from ..format import _COO
from ._shapes import as_2d, broadcast_shape, check_pair, pad_ranks, rewrite_op

__all__ = ["gsddmm"]

target_mapping = {"u": 0, "e": 1, "v": 2, "src": 0, "edge": 1, "dst": 2}

# leaves for gsampler_b200.jit's tracer
torch.fx.wrap("sddmm_prepare")
torch.fx.wrap("sddmm_finish")


def sddmm_prepare(num_edges, op, lhs_data, rhs_data):
    if op not in ("copy_lhs", "copy_rhs"):
        lhs_data, rhs_data = pad_ranks(lhs_data, rhs_data)
    op, rhs_data = rewrite_op(op, rhs_data)
    use_l, use_r = op != "copy_rhs", op != "copy_lhs"
    lhs, rhs = lhs_data, rhs_data
    if use_l and use_r:
        check_pair(lhs, rhs, "gsddmm")
    scalar_l = scalar_r = False
    if use_l:
        lhs, scalar_l = as_2d(lhs)
    if use_r:
        rhs, scalar_r = as_2d(rhs)
    ref = lhs if use_l else rhs
    l_shp = lhs.shape if use_l else (0,)
    r_shp = rhs.shape if use_r else (0,)
    # every edge's entry is written exactly once, so no zero fill
    out = torch.empty((num_edges,) + broadcast_shape(op, l_shp[1:], r_shp[1:]), dtype=ref.dtype,
                      device=ref.device)
    squeeze = (scalar_l or not use_l) and (scalar_r or not use_r)
    return op, lhs, rhs, out, squeeze


def sddmm_finish(out, squeeze):
    return out.squeeze(-1) if squeeze else out


def gsddmm(g, op, lhs_data, rhs_data, lhs_target="u", rhs_target="v", on_format=_COO):
    graph = g._graph
    prep = sddmm_prepare(graph._CAPI_GetNumEdges(), op, lhs_data, rhs_data)
    # (op, lhs, rhs, out, squeeze); indexed, not unpacked, so that a trace records it
    graph._CAPI_SDDMM(prep[0], prep[1], prep[2], prep[3], target_mapping[lhs_target],
                      target_mapping[rhs_target], on_format)
    return sddmm_finish(prep[3], prep[4])
