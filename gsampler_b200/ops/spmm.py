"""Generalised SpMM: ``out[dst] = reduce_{e -> dst} op(u[src(e)], e[e])``
(wrapper with the behaviour of python/gs/ops/spmm.py:109-124 in gSampler)."""
import torch

from ._shapes import as_2d, broadcast_shape, check_pair, pad_ranks, rewrite_op

__all__ = ["gspmm"]

# leaves for gsampler_b200.jit's tracer: operand preparation works on real tensors and shapes
torch.fx.wrap("spmm_prepare")
torch.fx.wrap("spmm_finish")


def spmm_prepare(num_rows, num_cols, op, reduce_op, lhs_data, rhs_data, lhs_target):
    if op not in ("copy_lhs", "copy_rhs"):
        lhs_data, rhs_data = pad_ranks(lhs_data, rhs_data)
    op, rhs_data = rewrite_op(op, rhs_data)
    use_u, use_e = op != "copy_rhs", op != "copy_lhs"
    u, e = lhs_data, rhs_data
    if use_u and use_e:
        check_pair(u, e, "gspmm")
    scalar_u = scalar_e = False
    if use_u:
        u, scalar_u = as_2d(u)
    if use_e:
        e, scalar_e = as_2d(e)
    ref = u if use_u else e
    u_shp = u.shape if use_u else (0,)
    e_shp = e.shape if use_e else (0,)
    n_out = num_cols if lhs_target == 0 else num_rows
    v = torch.zeros((n_out,) + broadcast_shape(op, u_shp[1:], e_shp[1:]), dtype=ref.dtype,
                    device=ref.device)
    arg_u = arg_e = None
    if reduce_op in ("max", "min"):
        if use_u:
            arg_u = torch.zeros(v.shape, dtype=torch.int64, device=ref.device)
        if use_e:
            arg_e = torch.zeros(v.shape, dtype=torch.int64, device=ref.device)
    squeeze = (scalar_u or not use_u) and (scalar_e or not use_e)
    return op, u, e, v, arg_u, arg_e, squeeze


def spmm_finish(v, squeeze):
    return v.squeeze(-1) if squeeze else v


def gspmm(g, op, reduce_op, lhs_data, rhs_data, lhs_target, on_format):
    graph = g._graph
    prep = spmm_prepare(graph._CAPI_GetNumRows(), graph._CAPI_GetNumCols(), op, reduce_op, lhs_data,
                        rhs_data, lhs_target)
    # (op, u, e, out, arg_u, arg_e, squeeze); indexed, not unpacked, so that a trace records it
    graph._CAPI_SpMM(prep[0], reduce_op, prep[1], prep[2], prep[3], prep[4], prep[5], lhs_target, on_format)
    return spmm_finish(prep[3], prep[6])
