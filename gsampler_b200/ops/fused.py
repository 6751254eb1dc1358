"""Fused edge-map + reduce operators (python/gs/ops/fused_op.py:92-243 in gSampler):
``e_square_sum``: out[n] = sum of e^2 over the edges of node n;
``e_div_u_sum`` : out[n] = sum of e / u[src] over the edges of node n."""
import torch

__all__ = ["e_square_sum", "e_div_u_sum"]


def _out(graph, e, u_target):
    n = graph._CAPI_GetNumCols() if u_target == 0 else graph._CAPI_GetNumRows()
    return torch.zeros((n, 1), dtype=e.dtype, device=e.device)


def e_square_sum(g, edata, u_target, on_format):
    graph = g._graph
    e = edata.unsqueeze(-1) if edata.dim() == 1 else edata
    out = _out(graph, e, u_target)
    graph._CAPI_FusedESquareSum("copy_rhs", "sum", None, e, out, None, None, u_target, on_format)
    return out.squeeze(-1)


def e_div_u_sum(g, edata, udata, u_target, on_format):
    graph = g._graph
    e = edata.unsqueeze(-1) if edata.dim() == 1 else edata
    u = udata.unsqueeze(-1) if udata.dim() == 1 else udata
    out = _out(graph, e, u_target)
    graph._CAPI_FusedEDivUSum("div", "sum", u, e, out, None, None, u_target, on_format)
    return out.squeeze(-1)
