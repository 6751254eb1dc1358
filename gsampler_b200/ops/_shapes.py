"""Operand preparation shared by the SpMM / SDDMM wrappers: the rules of
python/gs/ops/spmm.py:13-105 and python/gs/ops/sddmm.py:16-100 in gSampler (rank padding,
``sub`` -> ``add`` of the negation, ``div`` -> ``mul`` by the reciprocal, scalar features
carried as a trailing unit dimension, broadcast of the feature shapes)."""
import torch


def pad_ranks(lhs, rhs):
    if lhs.dim() != rhs.dim():
        nd = max(lhs.dim(), rhs.dim())
        lhs = lhs.view((lhs.shape[0],) + (1,) * (nd - lhs.dim()) + tuple(lhs.shape[1:]))
        rhs = rhs.view((rhs.shape[0],) + (1,) * (nd - rhs.dim()) + tuple(rhs.shape[1:]))
    return lhs, rhs


def rewrite_op(op, rhs):
    if op == "sub":
        return "add", -rhs
    if op == "div":
        return "mul", 1.0 / rhs
    return op, rhs


def broadcast_shape(op, shp1, shp2):
    shp1, shp2 = tuple(shp1), tuple(shp2)
    if op == "dot" and shp1[-1] != shp2[-1]:
        raise ValueError("dot needs equal last dimensions, got %s and %s" % (shp1, shp2))
    if len(shp1) > len(shp2):
        shp2 = (1,) * (len(shp1) - len(shp2)) + shp2
    elif len(shp1) < len(shp2):
        shp1 = (1,) * (len(shp2) - len(shp1)) + shp1
    for d1, d2 in zip(shp1, shp2):
        if d1 != d2 and d1 != 1 and d2 != 1:
            raise ValueError("feature shapes %s and %s do not broadcast" % (shp1, shp2))
    out = tuple(max(d1, d2) for d1, d2 in zip(shp1, shp2))
    return out[:-1] + (1,) if op == "dot" else out


def check_pair(a, b, what):
    if a.device != b.device:
        raise ValueError("%s: operands live on different devices (%s, %s)" % (what, a.device, b.device))
    if a.dtype != b.dtype:
        raise ValueError("%s: operand dtypes differ (%s, %s)" % (what, a.dtype, b.dtype))


def as_2d(t):
    """scalar features ([N]) travel as [N, 1]; returns (tensor, was_scalar)"""
    if t.dim() == 1:
        return t.unsqueeze(-1), True
    return t, False
