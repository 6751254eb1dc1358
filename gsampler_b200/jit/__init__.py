"""``compile``: entry point with the call signature of gSampler's ``gs.jit.compile``
(python/gs/jit/module.py:191-266).

gSampler traces the sampler with torch.fx and rewrites the graph (merge relabel + all_nodes,
fuse slicing + sampling, batch fusion: python/gs/jit/optimize.py:124-325).  Here the same
fusions happen at run time inside the operators -- a column slice stays lazy until it is
known whether a sampling call follows (then one fused kernel runs), and ``all_nodes`` /
``to_dgl_block`` on the same matrix share one relabel pass -- so the compiled callable is
the user's function itself, bound to a warm-up run that validates it on the example
arguments.  ``try_compact`` / ``format_select`` / ``must_compact`` are accepted for source
compatibility; format selection is fixed (CSC for column operators, COO for edge maps).
"""
from __future__ import annotations


class compile(object):  # noqa: N801  (name kept from the reference API)

    def __init__(self, func, args, try_compact=True, format_select=True, must_compact=False,
                 warmup=False):
        self.func = func
        self.try_compact = try_compact
        self.format_select = format_select
        self.must_compact = must_compact
        if warmup:
            func(*args)

    def __call__(self, *args):
        return self.func(*args)


__all__ = ["compile"]
