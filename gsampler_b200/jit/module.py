"""``compile``: trace a sampler once, rewrite the trace, pick formats by measurement, and call
the result from then on (the job of ``gs.jit.compile``, python/gs/jit/module.py:191-446 in
gSampler; same constructor arguments and call convention).

Arguments of the example call are classified the way gSampler does (module.py:72-110): a
``Matrix`` / ``BatchMatrix`` contributes its graph object (a placeholder of the trace) and its
node / edge data (specialised into the trace); lists, ints, floats and bools are constants of the
trace (fanouts, walk lengths); everything else (seed tensors) is passed through at every call.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional, Sequence

import torch
import torch.fx as fx

from ..format import _COO, _CSC, _CSR
from ..matrix_api import BatchMatrix, Matrix
from . import passes
from .trace import trace_sampler

# Operators whose format arguments may be chosen freely: name -> (position of on_format,
# position of output_format or None), positions counted with the graph as argument 0
# (python/gs/jit/module.py:21-31).
FORMAT_ARGS = {
    "_CAPI_Slicing": (3, 4), "_CAPI_Sampling": (4, 5), "_CAPI_SamplingProbs": (5, 6),
    "_CAPI_SlicingSampling": (5, 6), "_CAPI_SDDMM": (7, None), "_CAPI_SpMM": (9, None),
    "_CAPI_FusedUOPV": (8, None), "_CAPI_FusedESquareSum": (9, None), "_CAPI_FusedEDivUSum": (9, None),
}
# Formats an operator can run on, best guess first: name -> (position of the argument that decides
# (axis / u_target) or None, {value: [formats]} or [formats])  (python/gs/jit/module.py:33-64).
FORMAT_CHOICES = {
    "_CAPI_Slicing": (2, {0: [_CSR, _COO, _CSC], 1: [_CSC, _COO, _CSR]}),
    "_CAPI_Sampling": (1, {0: [_CSR], 1: [_CSC]}),
    "_CAPI_SamplingProbs": (1, {0: [_CSR], 1: [_CSC]}),
    "_CAPI_SlicingSampling": (1, {0: [_CSR], 1: [_CSC]}),
    "_CAPI_SDDMM": (None, [_COO, _CSC, _CSR]),
    "_CAPI_SpMM": (8, {2: [_CSR, _COO], 0: [_CSC, _COO]}),
    "_CAPI_FusedUOPV": (None, [_COO, _CSC]),
    "_CAPI_FusedESquareSum": (8, {2: [_CSR, _COO], 0: [_CSC, _COO]}),
    "_CAPI_FusedEDivUSum": (8, {2: [_CSR, _COO], 0: [_CSC, _COO]}),
}


class _Plan(object):
    """Which argument of the sampler is a graph, a trace constant, or passed through."""

    def __init__(self, args: Sequence):
        self.kinds: List[str] = []
        self.static = {}
        for i, a in enumerate(args):
            if isinstance(a, BatchMatrix):
                self.kinds.append("batch")
            elif isinstance(a, Matrix):
                self.kinds.append("matrix")
            elif isinstance(a, (list, bool, int, float)):
                self.kinds.append("static")
                self.static[i] = a
            else:
                self.kinds.append("dynamic")

    def split(self, args: Sequence):
        graphs, data, dyn = [], [], []
        for kind, a in zip(self.kinds, args):
            if kind == "matrix":
                graphs.append(a._graph)
                data.append([a.row_ndata, a.col_ndata, a.edata])
            elif kind == "batch":
                graphs.append(a._graph)
                data.append([a.row_ndata, a.col_ndata, a.edata, a.encoding])
            elif kind == "dynamic":
                dyn.append(a)
        return dyn, graphs, data

    def rebuild(self, dyn, graphs, data, compact: bool):
        out, g, d = [], 0, 0
        for i, kind in enumerate(self.kinds):
            if kind == "matrix":
                out.append(Matrix(graphs[g], data[g][0], data[g][1], data[g][2], compact))
                g += 1
            elif kind == "batch":
                out.append(BatchMatrix(graphs[g], data[g][0], data[g][1], data[g][2], data[g][3]))
                g += 1
            elif kind == "static":
                out.append(self.static[i])
            else:
                out.append(dyn[d])
                d += 1
        return out


def _default_timer(run: Callable[[], None], iters: int) -> float:
    """Mean seconds per call over the second half of `iters` calls (the first half warms up), as
    gSampler's _bench_gm (python/gs/jit/module.py:268-278)."""
    times = []
    for _ in range(iters):
        t0 = time.perf_counter()
        run()
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    tail = times[iters // 2 + 1:] or times
    return sum(tail) / len(tail)


class compile(object):  # noqa: N801  (name kept from the reference API)
    """``compiled = compile(func, example_args); compiled(*args)``.

    try_compact / must_compact: trace the sampler with and without compacting every slice
    (``Matrix(..., compact=True)``) and keep the faster one / force compaction.
    format_select: choose, per operator, the sparse format it runs on by timing the candidates.
    pipeline: the rewriting passes (default: ``passes.DEFAULT_PIPELINE``).
    timer: ``timer(run, iters) -> seconds`` used by both measurements (default: wall clock around
    a synchronised call); lets tests drive the selection without a GPU.
    ``compiled.gm`` is the ``torch.fx.GraphModule`` that runs."""

    def __init__(self, func, args, try_compact=True, format_select=True, must_compact=False,
                 pipeline=passes.DEFAULT_PIPELINE, timer: Optional[Callable] = None, iters: int = 10):
        self.func = func
        self.plan = _Plan(args)
        self.pipeline = tuple(pipeline)
        self.iters = iters
        self._timer = timer or _default_timer
        self.report = {}
        batch = "batch" in self.plan.kinds
        if batch:                                   # super-batches are never compacted
            self.gm = self._build(args, False)
        elif must_compact:
            self.gm = self._build(args, True)
            if format_select:
                self.gm = self.select_formats(self.gm, args)
        elif try_compact:
            cands = []
            for compact in (True, False):
                gm = self._build(args, compact)
                if format_select:
                    gm = self.select_formats(gm, args)
                cands.append((self._time(gm, args), compact, gm))
            self.report["compact_seconds"] = {c: t for t, c, _ in cands}
            self.gm = min(cands, key=lambda c: c[0])[2]
        else:
            self.gm = self._build(args, False)
            if format_select:
                self.gm = self.select_formats(self.gm, args)

    def __call__(self, *args):
        dyn, graphs, data = self.plan.split(args)
        return self.gm(dyn, graphs, data)

    # -------------------------------------------------------------- trace + rewrite
    def _build(self, args, compact: bool) -> fx.GraphModule:
        plan, func = self.plan, self.func

        def sampler(dyn_args, graphs, graph_data):
            return func(*plan.rebuild(dyn_args, graphs, graph_data, compact))

        sampler.__name__ = getattr(func, "__name__", "sampler")
        _, _, data = plan.split(args)
        return passes.optimize(trace_sampler(sampler, data), self.pipeline)

    def _time(self, gm, args) -> float:
        def run():
            dyn, graphs, data = self.plan.split(args)
            gm(dyn, graphs, data)
        return self._timer(run, self.iters)

    # -------------------------------------------------------------- format selection
    def select_formats(self, gm: fx.GraphModule, args) -> fx.GraphModule:
        """Every graph a format-sensitive operator runs on is given a set of formats it may be
        kept in -- CSC + COO, or CSC + CSR + COO (graphs handed in by the caller count as CSC) --
        each operator takes the first of its preferred formats that its graph holds and asks for
        that format (plus COO) as output; every assignment is timed on the example arguments and
        the fastest is kept (python/gs/jit/module.py:306-421)."""
        ops = [n for n in gm.graph.nodes if n.op == "call_method" and n.target in FORMAT_ARGS]
        graphs: List[fx.Node] = []
        for n in ops:
            if n.args[0] not in graphs:
                graphs.append(n.args[0])
        if not ops:
            return gm
        fixed = {g: _CSC for g in graphs if _from_caller(g)}
        free = [g for g in graphs if g not in fixed]
        plans = []
        for mask in range(1 << len(free)):
            held = dict(fixed)
            for i, g in enumerate(free):
                held[g] = (_CSC | _CSR | _COO) if (mask >> i) & 1 else (_CSC | _COO)
            plans.append(held)
        original = [(n, tuple(n.args)) for n in ops]
        best = None
        timings = []
        for held in plans:
            if not _apply_formats(ops, held):
                timings.append(None)
                continue
            gm.recompile()
            try:
                t = self._time(gm, args)
            except Exception:                       # an operator rejected the combination
                t = None
            timings.append(t)
            if t is not None and (best is None or t < best[0]):
                best = (t, held)
        self.report.setdefault("format_seconds", []).append(timings)
        if best is None:
            for n, a in original:
                n.args = a
        else:
            _apply_formats(ops, best[1])
        gm.graph.lint()
        gm.recompile()
        return gm


def _from_caller(node: fx.Node) -> bool:
    """Is this graph one the caller passed in (``graphs[i]`` of the traced signature)?"""
    import operator

    return (node.op == "call_function" and node.target is operator.getitem and
            isinstance(node.args[0], fx.Node) and node.args[0].op == "placeholder")


def _apply_formats(ops, held) -> bool:
    for n in ops:
        on_pos, out_pos = FORMAT_ARGS[n.target]
        key_pos, choices = FORMAT_CHOICES[n.target]
        if key_pos is not None:
            choices = choices.get(n.args[key_pos])
            if choices is None:
                return False
        pick = next((f for f in choices if f & held[n.args[0]]), None)
        if pick is None:
            return False
        n.update_arg(on_pos, pick)
        if out_pos is not None:
            n.update_arg(out_pos, pick | _COO)
    return True
