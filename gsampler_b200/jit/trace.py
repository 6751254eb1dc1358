"""Tracing a sampler written against ``Matrix`` / ``BatchMatrix`` into a ``torch.fx`` graph
(the job of ``GSTracer`` / ``gs_symbolic_trace`` in gSampler, python/gs/jit/trace.py:9-35).

The traced callable takes three arguments: the caller's dynamic arguments (seed tensors ...),
the ``gs_classes.Graph`` objects of its matrix arguments, and their node / edge data.  The data
dictionaries are specialised into the trace (their tensors become constants of the module, as
in gSampler), the graphs and the dynamic arguments are placeholders, and everything a ``Matrix``
method does to its graph shows up as a ``call_method`` node on the graph's proxy
(``_CAPI_Slicing`` ...), which is what the passes rewrite."""
from __future__ import annotations

import math
import warnings

import torch
from torch.fx import GraphModule, Tracer

from ..matrix_api import matrix as _matrix


class SamplerTracer(Tracer):

    def __init__(self):
        super().__init__(autowrap_modules=(math,), autowrap_functions=(), param_shapes_constant=False)


def trace_sampler(fn, data_args) -> GraphModule:
    """``fn(dyn_args, graphs, graph_data)`` -> GraphModule, with ``graph_data`` fixed to
    ``data_args``.  Column slices are traced eagerly (see ``_LAZY_SLICE``)."""
    tracer = SamplerTracer()
    lazy = _matrix._LAZY_SLICE[0]
    _matrix._LAZY_SLICE[0] = False
    try:
        with warnings.catch_warnings():
            # fx cannot emit an assertion that later calls pass the same data dictionaries; the
            # caller of the compiled sampler is told so in compile's documentation instead
            warnings.filterwarnings("ignore", message="Was not able to add assertion")
            graph = tracer.trace(fn, concrete_args={"graph_data": data_args})
    finally:
        _matrix._LAZY_SLICE[0] = lazy
    return GraphModule(tracer.root, graph, getattr(fn, "__name__", "sampler"))
