"""``Matrix``: the matrix-centric sampling API (mirror of python/gs/matrix_api/matrix.py:42-303
in gSampler -- same methods, argument meaning and results).

Differences that matter to a caller:

* ``to_dgl_block`` returns a :class:`gsampler_b200.utils.Block` (DGL is optional).
* ``A[:, seeds]`` is lazy: when the next call is ``individual_sampling`` the two run as the
  single fused kernel (what ``gs.jit.compile``'s ``fuse_slicing_and_sampling`` pass,
  python/gs/jit/optimize.py:182-277, obtains by graph rewriting); any other use materialises
  the slice first, so results are the same as eager execution.
* ``collective_sampling(K, None, replace)`` works (the reference dereferences ``probs``,
  matrix.py:187-189).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..format import _COO, _CSC, _CSR
from ..ops import gsddmm, gspmm
from ..utils import Block, create_block_from_coo

# Helpers that work on real tensors are leaves for ``gsampler_b200.jit``'s tracer (one
# call_function node each), as in python/gs/matrix_api/matrix.py:12-16 of gSampler.
torch.fx.wrap("create_block_from_coo")
torch.fx.wrap("assign_block")
torch.fx.wrap("data_index")
torch.fx.wrap("null_ids")

# While ``gsampler_b200.jit.compile`` traces a sampler the column slice is NOT lazy: the trace
# then holds the elementary operators and the fusion is the passes' job.
_LAZY_SLICE = [True]


def null_ids(graph=None):
    """The empty id tensor that stands for "no explicit row / column ids".  ``graph`` is unused; a
    traced sampler passes its graph so that the call is recorded instead of run while tracing."""
    return torch.empty(0, dtype=torch.int64, device="cuda")


def data_index(data, index):
    """``data[index]``; data kept in pinned host memory is gathered in place by a kernel
    (gSampler: python/gs/matrix_api/matrix.py:19-23)."""
    if not data.is_cuda and data.is_pinned():
        return torch.ops.gs_ops._CAPI_GatherRows(data, index)
    return data[index]


def assign_block(block: Block, e_ids, edata, unique_tensor) -> Block:
    if e_ids is not None:
        block.edata["_ID"] = e_ids
    for key, value in edata.items():
        block.edata[key] = value
    block.srcdata["_ID"] = unique_tensor
    return block


class Matrix(object):

    def __init__(self, graph=None, row_ndata=None, col_ndata=None, edata=None, compact=False):
        self._g = graph
        self._pending = None  # (parent graph, seeds, parent edata) of a not-yet-run column slice
        self.row_ndata = {} if row_ndata is None else row_ndata
        self.col_ndata = {} if col_ndata is None else col_ndata
        self._edata = {} if edata is None else edata
        self._compact = compact

    # ------------------------------------------------------------------ lazy slice plumbing
    def _materialize(self):
        if self._pending is not None:
            parent, seeds, pedata = self._pending
            self._pending = None
            graph, edge_index = parent._CAPI_Slicing(seeds, 1, _CSC, _COO)
            self._g = graph
            for key, value in pedata.items():
                self._edata[key] = data_index(value, edge_index)

    @property
    def _graph(self):
        self._materialize()
        return self._g

    @_graph.setter
    def _graph(self, g):
        self._pending = None
        self._g = g

    @property
    def edata(self):
        self._materialize()
        return self._edata

    @edata.setter
    def edata(self, value):
        self._materialize()
        self._edata = value

    @property
    def null_tensor(self):
        return null_ids(self._g)

    def _new(self) -> "Matrix":
        return Matrix()

    # ------------------------------------------------------------------ loading
    def load_graph(self, format: str, format_tensors: List[torch.Tensor]) -> "Matrix":
        assert format in ["CSC", "COO", "CSR"]
        assert len(format_tensors) == 2
        G = torch.classes.gs_classes.Graph
        if format == "COO":
            coo_row, coo_col = format_tensors
            self._graph = G(int(coo_row.max()) + 1, int(coo_col.max()) + 1)
            self._graph._CAPI_LoadCOO(coo_row, coo_col, False, False)
        elif format == "CSC":
            indptr, indices = format_tensors
            self._graph = G(int(indices.max()) + 1, indptr.numel() - 1)
            self._graph._CAPI_LoadCSC(indptr, indices)
        else:
            indptr, indices = format_tensors
            self._graph = G(indptr.numel() - 1, int(indices.max()) + 1)
            self._graph._CAPI_LoadCSR(indptr, indices)
        return self

    # ------------------------------------------------------------------ extract
    def __getitem__(self, data) -> "Matrix":
        assert len(data) == 2
        r_slice, c_slice = data
        has_c = isinstance(c_slice, (torch.Tensor, torch.fx.Proxy))   # a Proxy while being traced
        has_r = isinstance(r_slice, (torch.Tensor, torch.fx.Proxy))
        ret = self._new()

        if has_c and not has_r and not self._compact and _LAZY_SLICE[0]:
            # lazy column slice
            if "_ID" not in self.col_ndata:
                ret.col_ndata["_ID"] = c_slice
            for key, value in self.col_ndata.items():
                ret.col_ndata[key] = value[c_slice]
            for key, value in self.row_ndata.items():
                ret.row_ndata[key] = value
            ret._pending = (self._graph, c_slice, dict(self.edata))
            return ret

        graph = self._graph
        edge_index = None
        if has_c:
            if "_ID" not in self.col_ndata:
                ret.col_ndata["_ID"] = c_slice
            graph, edge_index = graph._CAPI_Slicing(c_slice, 1, _CSC, _COO)
        if has_r:
            if "_ID" not in self.row_ndata:
                ret.row_ndata["_ID"] = r_slice
            graph, _edge_index = graph._CAPI_Slicing(r_slice, 0, _CSR, _COO)
            edge_index = _edge_index if edge_index is None else edge_index[_edge_index]
        ret._graph = graph
        for key, value in self.edata.items():
            ret._edata[key] = data_index(value, edge_index) if edge_index is not None else value
        for key, value in self.col_ndata.items():
            ret.col_ndata[key] = value[c_slice] if has_c else value
        for key, value in self.row_ndata.items():
            ret.row_ndata[key] = value[r_slice] if has_r else value
        if self._compact:
            ret.compact(0)
            ret.compact(1)
        return ret

    def compact(self, axis):
        ndata = self.row_ndata if axis == 0 else self.col_ndata
        if "_ID" not in ndata:
            new_graph, unique_tensor = self._graph._CAPI_Compact(axis)
            for key, value in ndata.items():
                ndata[key] = value[unique_tensor]
            ndata["_ID"] = unique_tensor
            self._graph = new_graph
        return self

    # ------------------------------------------------------------------ select
    def individual_sampling(self, K: int, probs: Optional[torch.Tensor], replace: bool) -> "Matrix":
        ret = self._new()
        if self._pending is not None and probs is None:
            parent, seeds, pedata = self._pending
            subgraph, edge_index = parent._CAPI_SlicingSampling(1, seeds, K, replace, _CSC, _COO)
            src_edata = pedata
        else:
            if probs is None:
                subgraph, edge_index = self._graph._CAPI_Sampling(1, K, replace, _CSC, _COO)
            else:
                subgraph, edge_index = self._graph._CAPI_SamplingProbs(1, probs, K, replace, _CSC, _COO)
            src_edata = self.edata
        ret._graph = subgraph
        ret.row_ndata = self.row_ndata
        ret.col_ndata = self.col_ndata
        for key, value in src_edata.items():
            ret._edata[key] = data_index(value, edge_index)
        return ret

    def collective_sampling(self, K: int, probs: Optional[torch.Tensor], replace: bool):
        if probs is None:
            selected_index = torch.ops.gs_ops._CAPI_ListSampling(self.num_rows(), K, replace)
        else:
            selected_index = torch.ops.gs_ops._CAPI_ListSamplingWithProbs(probs, K, replace)
        return self[selected_index, :], selected_index

    # ------------------------------------------------------------------ compute
    def sum(self, key, axis, on_format=_CSC) -> torch.Tensor:
        rhs = self.edata[key]
        if axis == 0:
            return gspmm(self, "copy_rhs", "sum", None, rhs, 0, _CSC)
        elif axis == 1:
            return gspmm(self, "copy_rhs", "sum", None, rhs, 2, _CSR)
        raise ValueError("axis should be 0 or 1")

    def div(self, key, divisor, axis) -> "Matrix":
        ret_m = type(self)(self._graph, self.row_ndata, self.col_ndata)
        lhs = self.edata[key]
        if axis == 0:
            ret_data = gsddmm(ret_m, "div", lhs, divisor, "e", "v", _COO)
        elif axis == 1:
            ret_data = gsddmm(ret_m, "div", lhs, divisor, "e", "u", _COO)
        else:
            raise ValueError("axis should be 0 or 1")
        ret_m._edata = self.edata.copy()
        ret_m._edata[key] = ret_data
        return ret_m

    # ------------------------------------------------------------------ finalize
    def to_dgl_block(self, prefetch_edata={}) -> Block:
        col_seeds = self.col_ndata.get("_ID", self.null_tensor)
        unique_tensor, format_tensor1, format_tensor2, e_ids = self._graph._CAPI_GraphRelabel(
            col_seeds, self.row_ndata.get("_ID", self.null_tensor))
        block = create_block_from_coo(format_tensor1, format_tensor2,
                                      num_src=unique_tensor.numel(), num_dst=col_seeds.numel())
        assign_edata = {key: self.edata[key] for key in prefetch_edata}
        return assign_block(block, e_ids, assign_edata, unique_tensor)

    def ladies_layer(self, seeds, num_pick, weight_key="w"):
        """One layer of the layer-wise (LADIES) sampler in a single native call: the operator
        sequence of gSampler's examples/ladies/ladies.py:7-21 (``A[:, seeds]``, row weights
        ``sum(w**2)``, collective sampling of ``num_pick`` rows, ``w / p[row]``, ``w / column
        sum``, ``all_nodes``, ``to_dgl_block``).  Returns ``(block, next_seeds, picked_rows)``; the
        block carries the renormalised weights as ``edata[weight_key]`` and the positions of its
        edges in this matrix as ``edata["_ID"]``."""
        nodes, brow, bcol, w, picked, edge_pos, _ = self._graph._CAPI_LadiesLayer(
            seeds, int(num_pick), self.edata[weight_key])
        block = create_block_from_coo(brow, bcol, num_src=nodes.numel(), num_dst=seeds.numel())
        block.edata[weight_key] = w
        block.edata["_ID"] = edge_pos
        block.srcdata["_ID"] = nodes
        return block, nodes, picked

    def all_nodes(self) -> torch.Tensor:
        return self._graph._CAPI_GetValidNodes(self.col_ndata.get("_ID", self.null_tensor),
                                               self.row_ndata.get("_ID", self.null_tensor))

    def num_rows(self) -> int:
        return self._graph._CAPI_GetNumRows()

    def num_cols(self) -> int:
        return self._graph._CAPI_GetNumCols()

    def num_edges(self) -> int:
        return self._graph._CAPI_GetNumEdges()

    @property
    def csc(self) -> List[torch.Tensor]:
        g = self._graph
        return [g._CAPI_GetCSCIndptr(), g._CAPI_GetCSCIndices(), g._CAPI_GetCSCEids()]

    @property
    def csr(self) -> List[torch.Tensor]:
        g = self._graph
        return [g._CAPI_GetCSRIndptr(), g._CAPI_GetCSRIndices(), g._CAPI_GetCSREids()]

    @property
    def coo(self) -> List[torch.Tensor]:
        g = self._graph
        return [g._CAPI_GetCOORows(), g._CAPI_GetCOOCols(), g._CAPI_GetCOOEids()]

    def random_walk(self, seeds, walk_length) -> torch.Tensor:
        return self._graph._CAPI_RandomWalk(seeds, walk_length)

    def node2vec(self, seeds, walk_length, p, q) -> torch.Tensor:
        return self._graph._CAPI_Node2Vec(seeds, walk_length, p, q)

    def rows(self) -> torch.Tensor:
        if "_ID" in self.row_ndata:
            return self.row_ndata["_ID"]
        return torch.arange(self.num_rows(), dtype=torch.int64, device="cuda")

    def cols(self) -> torch.Tensor:
        if "_ID" in self.col_ndata:
            return self.col_ndata["_ID"]
        return torch.arange(self.num_cols(), dtype=torch.int64, device="cuda")
