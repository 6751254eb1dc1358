"""``BatchMatrix``: super-batch flavour of :class:`Matrix` (mirror of
python/gs/matrix_api/batch_matrix.py:39-263 in gSampler).  Slices are written
``A[:, seeds::seeds_ptr]``: ``seeds`` concatenates the minibatches and ``seeds_ptr`` holds
their offsets.

Differences from the reference: blocks are :class:`Block` objects; with ``encoding=False``
the column slice is lazy and fuses with a following ``individual_sampling`` (the reference
obtains this through ``batch_fuse_slicing_and_sampling``, python/gs/jit/optimize.py:280-325);
``individual_sampling`` with probabilities calls the registered
``_CAPI_BatchRowSamplingProbs`` (the reference calls an unregistered name,
batch_matrix.py:183-184); ``all_nodes`` + ``to_dgl_block`` share one relabel pass.
"""
import torch

from ..format import _COO, _CSC, _CSR
from ..ops import gsddmm, gspmm
from ..utils import create_block_from_coo, create_block_from_csc
from . import matrix as _matrix
from .matrix import Matrix, data_index

torch.fx.wrap("batch_gen_block")
torch.fx.wrap("data_index")


def batch_gen_block(frontier_list, coo_row_list, coo_col_list, coo_eids, coo_ptr, edata, col_counts):
    edata_list = {}
    if coo_eids is not None:
        edata_list["_ID"] = torch.ops.gs_ops._CAPI_BatchSplitByOffset(coo_eids, coo_ptr)
    for key, value in edata.items():
        edata_list[key] = torch.ops.gs_ops._CAPI_BatchSplitByOffset(value, coo_ptr)
    block_list = []
    for i in range(len(frontier_list)):
        block = create_block_from_coo(coo_row_list[i], coo_col_list[i], frontier_list[i].numel(),
                                      col_counts[i])
        block.srcdata["_ID"] = frontier_list[i]
        for key, value in edata_list.items():
            block.edata[key] = value[i]
        block_list.append(block)
    return block_list


def batch_gen_block_csc(frontier_list, indptr_list, row_list, coo_eids, coo_ptr, edata, col_counts):
    """The same blocks in compressed form: block b = (indptr over its seed slots, relabelled row ids),
    what gSampler's ``_BatchCSCRelabelByKey`` prepares (src/cuda/batch/batch_relabel.cu:215-321,
    not bound in its Python layer)."""
    edata_list = {}
    if coo_eids is not None:
        edata_list["_ID"] = torch.ops.gs_ops._CAPI_BatchSplitByOffset(coo_eids, coo_ptr)
    for key, value in edata.items():
        edata_list[key] = torch.ops.gs_ops._CAPI_BatchSplitByOffset(value, coo_ptr)
    block_list = []
    for i in range(len(frontier_list)):
        block = create_block_from_csc(indptr_list[i], row_list[i], None, frontier_list[i].numel(), col_counts[i])
        block.srcdata["_ID"] = frontier_list[i]
        for key, value in edata_list.items():
            block.edata[key] = value[i]
        block_list.append(block)
    return block_list


torch.fx.wrap("batch_gen_block_csc")


class BatchMatrix(Matrix):

    def __init__(self, graph=None, row_ndata=None, col_ndata=None, edata=None, encoding=True):
        super().__init__(graph, row_ndata, col_ndata, edata, False)
        self.encoding = encoding
        self._pending_ptr = None

    def _new(self):
        return BatchMatrix(encoding=self.encoding)

    def load_from_matrix(self, matrix, encoding=True):
        self.__init__(matrix._graph, matrix.row_ndata, matrix.col_ndata, matrix.edata)
        self.encoding = encoding

    def _materialize(self):
        if self._pending is not None:
            parent, seeds, pedata = self._pending
            ptr = self._pending_ptr
            self._pending = None
            graph, edge_index = parent._CAPI_BatchColSlicing(seeds, ptr, False)
            self._g = graph
            for key, value in pedata.items():
                self._edata[key] = data_index(value, edge_index)

    def __getitem__(self, data):
        assert len(data) == 2
        r, c = data
        assert isinstance(r, slice) and isinstance(c, slice)
        r_slice, r_ptr, c_slice, c_ptr = r.start, r.step, c.start, c.step
        has_r = r_slice is not None and r_ptr is not None
        has_c = c_slice is not None and c_ptr is not None
        ret = self._new()

        if has_r and has_c:
            graph, edge_index = self._graph._CAPI_BatchColRowSlcing(c_slice, c_ptr, r_slice, r_ptr)
            if "_ID" in self.row_ndata or "_ID" in self.col_ndata:
                raise NotImplementedError
            ret._graph = graph
            ret.row_ndata["_ID"] = r_slice
            ret.col_ndata["_ID"] = c_slice
            for key, value in self.edata.items():
                ret._edata[key] = data_index(value, edge_index)
            for key, value in self.row_ndata.items():
                ret.row_ndata[key] = value[r_slice]
            for key, value in self.col_ndata.items():
                ret.col_ndata[key] = value[c_slice]
            return ret

        if has_r and not has_c:
            graph, edge_index = self._graph._CAPI_BatchRowSlicing(r_slice, r_ptr)
            ret._graph = graph
            if "_ID" not in self.row_ndata:
                ret.row_ndata["_ID"] = r_slice
            for key, value in self.edata.items():
                ret._edata[key] = data_index(value, edge_index)
            for key, value in self.row_ndata.items():
                ret.row_ndata[key] = value[r_slice]
            for key, value in self.col_ndata.items():
                ret.col_ndata[key] = value
            return ret

        if has_c and not has_r:
            if "_ID" in self.col_ndata:
                raise NotImplementedError
            ret.col_ndata["_ID"] = c_slice
            for key, value in self.col_ndata.items():
                ret.col_ndata[key] = value[c_slice]
            if self.encoding or not _matrix._LAZY_SLICE[0]:
                graph, edge_index = self._graph._CAPI_BatchColSlicing(c_slice, c_ptr, self.encoding)
                if self.encoding:
                    if "_ID" in self.row_ndata:
                        raise NotImplementedError
                    row_ids, _ = graph._CAPI_BatchGetRows()
                    ret.row_ndata["_ID"] = row_ids
                ret._graph = graph
                for key, value in self.edata.items():
                    ret._edata[key] = data_index(value, edge_index)
            else:
                ret._pending = (self._graph, c_slice, dict(self.edata))
                ret._pending_ptr = c_ptr
            for key, value in self.row_ndata.items():
                ret.row_ndata.setdefault(key, value)
            return ret

        raise NotImplementedError

    def individual_sampling(self, K, probs, replace):
        ret = self._new()
        if self._pending is not None and probs is None:
            parent, seeds, pedata = self._pending
            subgraph, edge_index = parent._CAPI_BatchFusedSlicingSampling(
                seeds, self._pending_ptr, K, replace)
            src_edata = pedata
        else:
            if probs is None:
                subgraph, edge_index = self._graph._CAPI_BatchRowSampling(K, replace)
            else:
                subgraph, edge_index = self._graph._CAPI_BatchRowSamplingProbs(K, replace, probs)
            src_edata = self.edata
        ret._graph = subgraph
        ret.row_ndata = self.row_ndata
        ret.col_ndata = self.col_ndata
        for key, value in src_edata.items():
            ret._edata[key] = data_index(value, edge_index)
        return ret

    def collective_sampling(self, K, probs, probs_ptr, replace):
        if probs is None:
            raise NotImplementedError
        selected_index, index_ptr = torch.ops.gs_ops._CAPI_BatchListSamplingWithProbs(
            probs, K, replace, probs_ptr)
        return self[selected_index::index_ptr, :], selected_index

    def to_dgl_block(self, prefetch_edata={}, block_format="coo"):
        """One block per minibatch.  ``block_format="csc"`` gives the compressed form instead of
        the COO: the offsets of the minibatch's seed slots (one column per slot, also where a seed
        repeats an earlier one) and the relabelled row ids."""
        (frontiers, frontiers_ptr, coo_row, coo_col, coo_eids,
         coo_bptr) = self._graph._CAPI_BatchGraphRelabel(
             self.col_ndata.get("_ID", self.null_tensor), self.row_ndata.get("_ID", self.null_tensor))
        split = torch.ops.gs_ops._CAPI_BatchSplitByOffset
        frontier_list = split(frontiers, frontiers_ptr)
        coo_row_list = split(coo_row, coo_bptr)
        col_counts = self._graph._CAPI_BatchGetColCounts()
        assign_edata = {key: self.edata[key] for key in prefetch_edata}
        if block_format == "csc":
            indptr_list = torch.ops.gs_ops._CAPI_BatchIndptrSplitByOffset(
                self._graph._CAPI_GetCSCIndptr(), self._graph._CAPI_GetColBptr())
            return batch_gen_block_csc(frontier_list, indptr_list, coo_row_list, coo_eids, coo_bptr,
                                       assign_edata, col_counts)
        coo_col_list = split(coo_col, coo_bptr)
        return batch_gen_block(frontier_list, coo_row_list, coo_col_list, coo_eids, coo_bptr,
                               assign_edata, col_counts)

    def sum(self, key, axis) -> torch.Tensor:
        rhs = self.edata[key]
        if axis == 0:
            return gspmm(self, "copy_rhs", "sum", None, rhs, 0, _COO)
        elif axis == 1:
            return gspmm(self, "copy_rhs", "sum", None, rhs, 2, _COO)
        raise ValueError("axis should be 0 or 1")

    def div(self, key, divisor, axis):
        ret_m = BatchMatrix(self._graph, self.row_ndata, self.col_ndata, self.edata.copy(),
                            self.encoding)
        lhs = self.edata[key]
        if axis == 0:
            ret_data = gsddmm(ret_m, "div", lhs, divisor, "e", "v", _COO)
        elif axis == 1:
            ret_data = gsddmm(ret_m, "div", lhs, divisor, "e", "u", _COO)
        else:
            raise ValueError("axis should be 0 or 1")
        ret_m._edata[key] = ret_data
        return ret_m

    def all_nodes(self):
        return self._graph._CAPI_BatchGetValidNodes(self.col_ndata.get("_ID", self.null_tensor),
                                                    self.row_ndata.get("_ID", self.null_tensor))

    def all_rows(self):
        return self._graph._CAPI_BatchGetRows()

    def all_cols(self):
        return self._graph._CAPI_BatchGetCols()

    def random_walk(self, seeds, seeds_ptr, walk_length):
        return torch.ops.gs_ops._CAPI_BatchSplitByOffset(
            self._graph._CAPI_RandomWalk(seeds, walk_length), seeds_ptr)

    def node2vec(self, seeds, seeds_ptr, walk_length, p, q):
        return torch.ops.gs_ops._CAPI_BatchSplitByOffset(
            self._graph._CAPI_Node2Vec(seeds, walk_length, p, q), seeds_ptr)

    def graphsage(self, seeds, seeds_ptr, fanouts):
        """All layers of the GraphSAGE super-batch sampler in one native call (no host
        synchronisation between layers).  Returns the per-layer tensors of
        ``Graph._CAPI_BatchGraphSAGE``."""
        return self._graph._CAPI_BatchGraphSAGE(seeds, seeds_ptr, list(fanouts))

    def graphsage_async(self, seeds, seeds_ptr, fanouts):
        """Enqueue the GraphSAGE super-batch sampler on the current CUDA stream and return at
        once.  ``.wait()`` on the returned object gives what :meth:`graphsage` returns.  A data
        loader keeps two or three super-batches in flight, each on its own stream, so that the
        copies and the host work of one overlap the kernels of another."""
        return GraphSAGEResult(self._graph._CAPI_BatchGraphSAGEAsync(seeds, seeds_ptr, list(fanouts)),
                               len(fanouts), (seeds, seeds_ptr))


class GraphSAGEResult:
    """Pending result of :meth:`BatchMatrix.graphsage_async`."""

    _pinned = {}      # free pinned count buffers by length (page-locking memory is slow)

    def __init__(self, tensors, num_layers, inputs):
        self._t = tensors
        self._L = num_layers
        self._inputs = inputs                      # kept alive until the kernels have run
        free = GraphSAGEResult._pinned.setdefault(3 * num_layers + 1, [])
        self._host = free.pop() if free else torch.empty(3 * num_layers + 1, dtype=torch.int64,
                                                         pin_memory=True)
        self._host.copy_(tensors[-1], non_blocking=True)
        self._done = torch.cuda.Event()
        self._done.record()

    def wait(self):
        if self._host is None:
            return self._result
        self._done.synchronize()
        c = self._host.tolist()
        if c[3 * self._L]:
            raise RuntimeError("graphsage_sample reported device-side error bits 0x%x" % c[3 * self._L])
        out = []
        for l in range(self._L):
            S, E, U = c[3 * l:3 * l + 3]
            t = self._t[9 * l:9 * l + 9]
            out += [t[0][:S + 1], t[1][:E], t[2][:E], t[3][:E], t[4], t[5][:U], t[6], t[7][:E], t[8][:E]]
        out.append(self._host[:3 * self._L].clone())
        GraphSAGEResult._pinned[3 * self._L + 1].append(self._host)
        self._host = None
        self._result = out
        return out
