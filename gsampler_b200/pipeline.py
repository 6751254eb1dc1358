"""``GraphSAGESampler``: the whole L-layer super-batch sampler as a stream-ordered call with
pre-allocated buffers.

``BatchMatrix.graphsage`` (one native call per super-batch) allocates its outputs and reads the
per-layer sizes back to the host.  A training loop that wants neither keeps one of these
objects instead: buffers are allocated once for stated capacities, :meth:`sample` only
enqueues kernels on the current CUDA stream (no allocation, no synchronisation), and the
per-layer sizes stay in device memory until :meth:`counts` is called.

The object talks to the C ABI (``include/gsb200.h``: ``gsb_graphsage_sample``) through ctypes;
torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import LIB_CUDA

_lib = None


class _LayerBuffers(C.Structure):
    _fields_ = [("S_cap", C.c_int64), ("E_cap", C.c_int64)] + [
        (n, C.c_void_p) for n in ("sub_indptr", "rows", "cols", "sel", "edge_ptr", "unique",
                                  "unique_ptr", "block_row", "block_col")]


_FIELDS = ("sub_indptr", "rows", "cols", "sel", "edge_ptr", "unique", "unique_ptr", "block_row",
           "block_col")


def cabi():
    """The C ABI library with result types set (shared with bench / tests)."""
    global _lib
    if _lib is None:
        lib = C.CDLL(LIB_CUDA)
        lib.gsb_graphsage_workspace_bytes.restype = C.c_size_t
        lib.gsb_graphsage_sample.restype = C.c_int
        lib.gsb_status_string.restype = C.c_char_p
        lib.gsb_last_cuda_error.restype = C.c_char_p
        lib.gsb_kernel_launches.restype = C.c_uint64
        lib.gsb_timing_enable.restype = C.c_int
        lib.gsb_timing_collect.restype = C.c_int
        _lib = lib
    return _lib


def kernel_launches() -> int:
    return int(cabi().gsb_kernel_launches())


def timing_enable(on: bool) -> None:
    cabi().gsb_timing_enable(1 if on else 0)


def timing_collect(max_entries: int = 256):
    """[(kernel name, tag, total ms, launches)] since :func:`timing_enable`; synchronises."""
    names = (C.c_char_p * max_entries)()
    tags = (C.c_int * max_entries)()
    ms = (C.c_double * max_entries)()
    cnt = (C.c_int64 * max_entries)()
    n = cabi().gsb_timing_collect(max_entries, names, tags, ms, cnt)
    if n < 0:
        raise RuntimeError("gsb_timing_collect failed: %s" % cabi().gsb_last_cuda_error().decode())
    return [(names[i].decode(), int(tags[i]), float(ms[i]), int(cnt[i])) for i in range(n)]


class GraphSAGESampler(object):
    """Pre-allocated L-layer sampler over a CSC graph resident on one GPU.

    indptr            int64 [N+1] CUDA tensor
    indices           int32 or int64 [nnz] CUDA tensor (or both tensors in pinned host memory)
    num_batches       minibatches per super-batch (B)
    max_seeds         upper bound of the number of seeds in one super-batch
    fanouts           per-layer fanout
    num_nodes         exclusive upper bound of the node ids (default: number of columns)
    capacities        optional [(S_cap, E_cap)] per layer; default = worst case
                      (S_cap[l+1] = S_cap[l] + E_cap[l], E_cap[l] = S_cap[l] * fanout[l]).
                      Smaller capacities save memory; overflow is reported through the error
                      word (``check``), never written out of bounds.
    narrow_ids        keep a 32-bit copy of 64-bit row ids and sample from it (graphs of fewer
                      than 2^31 nodes, resident on the GPU): a random pick then costs fewer DRAM
                      bursts per column and L2 holds twice the share of the array; outputs stay
                      int64 and are the same.  Costs half the array's size again in device memory.
    """

    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor, num_batches: int,
                 max_seeds: int, fanouts: Sequence[int], seed: int = 7777,
                 capacities: Optional[Sequence] = None, num_nodes: Optional[int] = None,
                 narrow_ids: bool = True):
        on_gpu = indptr.is_cuda and indices.is_cuda
        if not on_gpu and not (indptr.is_pinned() and indices.is_pinned()):
            raise ValueError("the graph must live on a CUDA device or in pinned host memory, which "
                             "the kernels read in place (there is no CPU path)")
        if indptr.dtype != torch.int64 or indices.dtype not in (torch.int32, torch.int64):
            raise ValueError("indptr must be int64, indices int32 or int64")
        self.indptr, self.indices = indptr.contiguous(), indices.contiguous()
        self.device = indptr.device if on_gpu else torch.device("cuda", torch.cuda.current_device())
        self.B, self.L = int(num_batches), len(fanouts)
        self.fanouts = [int(k) for k in fanouts]
        self.seed = int(seed)
        self.max_seeds = int(max_seeds)
        # exclusive bound of all node ids (seeds and row ids); lets the relabel stage pick
        # direct-address tables when that is the smaller representation
        self.num_nodes = int(indptr.numel() - 1 if num_nodes is None else num_nodes)
        opt = dict(dtype=torch.int64, device=self.device)
        self._bufs = (_LayerBuffers * self.L)()
        self.layers: List[dict] = []
        s_cap = self.max_seeds
        for l, k in enumerate(self.fanouts):
            if capacities is not None:
                s_cap, e_cap = int(capacities[l][0]), int(capacities[l][1])
            else:
                e_cap = s_cap * k
            sizes = dict(sub_indptr=s_cap + 1, rows=e_cap, cols=e_cap, sel=e_cap, edge_ptr=self.B + 1,
                         unique=s_cap + e_cap, unique_ptr=self.B + 1, block_row=e_cap, block_col=e_cap)
            t = {n: torch.empty(sz, **opt) for n, sz in sizes.items()}
            t["S_cap"], t["E_cap"] = s_cap, e_cap
            self.layers.append(t)
            b = self._bufs[l]
            b.S_cap, b.E_cap = s_cap, e_cap
            for n in _FIELDS:
                setattr(b, n, t[n].data_ptr())
            s_cap = s_cap + e_cap
        self._fan = (C.c_int64 * self.L)(*self.fanouts)
        lib = cabi()
        nbytes = lib.gsb_graphsage_workspace_bytes(C.c_int64(self.B), self.L, self._bufs, self._fan)
        self._ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
        self._counts = torch.zeros(3 * self.L, **opt)
        self._err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._ids = self.indices
        if narrow_ids and on_gpu and indices.dtype == torch.int64 and self.num_nodes <= 0x7FFFFFFF:
            try:
                self._ids = self.indices.to(torch.int32)
            except torch.cuda.OutOfMemoryError:   # no room for the copy: sample from the 64-bit array
                self._ids = self.indices
        self._dtype = 0 if self._ids.dtype == torch.int32 else 1
        # every call draws from fresh random streams: call c, layer l uses stream c * L + l
        # (``stream_base`` can be saved and restored to resume a run)
        self.stream_base = 0

    def sample(self, seeds: torch.Tensor, seeds_ptr: torch.Tensor,
               counts_out: Optional[torch.Tensor] = None) -> None:
        """Enqueue one super-batch on the current stream.  ``seeds`` int64 [S] and
        ``seeds_ptr`` int64 [B+1] are CUDA tensors; ``counts_out`` (int64 [3L], CUDA) receives
        {S_l, E_l, U_l} per layer instead of the internal buffer."""
        if seeds.numel() > self.max_seeds or seeds_ptr.numel() != self.B + 1:
            raise ValueError("super-batch exceeds the sampler's declared shape")
        counts = self._counts if counts_out is None else counts_out
        rc = cabi().gsb_graphsage_sample(
            C.c_void_p(self.indptr.data_ptr()), C.c_void_p(self._ids.data_ptr()), self._dtype,
            C.c_int64(self.indptr.numel() - 1), C.c_int64(self.num_nodes), C.c_void_p(seeds.data_ptr()), C.c_void_p(seeds_ptr.data_ptr()),
            C.c_int64(self.B), C.c_int64(seeds.numel()), self.L, self._fan, C.c_uint64(self.seed),
            C.c_uint32(self.stream_base & 0xFFFFFFFF), self._bufs, C.c_void_p(counts.data_ptr()), C.c_void_p(self._ws.data_ptr()),
            C.c_size_t(self._ws.numel()), C.c_void_p(self._err.data_ptr()),
            C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        if rc != 0:
            raise RuntimeError("gsb_graphsage_sample: %s (%s)" % (
                cabi().gsb_status_string(rc).decode(), cabi().gsb_last_cuda_error().decode()))
        self.stream_base += self.L

    def capture(self) -> None:
        """Record the whole pipeline into a CUDA graph (``max_seeds`` seed slots, the sampler's own
        input buffers).  The recording fixes the random streams: every replay draws from the
        streams of the recorded call, so replays of the same seeds repeat the same sample.  Afterwards :meth:`replay` copies a super-batch into those buffers and
        launches the graph: one launch instead of about 36, which removes the launch gaps of a
        single stream (measured 1.46 -> 1.41 ms per step on the 2.4 M-node benchmark graph; with
        two or more samplers in flight on their own streams the gaps are hidden anyway)."""
        self._in_seeds = torch.zeros(self.max_seeds, dtype=torch.int64, device=self.device)
        self._in_ptr = torch.zeros(self.B + 1, dtype=torch.int64, device=self.device)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        base = self.stream_base
        with torch.cuda.stream(side):
            self.sample(self._in_seeds, self._in_ptr)      # warm-up outside the capture
        self.stream_base = base                            # the recorded call draws from these streams
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        before = kernel_launches()
        self._cuda_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._cuda_graph, stream=side, capture_error_mode="relaxed"):
            self.sample(self._in_seeds, self._in_ptr)
        self._graph_launches = kernel_launches() - before
        self.replayed_launches = 0

    def replay(self, seeds: torch.Tensor, seeds_ptr: torch.Tensor) -> None:
        """Enqueue one super-batch through the recorded graph on the current stream."""
        if getattr(self, "_cuda_graph", None) is None:
            raise RuntimeError("call capture() first")
        if seeds.numel() > self.max_seeds or seeds_ptr.numel() != self.B + 1:
            raise ValueError("super-batch exceeds the sampler's declared shape")
        self._in_seeds[:seeds.numel()].copy_(seeds, non_blocking=True)
        self._in_ptr.copy_(seeds_ptr, non_blocking=True)
        self._cuda_graph.replay()
        self.replayed_launches += self._graph_launches   # kernels run by replays (not counted by the library)

    def counts(self) -> List[List[int]]:
        """Synchronises and returns [[S_l, E_l, U_l]] of the last :meth:`sample`."""
        c = self._counts.cpu().tolist()
        self.check()
        return [c[3 * l:3 * l + 3] for l in range(self.L)]

    def check(self) -> None:
        err = int(self._err.item())
        if err:
            raise RuntimeError("sampler reported device-side error bits 0x%x "
                               "(1 prefix wait, 2 table full, 4 missing id, 8 capacity, 16 bad id)" % err)

    def layer(self, l: int, counts: Sequence[int]) -> dict:
        """Views of layer ``l`` narrowed to the live sizes ``counts`` = [S, E, U]."""
        S, E, U = counts
        t = self.layers[l]
        return dict(sub_indptr=t["sub_indptr"][:S + 1], rows=t["rows"][:E], cols=t["cols"][:E],
                    select=t["sel"][:E], edge_ptr=t["edge_ptr"], unique=t["unique"][:U],
                    unique_ptr=t["unique_ptr"], block_row=t["block_row"][:E],
                    block_col=t["block_col"][:E])
