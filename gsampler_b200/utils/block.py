"""Message-flow block returned by ``to_dgl_block``.

gSampler wraps the relabelled COO into a ``DGLBlock`` (python/gs/utils/to_dgl_block.py:5-23).
DGL is an optional dependency here: ``Block`` carries the same information (relabelled
row/col ids, number of source / destination nodes, ``srcdata`` / ``edata`` dictionaries) as
plain tensors and converts to a real ``DGLBlock`` on request when DGL is importable.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch


class Block(object):
    __slots__ = ("row", "col", "indptr", "num_src", "num_dst", "srcdata", "dstdata", "edata")

    def __init__(self, row: Optional[torch.Tensor], col: Optional[torch.Tensor], num_src: int,
                 num_dst: int, indptr: Optional[torch.Tensor] = None):
        self.row = row
        self.col = col
        self.indptr = indptr
        self.num_src = int(num_src)
        self.num_dst = int(num_dst)
        self.srcdata: Dict[str, torch.Tensor] = {}
        self.dstdata: Dict[str, torch.Tensor] = {}
        self.edata: Dict[str, torch.Tensor] = {}

    def num_src_nodes(self) -> int:
        return self.num_src

    def num_dst_nodes(self) -> int:
        return self.num_dst

    def num_edges(self) -> int:
        return int(self.row.numel())

    def edges(self):
        return self.row, self.col

    def to_dgl(self):
        import dgl  # optional
        from dgl.heterograph import DGLBlock

        hgidx = dgl.heterograph_index.create_unitgraph_from_coo(
            2, self.num_src, self.num_dst, self.row, self.col, formats=["coo", "csr", "csc"])
        blk = DGLBlock(hgidx, (["_N"], ["_N"]), ["_E"])
        for k, v in self.srcdata.items():
            blk.srcdata[k] = v
        for k, v in self.edata.items():
            blk.edata[k] = v
        return blk

    def __repr__(self):
        return "Block(num_src_nodes=%d, num_dst_nodes=%d, num_edges=%d)" % (
            self.num_src, self.num_dst, self.num_edges())


def create_block_from_coo(row, col, num_src, num_dst) -> Block:
    return Block(row, col, num_src, num_dst)


def create_block_from_csc(indptr, indices, e_ids, num_src, num_dst) -> Block:
    blk = Block(indices, None, num_src, num_dst, indptr=indptr)
    if e_ids is not None:
        blk.edata["_ID"] = e_ids
    return blk
