"""Loads the reference's OWN Python package (python/gs of gSampler, staged unmodified under
oracle/_ref/python by oracle/build_ref.py) on top of this repository's libraries, the way a
maintainer would switch an installation over:

* ``torch.classes.load_library(<package>/libgs.so)`` -- the one line of gs/__init__.py that binds
  the native library -- is answered with this repository's ``libgs_b200_torch.so`` (already
  loaded by ``import gsampler_b200``);
* ``dgl`` and ``ogb`` are not installed here, and the sampling path only uses DGL to wrap the
  relabelled COO into a block object and to gather rows of pinned tensors, so small stand-ins
  are put into ``sys.modules``: a block that keeps what it was built from, and a row gather
  that calls this library's kernel.

Nothing of the staged package is edited.  Test infrastructure only."""
import importlib
import os
import sys
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class UnitGraph(object):
    """What dgl.heterograph_index.create_unitgraph_from_coo / _csr were given."""

    def __init__(self, kind, num_src, num_dst, a, b, e_ids=None):
        self.kind, self.num_src, self.num_dst, self.a, self.b, self.e_ids = kind, num_src, num_dst, a, b, e_ids


class DGLBlock(object):
    def __init__(self, hgidx, ntypes=None, etypes=None):
        self.index = hgidx
        self.srcdata, self.dstdata, self.edata = {}, {}, {}

    def num_src_nodes(self):
        return self.index.num_src

    def num_dst_nodes(self):
        return self.index.num_dst

    def coo(self):
        assert self.index.kind == "coo"
        return self.index.a, self.index.b


def _install_stubs():
    import torch

    if "dgl" in sys.modules and not getattr(sys.modules["dgl"], "_gs_stub", False):
        return  # a real DGL is installed: use it
    dgl = types.ModuleType("dgl")
    dgl._gs_stub = True
    het = types.ModuleType("dgl.heterograph")
    het.DGLBlock = DGLBlock
    hidx = types.ModuleType("dgl.heterograph_index")
    hidx.create_unitgraph_from_coo = lambda nt, ns, nd, row, col, formats=None: UnitGraph("coo", ns, nd, row, col)
    hidx.create_unitgraph_from_csr = (lambda nt, ns, nd, indptr, indices, e_ids, formats=None, transpose=False:
                                      UnitGraph("csc" if transpose else "csr", ns, nd, indptr, indices, e_ids))
    utils = types.ModuleType("dgl.utils")
    utils.gather_pinned_tensor_rows = lambda data, index: torch.ops.gs_ops._CAPI_GatherRows(data, index)
    data = types.ModuleType("dgl.data")
    data.RedditDataset = object
    fn = types.ModuleType("dgl.function")
    loading = types.ModuleType("dgl.dataloading")
    loading.DataLoader = object
    loading.MultiLayerFullNeighborSampler = object
    dgl.heterograph, dgl.heterograph_index, dgl.utils, dgl.data, dgl.function, dgl.dataloading = (
        het, hidx, utils, data, fn, loading)
    ogb = types.ModuleType("ogb")
    npp = types.ModuleType("ogb.nodeproppred")
    npp.DglNodePropPredDataset = object
    ogb.nodeproppred = npp
    for m in (dgl, het, hidx, utils, data, fn, loading, ogb, npp):
        sys.modules[m.__name__] = m


def load():
    """The staged ``gs`` package bound to this repository's libraries, or None when it has not
    been staged (``python oracle/build_ref.py`` needs the reference tree)."""
    pkg_root = os.path.join(ROOT, "oracle", "_ref", "python")
    if not os.path.isdir(os.path.join(pkg_root, "gs")):
        return None
    if "gs" in sys.modules:
        return sys.modules["gs"]
    import torch

    import gsampler_b200  # noqa: F401  (registers gs_classes.Graph and gs_ops from the new libraries)

    _install_stubs()
    real = torch.classes.load_library

    def load_library(path):
        if os.path.basename(path) == "libgs.so":
            return None  # the new libraries are loaded already and register the same names
        return real(path)

    torch.classes.load_library = load_library
    sys.path.insert(0, pkg_root)
    try:
        return importlib.import_module("gs")
    finally:
        sys.path.remove(pkg_root)
        torch.classes.load_library = real
