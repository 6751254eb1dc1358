"""gsampler_b200 -- gSampler's matrix-centric sampling hot path on B200 (sm_100a).

Importing the package loads the two in-tree shared libraries (CUDA kernels behind
the C ABI of ``include/gsb200.h``; the C++ host layer that registers
``torch.classes.gs_classes.Graph`` and ``torch.ops.gs_ops``) and exposes the same
Python surface as gSampler's ``gs`` package (python/gs/__init__.py:1-13 there):
``Matrix``, ``BatchMatrix``, ``jit.compile``, ``ops``, ``Graph`` and the format
constants.  There is no CPU or pure-PyTorch fallback: if the libraries are
missing the import fails.
"""
import os

import torch

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_CUDA = os.path.join(_HERE, "libgsb200.so")
LIB_TORCH = os.path.join(_HERE, "libgs_b200_torch.so")


def _load():
    missing = [p for p in (LIB_CUDA, LIB_TORCH) if not os.path.exists(p)]
    if missing:
        raise ImportError(
            "gsampler_b200: native libraries not built (%s). Run `python -m gsampler_b200.build` "
            "(needs nvcc); there is no fallback implementation." % ", ".join(missing))
    import ctypes

    ctypes.CDLL(LIB_CUDA, mode=ctypes.RTLD_GLOBAL)
    torch.classes.load_library(LIB_TORCH)


_load()

from .format import _COO, _CSC, _CSR  # noqa: E402
from .matrix_api import Matrix, BatchMatrix  # noqa: E402
from . import jit, ops, utils  # noqa: E402
from .jit import compile  # noqa: E402,A001

Graph = torch.classes.gs_classes.Graph


def gather_rows(data: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``data[index]`` along the first dimension by the library's row-gather kernel: ``data`` on
    the index's GPU or in pinned host memory (read in place), no synchronisation.  This is the
    feature fetch that follows sampling (examples/graphsage/graphsage_e2e.py:111-118 in
    gSampler, where DGL's ``gather_pinned_tensor_rows`` does it).  A bad index is reported by
    ``check_async_errors()``."""
    return torch.ops.gs_ops._CAPI_GatherRows(data, index)


def check_async_errors() -> None:
    """Raise if a sync-free operator (``gather_rows``) met invalid input since the last check."""
    torch.ops.gs_ops._CAPI_CheckAsyncErrors()

__all__ = ["Matrix", "BatchMatrix", "Graph", "gather_rows", "check_async_errors", "jit", "ops", "utils", "compile", "_COO", "_CSC", "_CSR"]
from .pipeline import GraphSAGESampler  # noqa: E402
