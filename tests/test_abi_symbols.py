"""The shared library must load without a GPU and export every entry point the header
declares (no compute call is made here)."""
import ctypes
import os

from tests import abi


def test_library_exports_every_declared_symbol():
    from gsampler_b200 import build

    build.build_cuda()
    assert os.path.exists(abi.LIB)
    lib = ctypes.CDLL(abi.LIB)
    names = abi.declared_symbols()
    assert len(names) >= 12
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    lib.gsb_abi_version.restype = ctypes.c_int
    assert lib.gsb_abi_version() >= 1
    lib.gsb_status_string.restype = ctypes.c_char_p
    assert lib.gsb_status_string(0) == b"ok"
    lib.gsb_sample_cols_workspace_bytes.restype = ctypes.c_size_t
    assert lib.gsb_sample_cols_workspace_bytes(ctypes.c_int64(1000), ctypes.c_int64(10)) > 0


def test_argument_validation_without_device():
    lib = abi.lib()
    # null pointers / bad sizes are rejected before any CUDA call
    rc = lib.gsb_sample_cols(None, None, 1, abi.i64(4), None, abi.i64(4), None, abi.i64(2), 0,
                             ctypes.c_uint64(0), ctypes.c_uint32(0), None, None, None, None,
                             abi.i64(8), None, None, ctypes.c_size_t(0), None, None)
    assert rc == 1
    rc = lib.gsb_batch_relabel(None, None, abi.i64(0), abi.i64(0), None, None, None, abi.i64(0),
                               abi.i64(0), None, abi.i64(0), None, None, None, None,
                               ctypes.c_size_t(0), None, None)
    assert rc == 1
