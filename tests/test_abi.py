"""CPU-side checks of the drop-in boundary: the shared library loads and exports every symbol
the public header declares (no kernel is launched here)."""
import ctypes
import os

from flash_msa_b200 import _lib, build


def test_library_builds_and_exports_declared_symbols():
    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    names = _lib.declared_symbols()
    assert "fmsa_select_topk" in names and "fmsa_reverse_index" in names
    for name in names:
        assert hasattr(lib, name), name
    assert lib.fmsa_abi_version() >= 1


def test_argument_errors_do_not_launch():
    lib = _lib.load()
    assert lib.fmsa_select_topk(None, None, 1, 128, 1, None) == -1
    assert lib.fmsa_reverse_index_workspace_bytes(0, 128) == 0
    assert lib.fmsa_reverse_index_workspace_bytes(2, 1024) > 0
