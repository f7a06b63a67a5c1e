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
    assert lib.fmsa_abi_version() == 8          # 8: fmsa_select_fused (block scores and top-k in one kernel)


def test_argument_errors_do_not_launch():
    lib = _lib.load()
    assert lib.fmsa_select_topk(None, None, 1, 128, 1, None) == -1
    assert lib.fmsa_reverse_index_workspace_bytes(0, 128) == 0
    assert lib.fmsa_reverse_index_workspace_bytes(2, 1024) > 0
    # null pointers / nonsense sizes are rejected before anything touches the device
    assert lib.fmsa_copy2d_async(None, 0, None, 0, 0, 0, None) == -1
    assert lib.fmsa_cast_scaled(None, None, 16, None, 1.0, 0, None) == -1
    assert lib.fmsa_cast_scaled_rows(None, None, 1, 1, 128, None, 1.0, 0, None) == -1
    assert lib.fmsa_bwd_delta(None, None, None, 1, 128, 1, 0, None) == -1
    pb = _lib.FmsaProblem(1, 100, 4, 2, 2, 2, 1, 0.1, 0)      # S is not a multiple of 128
    assert lib.fmsa_fwd_partial_slots(ctypes.byref(pb), 1, 0) <= 0


def test_fused_selection_refuses_what_it_cannot_hold():
    """More selected blocks than the fused kernel's register list holds is answered with FMSA_ERR_UNSUPPORTED (the caller
    then uses the score kernel and the top-k kernel), bad sizes with FMSA_ERR_ARGUMENT - both before anything touches the device."""
    lib = _lib.load()
    t = _lib.FmsaTensor()                    # never dereferenced: the size checks come first
    out = ctypes.c_void_p(16)
    big = 129 * 128
    assert lib.fmsa_select_fused(ctypes.byref(t), ctypes.byref(t), out, 1, 1, 1, big, 65, 0.1, 0, None, None, None) == -2
    assert lib.fmsa_select_fused(ctypes.byref(t), ctypes.byref(t), out, 1, 1, 1, 1024, 9, 0.1, 0, None, None, None) == -1
    assert lib.fmsa_select_fused(ctypes.byref(t), ctypes.byref(t), None, 1, 1, 1, 1024, 4, 0.1, 0, None, None, None) == -1
