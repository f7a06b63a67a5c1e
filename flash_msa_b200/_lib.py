"""ctypes binding of libflash_msa_b200.so.  There is no fallback: if the library is missing or a
call is rejected, an exception is raised."""
from __future__ import annotations

import ctypes
import os
import re
from ctypes import c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# FLASH_MSA_B200_LIB selects another build of the library (e.g. one compiled with extra diagnostics).
LIB_PATH = os.environ.get("FLASH_MSA_B200_LIB") or os.path.join(PKG_DIR, "libflash_msa_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(PKG_DIR), "include", "flash_msa_b200.h")

FMSA_OK = 0
FMSA_DTYPE_BF16, FMSA_DTYPE_FP16 = 0, 1
_ERRORS = {
    -1: (ValueError, "invalid argument (shape, alignment or null pointer)"),
    -2: (NotImplementedError, "request outside the implemented envelope"),
    -3: (RuntimeError, "workspace too small"),
    -4: (RuntimeError, "CUDA runtime refused the launch"),
}


class FmsaTensor(ctypes.Structure):
    """Mirror of ``fmsa_tensor``: base pointer + element strides of a (B,H,S,128) bf16 tensor."""
    _fields_ = [("ptr", c_void_p), ("stride_b", c_int64), ("stride_h", c_int64), ("stride_s", c_int64)]


_lib = None


def declared_symbols() -> list[str]:
    """Entry points declared in include/flash_msa_b200.h."""
    with open(HEADER_PATH) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fmsa_[a-z0-9_]+)\s*\(", text)))


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m flash_msa_b200.build` "
                "(flash_msa_b200 has no CPU or PyTorch fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(lib):
    P = c_void_p
    lib.fmsa_abi_version.restype = c_int
    lib.fmsa_abi_version.argtypes = []
    lib.fmsa_umma_selftest.restype = c_int
    lib.fmsa_umma_selftest.argtypes = [P, P, P, c_int, c_int, c_int, P, P]
    lib.fmsa_pipeline_selftest.restype = c_int
    lib.fmsa_pipeline_selftest.argtypes = [P, c_int64, P, P, P, P, P, c_int, c_int64, P, P]
    lib.fmsa_select_topk.restype = c_int
    lib.fmsa_select_topk.argtypes = [P, P, c_int64, c_int32, c_int32, P]
    lib.fmsa_reverse_index_workspace_bytes.restype = c_size_t
    lib.fmsa_reverse_index_workspace_bytes.argtypes = [c_int64, c_int32]
    lib.fmsa_reverse_index.restype = c_int
    lib.fmsa_reverse_index.argtypes = [P, P, P, P, c_int64, c_int32, c_int32, P, c_size_t, P]
    lib.fmsa_reverse_index_static.restype = c_int
    lib.fmsa_reverse_index_static.argtypes = [P, P, P, P, c_int64, c_int32, c_int32, P]
    T = ctypes.POINTER(FmsaTensor)
    PB = ctypes.POINTER(FmsaProblem)
    lib.fmsa_select_scores.restype = c_int
    lib.fmsa_select_scores.argtypes = [T, T, P, c_int32, c_int32, c_int32, c_int32, c_float, c_int32, P, P, P]
    lib.fmsa_select_fused.restype = c_int
    lib.fmsa_select_fused.argtypes = [T, T, P, c_int32, c_int32, c_int32, c_int32, c_int32, c_float, c_int32, P, P, P]
    lib.fmsa_fwd_partial_slots.restype = c_int64
    lib.fmsa_fwd_partial_slots.argtypes = [PB, c_int32, c_int32]
    lib.fmsa_sparse_fwd.restype = c_int
    lib.fmsa_sparse_fwd.argtypes = [PB, T, T, T, T, T, P, P, P, P, c_int64, c_int32, c_int32, c_int32, c_int32, P, P, P]
    lib.fmsa_sparse_fwd_combine.restype = c_int
    lib.fmsa_sparse_fwd_combine.argtypes = [PB, P, P, P, P, P, P, P, c_int32, c_int32, c_int32, P]
    lib.fmsa_bwd_delta.restype = c_int
    lib.fmsa_bwd_delta.argtypes = [P, T, P, c_int32, c_int32, c_int32, c_int32, P]
    lib.fmsa_sparse_bwd.restype = c_int
    lib.fmsa_sparse_bwd.argtypes = [PB, T, T, T, T, T, T, P, P, P, P, P, P, P, c_int64, c_int32, P, P, P, c_int32, c_int32,
                                    c_int32, c_int32, P, P, P, P]
    lib.fmsa_sparse_bwd_combine.restype = c_int
    lib.fmsa_sparse_bwd_combine.argtypes = [PB, P, P, c_int64, c_int32, P, P, T, T, P, c_int32, c_int32, c_int32, P]
    lib.fmsa_cast_scaled.restype = c_int
    lib.fmsa_cast_scaled.argtypes = [P, P, c_int64, P, c_float, c_int32, P]
    lib.fmsa_cast_scaled_rows.restype = c_int
    lib.fmsa_cast_scaled_rows.argtypes = [P, T, c_int32, c_int32, c_int32, P, c_float, c_int32, P]
    lib.fmsa_copy2d_async.restype = c_int
    lib.fmsa_copy2d_async.argtypes = [P, ctypes.c_size_t, P, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, P]


class FmsaProblem(ctypes.Structure):
    """Mirror of ``fmsa_problem``."""
    _fields_ = [("B", c_int32), ("S", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("Hp", c_int32),
                ("Hpkv", c_int32), ("top_k_blocks", c_int32), ("scale", c_float), ("dtype", c_int32),
                ("doc_start", ctypes.c_void_p)]


def check(status: int, what: str) -> None:
    if status == FMSA_OK:
        return
    exc, msg = _ERRORS.get(status, (RuntimeError, f"status {status}"))
    raise exc(f"{what}: {msg}")
