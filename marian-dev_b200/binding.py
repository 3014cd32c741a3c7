"""ctypes binding of libmarian_i8.so (the C ABI declared in include/marian_i8.h).

The shared object is built in-tree by ``csrc/Makefile``.  Nothing here falls back to another
implementation: if the library is missing the import raises, and every non-zero status raises
``Mi8Error`` the way Marian's host code turns an error into ABORT (src/common/logging.h:100-140).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmarian_i8.so")

MI8_F32, MI8_F16 = 0, 1

# Every symbol include/marian_i8.h declares.
EXPORTS = [
    "mi8_version", "mi8_strerror", "mi8_last_cuda_error", "mi8_last_cuda_error_string",
    "mi8_workspace_bytes", "mi8_workspace_init", "mi8_poll_status", "mi8_clear_status",
    "mi8_max_absolute_f32", "mi8_quantize_f32_i8", "mi8_prepare_a_f32", "mi8_prepare_b_f32",
    "mi8_multiply_i8", "mi8_multiply_i8_ex", "mi8_multiply_i8_static", "mi8_affine_f32", "mi8_multiply_plan",
    "mi8_launch_count", "mi8_launch_count_reset",
]


class Mi8Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"marian_i8 status {status}: {message}")
        self.status = status


def build_library(verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a into libmarian_i8.so (nvcc cross-compiles without a GPU)."""
    out = subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), "-B"], capture_output=True, text=True)
    if verbose or out.returncode != 0:
        print(out.stdout[-4000:])
        print(out.stderr[-8000:])
    if out.returncode != 0:
        raise RuntimeError("building libmarian_i8.so failed")
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `make -C {os.path.join(_HERE, 'csrc')}` "
                          "(there is no fallback implementation)")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz, ci, cf = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_float
    L.mi8_version.restype = ci
    L.mi8_strerror.restype = ctypes.c_char_p
    L.mi8_strerror.argtypes = [ci]
    L.mi8_last_cuda_error.restype = ci
    L.mi8_last_cuda_error_string.restype = ctypes.c_char_p
    L.mi8_workspace_bytes.restype = sz
    L.mi8_workspace_bytes.argtypes = [ci, ci, ci]
    L.mi8_workspace_init.argtypes = [vp, sz, vp]
    L.mi8_poll_status.argtypes = [ctypes.POINTER(ci)]
    L.mi8_clear_status.argtypes = [vp]
    L.mi8_max_absolute_f32.argtypes = [vp, sz, vp, vp, vp, sz, vp]
    L.mi8_quantize_f32_i8.argtypes = [vp, sz, vp, vp, vp]
    L.mi8_prepare_a_f32.argtypes = [vp, ci, ci, vp, vp, vp, sz, vp]
    L.mi8_prepare_b_f32.argtypes = [vp, ci, ci, ci, vp, vp, vp, sz, vp]
    L.mi8_multiply_i8.argtypes = [vp, vp, ci, ci, ci, vp, vp, cf, vp, ci, vp, ci, vp, vp, sz, vp]
    L.mi8_multiply_i8_ex.argtypes = [vp, vp, ci, ci, ci, vp, vp, cf, vp, ci, vp, ci, vp, vp, sz, vp, ci, ci]
    L.mi8_multiply_i8_static.argtypes = [vp, vp, ci, ci, ci, vp, vp, cf, vp, ci, vp, ci, vp]
    L.mi8_multiply_i8_static.restype = ci
    L.mi8_affine_f32.argtypes = [vp, ci, ci, vp, vp, ci, vp, cf, ci, vp, ci, vp, vp, sz, vp]
    L.mi8_multiply_plan.argtypes = [ci, ci, ci, ci, ci, ctypes.POINTER(ci * 8)]
    L.mi8_launch_count.restype = ctypes.c_ulonglong
    L.mi8_launch_count_reset.restype = None
    for name in ("mi8_workspace_init", "mi8_poll_status", "mi8_clear_status", "mi8_max_absolute_f32",
                 "mi8_quantize_f32_i8", "mi8_prepare_a_f32", "mi8_prepare_b_f32", "mi8_multiply_i8",
                 "mi8_multiply_i8_ex", "mi8_affine_f32", "mi8_multiply_plan"):
        getattr(L, name).restype = ci
    _lib = L
    return L


def check(status: int) -> None:
    """Raise Mi8Error for a non-zero mi8_status."""
    if status != 0:
        L = lib()
        msg = L.mi8_strerror(status).decode()
        if status == 5:
            msg += f" ({L.mi8_last_cuda_error_string().decode()})"
        raise Mi8Error(status, msg)


def multiply_plan(M: int, N: int, K: int, tile_m: int = 0, splits: int = 0) -> dict:
    """How the GEMM would be tiled on the current device (148 SMs are assumed without a GPU)."""
    out = (ctypes.c_int * 8)()
    check(lib().mi8_multiply_plan(M, N, K, tile_m, splits, ctypes.byref(out)))
    keys = ["tile_m", "stages", "splits", "n_tiles", "m_tiles", "grid", "smem_bytes", "sm_count"]
    return dict(zip(keys, list(out)))
