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
LIB_PATH = os.environ.get("MARIAN_I8_LIBRARY") or os.path.join(_HERE, "libmarian_i8.so")   # (the variable selects another build of the same ABI)

MI8_F32, MI8_F16 = 0, 1

class Mi8GemmRecord(ctypes.Structure):
    """mi8_gemm_record of include/marian_i8_measure.h."""
    _fields_ = [("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("out_bytes", ctypes.c_int), ("us", ctypes.c_float),
                ("rows_computed", ctypes.c_int)]


class Mi8KernelTime(ctypes.Structure):
    """mi8_kernel_time of include/marian_i8_measure.h."""
    _fields_ = [("name", ctypes.c_char * 160), ("launches", ctypes.c_longlong), ("total_us", ctypes.c_double)]


class Mi8dConfig(ctypes.Structure):
    """mi8d_config of include/marian_i8_decode.h."""
    _fields_ = [(n, ctypes.c_int) for n in ("dim_emb", "dim_ffn", "heads", "enc_depth", "dec_depth", "vocab", "ssru", "max_rows",
                                             "max_batch", "max_steps", "max_src")]


# Every symbol include/marian_i8_decode.h declares.
DECODE_EXPORTS = ["mi8d_arena_bytes", "mi8d_create", "mi8d_destroy", "mi8d_set_weight", "mi8d_set_param", "mi8d_set_positions",
                  "mi8d_start", "mi8d_encode", "mi8d_step", "mi8d_last_logits", "mi8d_history_reuse",
                  "mi8g_embed", "mi8g_add_layernorm", "mi8g_quantize_slot", "mi8g_attention1", "mi8g_lse_topk", "mi8g_nbest_merge",
                  "mi8g_output_scratch_bytes", "mi8g_output_topk", "mi8d_keep_logits", "mi8d_search", "mi8d_set_option", "mi8d_set_packed8_weight",
                  "mi8g_affine_slot", "mi8g_affine_slot_add_layernorm"]

# Every symbol include/marian_packed8.h declares.
PACKED8_EXPORTS = ["mi8p_packed_bytes", "mi8p_prepare_b_f32", "mi8p_unpack_b", "mi8p_quantize_rows", "mi8p_multiply", "mi8p_scratch_bytes",
                   "mi8p_gemm_int8_packed"]

# Every symbol include/marian_i8.h declares.
EXPORTS = [
    "mi8_version", "mi8_strerror", "mi8_last_cuda_error", "mi8_last_cuda_error_string",
    "mi8_workspace_bytes", "mi8_workspace_init", "mi8_poll_status", "mi8_clear_status",
    "mi8_max_absolute_f32", "mi8_quantize_f32_i8", "mi8_prepare_a_f32", "mi8_prepare_b_f32",
    "mi8_multiply_i8", "mi8_multiply_i8_ex", "mi8_multiply_i8_rows_from", "mi8_multiply_f32_slot", "mi8_multiply_i8_static", "mi8_affine_f32", "mi8_multiply_plan",
    "mi8_set_pdl", "mi8_multiply_i8_multi", "mi8_transpose_f32",
]

# Every symbol include/marian_i8_measure.h declares (measurement and test aids, not part of the drop-in surface).
MEASURE_EXPORTS = ["mi8_launch_count", "mi8_launch_count_reset", "mi8_measure_int8_peak", "mi8_kernel_times_begin", "mi8_kernel_times_end",
                   "mi8_profile_begin", "mi8_profile_end", "mi8_test_wait_fault", "mi8d_search_stats", "mi8_trace_begin", "mi8_trace_end"]


class Mi8dSearchConfig(ctypes.Structure):
    _fields_ = [("beam", ctypes.c_int), ("max_length_factor", ctypes.c_float), ("normalize", ctypes.c_float),
                ("word_penalty", ctypes.c_float), ("eos_id", ctypes.c_int)]


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
    L.mi8_multiply_i8_rows_from.argtypes = [vp, vp, ci, ci, ci, vp, vp, cf, vp, ci, vp, ci, vp, sz, vp, vp, vp, ci, ci]
    L.mi8_multiply_i8_rows_from.restype = ci
    L.mi8_multiply_f32_slot.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp, cf, vp, ci, vp, ci, vp, vp]
    L.mi8_multiply_f32_slot.restype = ci
    L.mi8_transpose_f32.argtypes = [vp, ci, ci, ci, vp, vp]
    L.mi8_transpose_f32.restype = ci
    L.mi8_multiply_i8_multi.argtypes = [vp, vp, ci, ci, ci, ci, vp, ctypes.POINTER(vp), cf, ctypes.POINTER(vp), ci, ctypes.POINTER(vp), ci, vp, sz, vp]
    L.mi8_multiply_i8_multi.restype = ci
    L.mi8_multiply_i8_static.argtypes = [vp, vp, ci, ci, ci, vp, vp, cf, vp, ci, vp, ci, vp]
    L.mi8_multiply_i8_static.restype = ci
    L.mi8_affine_f32.argtypes = [vp, ci, ci, vp, vp, ci, vp, cf, ci, vp, ci, vp, vp, sz, vp]
    L.mi8_multiply_plan.argtypes = [ci, ci, ci, ci, ci, ctypes.POINTER(ci * 8)]
    L.mi8_measure_int8_peak.argtypes = [ci, ctypes.POINTER(cf), vp]
    L.mi8_measure_int8_peak.restype = ci
    L.mi8_kernel_times_begin.restype = ci
    L.mi8_kernel_times_end.argtypes = [ctypes.POINTER(Mi8KernelTime), ci, ctypes.POINTER(ci)]
    L.mi8_kernel_times_end.restype = ci
    L.mi8_set_pdl.argtypes = [ci]
    L.mi8_set_pdl.restype = None
    L.mi8_profile_begin.argtypes = [ci]
    L.mi8_profile_begin.restype = ci
    L.mi8_profile_end.argtypes = [ctypes.POINTER(Mi8GemmRecord), ci, ctypes.POINTER(ci)]
    L.mi8_profile_end.restype = ci
    L.mi8_launch_count.restype = ctypes.c_ulonglong
    L.mi8_trace_begin.argtypes = [vp, ci]
    L.mi8_trace_begin.restype = ci
    L.mi8_trace_end.restype = ci
    L.mi8_test_wait_fault.argtypes = [ci, ctypes.c_uint]
    L.mi8_test_wait_fault.restype = None
    L.mi8d_search_stats.argtypes = [vp, ctypes.POINTER(ctypes.c_double * 4), ci]
    L.mi8d_search_stats.restype = ci
    L.mi8p_packed_bytes.restype = sz
    L.mi8p_packed_bytes.argtypes = [ci, ci]
    L.mi8p_unpack_b.argtypes = [vp, ci, ci, vp, vp]
    L.mi8p_prepare_b_f32.argtypes = [vp, ci, ci, vp, vp]
    L.mi8p_quantize_rows.argtypes = [vp, ci, ci, vp, vp, vp, vp, vp]
    L.mi8p_multiply.argtypes = [vp] * 8 + [ci, ci, ci, vp, ci, vp, vp, vp, sz, vp, ci, ci]
    L.mi8p_scratch_bytes.restype = sz
    L.mi8p_scratch_bytes.argtypes = [ci, ci]
    L.mi8p_gemm_int8_packed.argtypes = [vp] * 7 + [ci, ci, ci, vp, sz, vp, sz, vp]
    L.mi8_launch_count_reset.restype = None
    for name in ("mi8_workspace_init", "mi8_poll_status", "mi8_clear_status", "mi8_max_absolute_f32",
                 "mi8_quantize_f32_i8", "mi8_prepare_a_f32", "mi8_prepare_b_f32", "mi8_multiply_i8",
                 "mi8_multiply_i8_ex", "mi8_affine_f32", "mi8_multiply_plan"):
        getattr(L, name).restype = ci
    cfgp = ctypes.POINTER(Mi8dConfig)
    L.mi8d_arena_bytes.restype = sz
    L.mi8d_arena_bytes.argtypes = [cfgp]
    L.mi8d_create.argtypes = [cfgp, vp, sz, vp, sz, ctypes.POINTER(vp)]
    L.mi8d_destroy.argtypes = [vp]
    L.mi8d_destroy.restype = None
    L.mi8d_set_weight.argtypes = [vp, ctypes.c_char_p, vp, ci, ci]
    L.mi8d_set_param.argtypes = [vp, ctypes.c_char_p, vp]
    L.mi8d_set_packed8_weight.argtypes = [vp, ctypes.c_char_p, vp, vp, vp, vp, ci, ci]
    L.mi8d_set_packed8_weight.restype = ci
    L.mi8d_set_positions.argtypes = [vp, vp]
    L.mi8d_start.argtypes = [vp, vp, vp, ci, ci, vp]
    L.mi8d_encode.argtypes = [vp, vp, vp, ci, ci, vp]
    L.mi8d_encode.restype = ci
    L.mi8d_step.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, vp, vp, vp, vp]
    L.mi8d_history_reuse.argtypes = [vp, ctypes.POINTER(ctypes.c_uint * 2), ci]
    L.mi8d_history_reuse.restype = ci
    L.mi8d_search.argtypes = [vp, vp, vp, ci, ci, ctypes.POINTER(Mi8dSearchConfig), vp, ci, vp, vp, ctypes.POINTER(ctypes.c_ulonglong),
                              ctypes.POINTER(ctypes.c_ulonglong), vp]
    L.mi8d_search.restype = ci
    L.mi8d_set_option.argtypes = [vp, ci, ci]
    L.mi8d_set_option.restype = ci
    L.mi8d_keep_logits.argtypes = [vp, ci]
    L.mi8d_keep_logits.restype = ci
    L.mi8g_output_scratch_bytes.argtypes = [ci, ci]
    L.mi8g_output_scratch_bytes.restype = sz
    L.mi8g_output_topk.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp, ci, vp, vp, sz, vp, vp, vp, vp]
    L.mi8g_output_topk.restype = ci
    L.mi8d_last_logits.argtypes = [vp]
    L.mi8d_last_logits.restype = vp
    L.mi8g_embed.argtypes = [vp, vp, vp, ci, cf, ci, ci, vp, vp, vp, vp]
    L.mi8g_add_layernorm.argtypes = [vp, vp, vp, vp, cf, ci, ci, vp, vp, vp, vp]
    L.mi8g_quantize_slot.argtypes = [vp, sz, vp, vp, vp, vp]
    L.mi8g_attention1.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp, vp, vp]
    L.mi8g_lse_topk.argtypes = [vp, ci, ci, ci, vp, vp, vp, vp]
    L.mi8g_nbest_merge.argtypes = [vp, vp, ci, ci, ci, ci, vp, vp, vp, vp]
    L.mi8g_affine_slot.argtypes = [vp, vp, vp, vp, ci, ci, ci, cf, vp, ci, vp, vp, ci, ci, vp]
    L.mi8g_affine_slot_add_layernorm.argtypes = [vp, vp, vp, vp, ci, ci, ci, cf, vp, vp, vp, vp, cf, vp, vp, vp, vp, vp]
    for name in ("mi8g_embed", "mi8g_add_layernorm", "mi8g_quantize_slot", "mi8g_attention1", "mi8g_lse_topk", "mi8g_nbest_merge",
                 "mi8g_affine_slot", "mi8g_affine_slot_add_layernorm"):
        getattr(L, name).restype = ci
    for name in ("mi8d_create", "mi8d_set_weight", "mi8d_set_param", "mi8d_set_positions", "mi8d_start", "mi8d_step"):
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
