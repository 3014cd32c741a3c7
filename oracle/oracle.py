"""CPU checker for the int8 affine path: TEST INFRASTRUCTURE ONLY.

Two independent restatements of Marian's intgemm8 affine/dot sequence
(src/tensors/cpu/intgemm_interface.h:17-99, src/tensors/cpu/integer_common.h:101-111,169-182,
src/tensors/cpu/expression_graph_packable.h:153-253):

* ``numpy_*`` functions: plain NumPy, used for small cases and to cross-check the C build;
* ``COracle``: ctypes binding of ``liboracle_i8.so`` (``oracle_i8.c``), used for the larger
  parity cases and as the timed CPU baseline.

PARITY UNPINNED: the arithmetic of this path lives in the un-vendored intgemm submodule and the
reference has no test with an intgemm-typed operand, so neither restatement could be checked
against reference outputs.  Only tests, the smoke check and the bench's CPU-baseline leg may import
this module; the product package never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle_i8.so")


# --------------------------------------------------------------------------- NumPy restatement
def numpy_quant_mult(x: np.ndarray) -> np.float32:
    """computeQuantMult<intgemm8>: 127.0f / max|x| (integer_common.h:169-173); all-zero -> 1."""
    m = np.float32(np.max(np.abs(x.astype(np.float32, copy=False)))) if x.size else np.float32(0)
    if m == 0:
        return np.float32(1.0)
    return np.float32(127.0) / m


def numpy_quantize(x: np.ndarray, quant_mult: np.float32) -> np.ndarray:
    """Int8::PrepareA: fp32 multiply, round half to even, saturate to [-127, 127]."""
    y = np.rint(x.astype(np.float32, copy=False) * np.float32(quant_mult))
    return np.clip(y, -127, 127).astype(np.int8)


def numpy_prepare_b(w: np.ndarray, w_is_nk: bool = False):
    """marian-conv intgemm8 branch: W[K,N] -> (Bt[N,K] int8, quantMult) (expression_graph_packable.h:160-201)."""
    qm = numpy_quant_mult(w)
    wt = w if w_is_nk else np.ascontiguousarray(w.T)
    return numpy_quantize(wt, qm), qm


def numpy_multiply_i32(aq: np.ndarray, bt: np.ndarray) -> np.ndarray:
    """Exact int32 accumulators: acc[i,j] = sum_k Aq[i,k] * Bt[j,k]."""
    return aq.astype(np.int32) @ bt.astype(np.int32).T


def numpy_unquant_mult(qa, qb, scale=1.0) -> np.float32:
    """1.0f / (qa*qb), then * scale, all in fp32 (intgemm_interface.h:69-70)."""
    u = np.float32(1.0) / (np.float32(qa) * np.float32(qb))
    return np.float32(u * np.float32(scale))


def numpy_unquantize(acc: np.ndarray, unquant, bias=None, relu=False) -> np.ndarray:
    """float(acc)*unquant (+bias), then the separate ReLU (expression_operators.cpp:721-731)."""
    out = acc.astype(np.float32) * np.float32(unquant)
    if bias is not None:
        out = out + bias.astype(np.float32).reshape(1, -1)
    if relu:
        out = np.where(out > 0, out, np.float32(0)).astype(np.float32)
    return out.astype(np.float32)


def numpy_affine(a: np.ndarray, bt: np.ndarray, qb, bias=None, scale=1.0, relu=False):
    """Whole affineOrDotTyped sequence; returns (out fp32, acc int32, aq int8, qa)."""
    a2 = a.reshape(-1, a.shape[-1])
    qa = numpy_quant_mult(a2)
    aq = numpy_quantize(a2, qa)
    acc = numpy_multiply_i32(aq, bt)
    out = numpy_unquantize(acc, numpy_unquant_mult(qa, qb, scale), bias, relu)
    return out.reshape(a.shape[:-1] + (bt.shape[0],)), acc, aq, qa


# --------------------------------------------------------------------------- C build
def build(force: bool = False) -> str:
    """Compile oracle_i8.c with the Makefile beside it; returns the shared-object path."""
    src = os.path.join(_HERE, "oracle_i8.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _LIB


def _p(arr, ct):
    return arr.ctypes.data_as(ctypes.POINTER(ct)) if arr is not None else None


class COracle:
    """ctypes view of liboracle_i8.so."""

    def __init__(self, lib_path: str | None = None):
        if lib_path is None:
            lib_path = _LIB if os.path.exists(_LIB) else build()
        L = ctypes.CDLL(lib_path)
        f32p, i8p, i32p = (ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int8),
                           ctypes.POINTER(ctypes.c_int32))
        L.mo_max_absolute.restype = ctypes.c_float
        L.mo_max_absolute.argtypes = [f32p, ctypes.c_size_t]
        L.mo_compute_quant_mult.restype = ctypes.c_float
        L.mo_compute_quant_mult.argtypes = [f32p, ctypes.c_size_t]
        L.mo_prepare_a.restype = None
        L.mo_prepare_a.argtypes = [f32p, i8p, ctypes.c_float, ctypes.c_int, ctypes.c_int, f32p]
        L.mo_prepare_b.restype = ctypes.c_float
        L.mo_prepare_b.argtypes = [f32p, ctypes.c_int, ctypes.c_int, ctypes.c_int, i8p]
        L.mo_multiply_i32.restype = ctypes.c_int
        L.mo_multiply_i32.argtypes = [i8p, i8p, ctypes.c_int, ctypes.c_int, ctypes.c_int, i32p]
        L.mo_multiply_sat16.restype = ctypes.c_int
        L.mo_multiply_sat16.argtypes = [i8p, i8p, ctypes.c_int, ctypes.c_int, ctypes.c_int, i32p]
        L.mo_unquant_mult.restype = ctypes.c_float
        L.mo_unquant_mult.argtypes = [ctypes.c_float] * 3
        L.mo_unquantize_write.restype = None
        L.mo_unquantize_write.argtypes = [i32p, ctypes.c_int, ctypes.c_int, ctypes.c_float, f32p, ctypes.c_int, f32p]
        L.mo_affine.restype = ctypes.c_int
        L.mo_affine.argtypes = [f32p, ctypes.c_int, ctypes.c_int, i8p, ctypes.c_float, ctypes.c_int, f32p,
                                ctypes.c_float, ctypes.c_int, f32p, i8p, i32p, f32p]
        L.mo_add_layernorm.restype = None
        L.mo_add_layernorm.argtypes = [f32p, f32p, f32p, f32p, ctypes.c_float, ctypes.c_int, ctypes.c_int, f32p]
        L.mo_attention1.restype = None
        L.mo_attention1.argtypes = [f32p, f32p, f32p, f32p] + [ctypes.c_int] * 6 + [f32p]
        L.mo_lse_topk.restype = None
        L.mo_lse_topk.argtypes = [f32p, ctypes.c_int, ctypes.c_int, ctypes.c_int, f32p, f32p, i32p]
        L.mo_embed.restype = None
        L.mo_embed.argtypes = [f32p, i32p, f32p, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int, f32p]
        L.mo_ssru_cell.restype = None
        L.mo_ssru_cell.argtypes = [f32p, f32p, f32p, ctypes.c_size_t, f32p, f32p]
        L.mo_det_expf.restype = ctypes.c_float
        L.mo_det_expf.argtypes = [ctypes.c_float]
        L.mo_det_logf.restype = ctypes.c_float
        L.mo_det_logf.argtypes = [ctypes.c_float]
        L.mo_max_threads.restype = ctypes.c_int
        L.mo_set_threads.argtypes = [ctypes.c_int]
        self.L = L

    def max_threads(self) -> int:
        return int(self.L.mo_max_threads())

    def set_threads(self, n: int) -> None:
        self.L.mo_set_threads(int(n))

    def set_isa(self, isa: int) -> int:
        """Route of the int8 multiply: 0 portable C, 1 AVX2, 2 AVX512-VNNI, -1 the best the host has
        (values above that are clamped).  Returns the route in effect; all routes give identical sums."""
        self.L.mo_set_isa.restype = ctypes.c_int
        self.L.mo_set_isa.argtypes = [ctypes.c_int]
        return int(self.L.mo_set_isa(int(isa)))

    def quant_mult(self, x: np.ndarray) -> np.float32:
        x = np.ascontiguousarray(x, dtype=np.float32)
        return np.float32(self.L.mo_compute_quant_mult(_p(x, ctypes.c_float), x.size))

    def quantize(self, x: np.ndarray, qm) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.int8)
        rows = int(np.prod(x.shape[:-1])) if x.ndim > 1 else 1
        self.L.mo_prepare_a(_p(x, ctypes.c_float), _p(out, ctypes.c_int8), ctypes.c_float(float(qm)),
                            rows, x.shape[-1], None)
        return out

    def prepare_b(self, w: np.ndarray, w_is_nk: bool = False):
        w = np.ascontiguousarray(w, dtype=np.float32)
        k, n = (w.shape[1], w.shape[0]) if w_is_nk else (w.shape[0], w.shape[1])
        bt = np.empty((n, k), dtype=np.int8)
        qm = self.L.mo_prepare_b(_p(w, ctypes.c_float), k, n, int(w_is_nk), _p(bt, ctypes.c_int8))
        return bt, np.float32(qm)

    def multiply_i32(self, aq: np.ndarray, bt: np.ndarray, sat16: bool = False) -> np.ndarray:
        aq = np.ascontiguousarray(aq, dtype=np.int8)
        bt = np.ascontiguousarray(bt, dtype=np.int8)
        m, k = aq.shape
        n = bt.shape[0]
        acc = np.empty((m, n), dtype=np.int32)
        fn = self.L.mo_multiply_sat16 if sat16 else self.L.mo_multiply_i32
        rc = fn(_p(aq, ctypes.c_int8), _p(bt, ctypes.c_int8), m, k, n, _p(acc, ctypes.c_int32))
        if rc != 0:
            raise ValueError("oracle multiply rejected its arguments")
        return acc

    def unquantize(self, acc: np.ndarray, unquant, bias=None, relu=False) -> np.ndarray:
        acc = np.ascontiguousarray(acc, dtype=np.int32)
        m, n = acc.shape
        out = np.empty((m, n), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
        self.L.mo_unquantize_write(_p(acc, ctypes.c_int32), m, n, ctypes.c_float(float(unquant)),
                                   _p(b, ctypes.c_float), int(relu), _p(out, ctypes.c_float))
        return out

    def affine(self, a: np.ndarray, bt: np.ndarray, qb, bias=None, scale=1.0, relu=False, want_acc=False):
        a2 = np.ascontiguousarray(a, dtype=np.float32).reshape(-1, a.shape[-1])
        bt = np.ascontiguousarray(bt, dtype=np.int8)
        m, k = a2.shape
        n = bt.shape[0]
        out = np.empty((m, n), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
        aq = np.empty((m, k), dtype=np.int8) if want_acc else None
        acc = np.empty((m, n), dtype=np.int32) if want_acc else None
        qa = ctypes.c_float(0)
        rc = self.L.mo_affine(_p(a2, ctypes.c_float), m, k, _p(bt, ctypes.c_int8), ctypes.c_float(float(qb)), n,
                              _p(b, ctypes.c_float), ctypes.c_float(float(scale)), int(relu),
                              _p(out, ctypes.c_float), _p(aq, ctypes.c_int8), _p(acc, ctypes.c_int32),
                              ctypes.byref(qa))
        if rc != 0:
            raise ValueError("oracle affine rejected its arguments")
        out = out.reshape(a.shape[:-1] + (n,))
        if want_acc:
            return out, acc, aq, np.float32(qa.value)
        return out

    # ---- float glue in the fixed operation order (see oracle_i8.c) -------------------------------
    def add_layernorm(self, a, resid, gamma, beta, eps=1e-6):
        a = np.ascontiguousarray(a, dtype=np.float32)
        rows, dim = int(np.prod(a.shape[:-1])), a.shape[-1]
        r = None if resid is None else np.ascontiguousarray(resid, dtype=np.float32)
        g = np.ascontiguousarray(gamma, dtype=np.float32).reshape(-1)
        b = np.ascontiguousarray(beta, dtype=np.float32).reshape(-1)
        out = np.empty_like(a)
        self.L.mo_add_layernorm(_p(a, ctypes.c_float), _p(r, ctypes.c_float), _p(g, ctypes.c_float), _p(b, ctypes.c_float),
                                ctypes.c_float(eps), rows, dim, _p(out, ctypes.c_float))
        return out

    def attention1(self, q, k, v, log_mask, rows, heads, dh, length, batch, mode):
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        m = None if log_mask is None else np.ascontiguousarray(log_mask, dtype=np.float32)
        out = np.empty((rows, heads * dh), dtype=np.float32)
        self.L.mo_attention1(_p(q, ctypes.c_float), _p(k, ctypes.c_float), _p(v, ctypes.c_float), _p(m, ctypes.c_float),
                             rows, heads, dh, length, batch, mode, _p(out, ctypes.c_float))
        return out

    def lse_topk(self, logits, k, prev_scores=None):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        rows, vocab = logits.shape
        ps = None if prev_scores is None else np.ascontiguousarray(prev_scores, dtype=np.float32)
        cs = np.empty((rows, k), dtype=np.float32)
        cw = np.empty((rows, k), dtype=np.int32)
        self.L.mo_lse_topk(_p(logits, ctypes.c_float), rows, vocab, k, _p(ps, ctypes.c_float), _p(cs, ctypes.c_float),
                           _p(cw, ctypes.c_int32))
        return cs, cw

    def embed(self, wemb, words, pos, pos_mod, scale, rows):
        wemb = np.ascontiguousarray(wemb, dtype=np.float32)
        dim = wemb.shape[1]
        w = None if words is None else np.ascontiguousarray(words, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.float32)
        out = np.empty((rows, dim), dtype=np.float32)
        self.L.mo_embed(_p(wemb, ctypes.c_float), _p(w, ctypes.c_int32), _p(pos, ctypes.c_float), pos_mod, ctypes.c_float(scale),
                        rows, dim, _p(out, ctypes.c_float))
        return out

    def ssru_cell(self, cell, xw, f):
        cell = np.ascontiguousarray(cell, dtype=np.float32)
        xw = np.ascontiguousarray(xw, dtype=np.float32)
        f = np.ascontiguousarray(f, dtype=np.float32)
        cn, h = np.empty_like(cell), np.empty_like(cell)
        self.L.mo_ssru_cell(_p(cell, ctypes.c_float), _p(xw, ctypes.c_float), _p(f, ctypes.c_float), cell.size,
                            _p(cn, ctypes.c_float), _p(h, ctypes.c_float))
        return cn, h


# ---------------------------------------------------------------------------------------------
# packed8avx512 (mjdgemm route): restatement in oracle_packed8.c, and the reference's own code
# compiled into _ref/libref_mjdgemm.so by `make ref`.

_REF_MJD = os.path.join(_HERE, "_ref", "libref_mjdgemm.so")


def aligned_empty(shape, dtype, alignment: int = 64) -> np.ndarray:
    """A C-contiguous array whose first byte sits on `alignment` (the reference's AVX-512 route uses
    aligned loads on A, the bias, C and the per-column parameters)."""
    nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
    raw = np.zeros(nbytes + alignment, np.uint8)
    off = (-raw.ctypes.data) % alignment
    return raw[off:off + nbytes].view(dtype).reshape(shape)


def aligned_copy(a: np.ndarray, dtype=None) -> np.ndarray:
    out = aligned_empty(a.shape, dtype or a.dtype)
    out[...] = a
    return out


class Packed8Item:
    """Views into one packed8avx512 item: block-ordered int8 weights, then scaleB, zeroPointB, colOffsetsB."""

    def __init__(self, packed: np.ndarray, K: int, N: int):
        assert packed.dtype == np.int8 and packed.size == K * N + 12 * N
        self.packed, self.K, self.N = packed, K, N
        self.scale_b = packed[K * N:K * N + 4 * N].view(np.float32)
        self.zp_b = packed[K * N + 4 * N:K * N + 8 * N].view(np.int32)
        self.off_b = packed[K * N + 8 * N:].view(np.int32)


class Packed8Oracle:
    """ctypes view of the mo_p8_* functions of liboracle_i8.so."""

    def __init__(self, lib_path: str | None = None):
        if lib_path is None:
            lib_path = _LIB if os.path.exists(_LIB) else build()
        L = ctypes.CDLL(lib_path)
        if not hasattr(L, "mo_p8_gemm_packed"):
            L = ctypes.CDLL(build(force=True))
        vp, ci = ctypes.c_void_p, ctypes.c_int
        L.mo_p8_packed_bytes.restype = ctypes.c_size_t
        L.mo_p8_packed_bytes.argtypes = [ci, ci]
        L.mo_p8_prepare_b.argtypes = [vp, ci, ci, vp]
        L.mo_p8_pack_b.argtypes = [vp, ci, ci, vp]
        L.mo_p8_unpack_bt.argtypes = [vp, ci, ci, vp]
        L.mo_p8_quantize_rows.restype = None
        L.mo_p8_quantize_rows.argtypes = [vp, ci, ci, vp, vp, vp, vp]
        L.mo_p8_affine_bt.argtypes = [vp] * 6 + [ci, vp, vp, ci, ci, ci]
        L.mo_p8_gemm_packed.argtypes = [vp, vp, vp, vp, ci, ci, ci]
        L.mo_p8_set_threads.argtypes = [ci]
        self.L = L

    @staticmethod
    def _v(a):
        return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None

    def set_threads(self, n: int) -> None:
        self.L.mo_p8_set_threads(int(n))

    def prepare_b(self, w: np.ndarray) -> Packed8Item:
        """fp32 W [K,N] -> packed item (fbgemmPacked8Pack restated, min/max range)."""
        w = np.ascontiguousarray(w, np.float32)
        K, N = w.shape
        packed = aligned_empty((self.L.mo_p8_packed_bytes(K, N),), np.int8)
        if self.L.mo_p8_prepare_b(self._v(w), K, N, self._v(packed)):
            raise ValueError("packed8avx512 needs K % 256 == 0 and N % 32 == 0")
        return Packed8Item(packed, K, N)

    def pack_b(self, b: np.ndarray) -> np.ndarray:
        b = np.ascontiguousarray(b, np.int8)
        K, N = b.shape
        out = np.zeros(K * N, np.int8)
        if self.L.mo_p8_pack_b(self._v(b), K, N, self._v(out)):
            raise ValueError("bad shape")
        return out

    def unpack_bt(self, item: Packed8Item) -> np.ndarray:
        bt = np.zeros((item.N, item.K), np.int8)
        if self.L.mo_p8_unpack_bt(self._v(item.packed), item.K, item.N, self._v(bt)):
            raise ValueError("bad shape")
        return bt

    def quantize_rows(self, a: np.ndarray):
        a = np.ascontiguousarray(a, np.float32)
        M, K = a.shape
        aq = np.zeros((M, K), np.uint8)
        sa, za, su = np.zeros(M, np.float32), np.zeros(M, np.int32), np.zeros(M, np.int32)
        self.L.mo_p8_quantize_rows(self._v(a), M, K, self._v(aq), self._v(sa), self._v(za), self._v(su))
        return aq, sa, za, su

    def affine(self, a: np.ndarray, item: Packed8Item, bias=None, relu: bool = False, want_acc: bool = False):
        a = np.ascontiguousarray(a, np.float32)
        M, K = a.shape
        assert K == item.K
        bt = getattr(item, "_bt_cache", None)        # the row-major copy is made once per item
        if bt is None:
            bt = self.unpack_bt(item)
            try:
                item._bt_cache = bt
            except AttributeError:
                pass
        c = np.zeros((M, item.N), np.float32)
        acc = np.zeros((M, item.N), np.int32) if want_acc else None
        b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
        rc = self.L.mo_p8_affine_bt(self._v(a), self._v(bt), self._v(item.scale_b), self._v(item.zp_b), self._v(item.off_b),
                                    self._v(b), int(relu), self._v(c), self._v(acc), M, item.N, K)
        if rc:
            raise ValueError("bad arguments")
        return (c, acc) if want_acc else c


class RefMjdgemm:
    """The reference's own gemmInt8Packed, when `make -C oracle ref` has built it (raises FileNotFoundError otherwise)."""

    SHAPES_NK = [(512, 512), (1024, 1024), (4096, 1024), (3072, 1024), (1024, 4096), (8192, 512), (512, 8192), (1024, 512),
                 (512, 1024), (32000, 512)]

    def __init__(self, lib_path: str = _REF_MJD):
        if not os.path.exists(lib_path):
            raise FileNotFoundError(lib_path)
        self.L = ctypes.CDLL(lib_path)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        self.L.ref_mjd_gemm.argtypes = [vp, vp, vp, vp, ci, ci, ci]
        self.L.ref_mjd_pack_b.argtypes = [vp, vp, ci, ci]

    def isa(self) -> int:
        """marian::cpu::InstructionSet the reference picks on this host (5 and 6 are the AVX-512 route)."""
        return int(self.L.ref_mjd_isa())

    def supported(self, N: int, K: int) -> bool:
        return bool(self.L.ref_mjd_supported(N, K))

    def gemm(self, a: np.ndarray, item: Packed8Item, bias=None) -> np.ndarray:
        a = aligned_copy(np.asarray(a, np.float32))
        M, K = a.shape
        b = aligned_copy(np.asarray(bias, np.float32)) if bias is not None else None
        packed = item.packed if item.packed.ctypes.data % 64 == 0 else aligned_copy(item.packed)
        c = aligned_empty((M, item.N), np.float32)
        v = Packed8Oracle._v
        if self.L.ref_mjd_gemm(v(a), v(packed), v(b), v(c), M, item.N, K):
            raise ValueError("the reference does not instantiate this weight shape")
        return np.array(c)

    def pack_b(self, b: np.ndarray) -> np.ndarray:
        b = np.ascontiguousarray(b, np.int8)
        K, N = b.shape
        out = np.zeros(K * N, np.int8)
        if self.L.ref_mjd_pack_b(Packed8Oracle._v(b), Packed8Oracle._v(out), N, K):
            raise ValueError("the reference does not instantiate this weight shape")
        return out
