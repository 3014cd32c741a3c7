"""Python mirror of Marian's operator surface for the int8 path, on CUDA tensors.

Names, argument meaning and error behaviour follow the reference:

* ``affine(a, b, bias, transA, transB, scale)``   src/graph/expression_operators.cpp:647-718
* ``dot(a, b, transA, transB, scale)``            src/graph/expression_operators.cpp:554-619
* ``affineWithReluDropout(x, W, bias, dropProb)`` src/graph/expression_operators.cpp:721-731
* ``prepareA(a)``                                 src/tensors/cpu/intgemm_interface.h:17-32
* ``IntgemmTensor``: an ``intgemm8`` parameter - int8 payload ``Bt[N,K]`` followed by the fp32
  multiplier (src/common/types.cpp:32-37, src/tensors/cpu/integer_common.h:101-111), logical shape
  ``[K,N]`` (src/tensors/cpu/expression_graph_packable.h:242-250).

torch is used for device memory and streams only; all arithmetic runs in libmarian_i8.so.
"""
from __future__ import annotations

import ctypes

import torch

from . import binding
from .binding import MI8_F16, MI8_F32, Mi8Error, check, lib



def launch_count() -> int:
    return int(lib().mi8_launch_count())


def reset_launch_count() -> None:
    lib().mi8_launch_count_reset()


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise Mi8Error(1, f"{what} must live on a CUDA device (there is no CPU fallback)")


class Workspace:
    """Scratch memory for one stream: split-K partial accumulators, arrival counters, abs-max partials.

    Allocated (and zero-filled) once by the caller, as Marian's graph allocator would; the library
    itself never allocates.  Calls sharing a workspace must be ordered on one stream.
    """

    def __init__(self, device="cuda", nbytes: int | None = None):
        n = int(lib().mi8_workspace_bytes(0, 0, 0)) if nbytes is None else int(nbytes)
        self.buf = torch.zeros(n, dtype=torch.uint8, device=device)
        self.nbytes = n

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()


_default_ws: dict[tuple, Workspace] = {}


def default_workspace(device: torch.device) -> Workspace:
    """The workspace ops.* calls use when none is passed: one per (device, current stream), because calls that
    share a workspace must not overlap on the device and two streams give no such ordering."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    ws = _default_ws.get(key)
    if ws is None:
        with torch.cuda.stream(torch.cuda.current_stream(idx)):
            ws = Workspace(device=torch.device("cuda", idx))
        _default_ws[key] = ws
    return ws


class IntgemmTensor:
    """An intgemm8-typed tensor: int8 elements plus the fp32 quantisation multiplier behind them.

    ``storage`` is a uint8 CUDA tensor of ``elements + 4`` bytes (rounded up to 256 like Marian's
    allocator does); ``data`` views the int8 payload as ``[rows, cols]`` and ``quant_mult`` views the
    4 trailing bytes as one float, the slot getQuantMult() addresses in the reference.
    For a weight the payload is ``Bt[N,K]`` while ``shape`` keeps Marian's logical ``[K,N]``.
    """

    def __init__(self, rows: int, cols: int, device, logical_shape=None, storage: torch.Tensor | None = None):
        n = rows * cols
        if n % 4 != 0:
            raise Mi8Error(2, "intgemm8 tensors need a multiple of 4 elements so the multiplier is aligned")
        need = ((n + 4 + 255) // 256) * 256
        if storage is None:
            storage = torch.empty(need, dtype=torch.uint8, device=device)
        elif storage.numel() < n + 4:
            raise Mi8Error(4, "storage too small for an intgemm8 tensor")
        self.storage = storage
        self.rows, self.cols = rows, cols
        self.data = storage[:n].view(torch.int8).view(rows, cols)
        self.quant_mult = storage[n:n + 4].view(torch.float32)
        self.shape = tuple(logical_shape) if logical_shape is not None else (rows, cols)

    @property
    def device(self):
        return self.storage.device


def prepareA(a: torch.Tensor, out: IntgemmTensor | None = None, ws: Workspace | None = None) -> IntgemmTensor:
    """Quantise a float32 activation tensor with one multiplier for the whole tensor."""
    _require_cuda(a, "A")
    if a.dtype != torch.float32:
        raise Mi8Error(1, f"Intgemm expects type of A to be float32 not {a.dtype}")
    a = a.contiguous()
    cols = a.shape[-1]
    rows = a.numel() // cols
    if out is None:
        out = IntgemmTensor(rows, cols, a.device, logical_shape=a.shape)
    ws = ws or default_workspace(a.device)
    check(lib().mi8_prepare_a_f32(a.data_ptr(), rows, cols, out.data.data_ptr(), out.quant_mult.data_ptr(),
                                  ws.ptr, ws.nbytes, _stream_ptr()))
    return out


def max_absolute(a: torch.Tensor, ws: Workspace | None = None) -> torch.Tensor:
    """max|a| as a one-element float32 device tensor (intgemm::MaxAbsolute, integer_common.h:173)."""
    _require_cuda(a, "a")
    if a.dtype != torch.float32:
        raise Mi8Error(1, "max_absolute expects float32")
    a = a.contiguous()
    ws = ws or default_workspace(a.device)
    out = torch.empty(2, dtype=torch.float32, device=a.device)      # [max|a|, 127/max|a|]
    check(lib().mi8_max_absolute_f32(a.data_ptr(), a.numel(), out.data_ptr(), out[1:].data_ptr(), ws.ptr, ws.nbytes, _stream_ptr()))
    return out[:1]


def quantize_with_absmax(a: torch.Tensor, absmax: torch.Tensor, out: IntgemmTensor | None = None) -> IntgemmTensor:
    """Int8::PrepareA with quantMult = 127 / absmax[0] taken from a device tensor (for instance a maximum
    that several ranks agreed on); the multiplier is stored behind the data as usual."""
    _require_cuda(a, "a")
    a = a.contiguous()
    rows = a.numel() // a.shape[-1]
    cols = a.shape[-1]
    q = out if out is not None else IntgemmTensor(rows, cols, a.device)
    check(lib().mi8g_quantize_slot(a.data_ptr(), a.numel(), absmax.data_ptr(), q.data.data_ptr(), q.quant_mult.data_ptr(), _stream_ptr()))
    return q


def prepareB(w: torch.Tensor, w_is_nk: bool = False, ws: Workspace | None = None) -> IntgemmTensor:
    """marian-conv's intgemm8 conversion of one weight: W[K,N] fp32 -> Bt[N,K] int8 + multiplier."""
    _require_cuda(w, "W")
    if w.dtype != torch.float32 or w.dim() != 2:
        raise Mi8Error(1, "weights must be 2-D float32")
    w = w.contiguous()
    if w_is_nk:
        n, k = w.shape
    else:
        k, n = w.shape
    out = IntgemmTensor(n, k, w.device, logical_shape=(k, n))
    ws = ws or default_workspace(w.device)
    check(lib().mi8_prepare_b_f32(w.data_ptr(), k, n, int(w_is_nk), out.data.data_ptr(), out.quant_mult.data_ptr(),
                                  ws.ptr, ws.nbytes, _stream_ptr()))
    return out


def multiply(aq: IntgemmTensor, b: IntgemmTensor, bias: torch.Tensor | None = None, scale: float = 1.0,
             relu: bool = False, out: torch.Tensor | None = None, out_dtype=torch.float32,
             acc_out: torch.Tensor | None = None, ws: Workspace | None = None, tile_m: int = 0, splits: int = 0,
             out_shape=None) -> torch.Tensor:
    """The multiply node of affineOrDotTyped with the fused write-back (and optional ReLU)."""
    m, k = aq.rows, aq.cols
    n = b.rows
    if b.cols != k:
        raise Mi8Error(1, f"inner dimensions differ: A has {k} columns, B has {b.cols} rows")
    if bias is not None:
        _require_cuda(bias, "bias")
        if bias.dtype != torch.float32 or bias.numel() != n:
            raise Mi8Error(1, "bias must be float32 with one value per output column")
        bias = bias.contiguous()
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=aq.device)
    elif out.dtype != out_dtype or out.numel() != m * n or not out.is_contiguous():
        raise Mi8Error(1, "output tensor has the wrong type, size or layout")
    if acc_out is not None and (acc_out.dtype != torch.int32 or acc_out.numel() != m * n):
        raise Mi8Error(1, "acc_out must be int32 [M,N]")
    ws = ws or default_workspace(aq.device)
    dt = MI8_F32 if out_dtype == torch.float32 else MI8_F16
    if out_dtype not in (torch.float32, torch.float16):
        raise Mi8Error(1, "output type must be float32 or float16")
    check(lib().mi8_multiply_i8_ex(aq.data.data_ptr(), b.data.data_ptr(), m, n, k, aq.quant_mult.data_ptr(),
                                   b.quant_mult.data_ptr(), float(scale),
                                   bias.data_ptr() if bias is not None else None, int(relu), out.data_ptr(), dt,
                                   acc_out.data_ptr() if acc_out is not None else None, ws.ptr, ws.nbytes,
                                   _stream_ptr(), tile_m, splits))
    if out_shape is not None:
        out = out.view(out_shape)
    return out


def measure_int8_peak(k_blocks: int = 8192) -> float:
    """TOPS of a loop of the library's int8 MMAs alone on every SM (mi8_measure_int8_peak)."""
    out = ctypes.c_float(0.0)
    check(lib().mi8_measure_int8_peak(int(k_blocks), ctypes.byref(out), _stream_ptr()))
    return float(out.value)


def multiply_from_slot(a: torch.Tensor, absmax_slot: torch.Tensor, b: IntgemmTensor, bias: torch.Tensor | None = None,
                       scale: float = 1.0, relu: bool = False, out_dtype=torch.float32, acc_out: torch.Tensor | None = None,
                       qa_out: torch.Tensor | None = None) -> torch.Tensor | None:
    """mi8_multiply_f32_slot: the affine with PrepareA inside the GEMM kernel.  `a` fp32 [M,K], `absmax_slot` a
    4-byte device tensor holding the bit pattern of max|a|.  Returns None when the shape does not qualify."""
    _require_cuda(a, "a")
    if a.dtype != torch.float32 or a.dim() != 2 or not a.is_contiguous():
        raise Mi8Error(1, "a must be a contiguous float32 matrix")
    m, k = a.shape
    n = b.rows
    if b.cols != k:
        raise Mi8Error(1, f"inner dimensions differ: A has {k} columns, B has {b.cols} rows")
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    rc = lib().mi8_multiply_f32_slot(a.data_ptr(), absmax_slot.data_ptr(), qa_out.data_ptr() if qa_out is not None else None,
                                     b.data.data_ptr(), m, n, k, b.quant_mult.data_ptr(), float(scale),
                                     bias.data_ptr() if bias is not None else None, int(relu), out.data_ptr(),
                                     MI8_F32 if out_dtype == torch.float32 else MI8_F16,
                                     acc_out.data_ptr() if acc_out is not None else None, _stream_ptr())
    if rc == 3:      # MI8_ERR_UNSUPPORTED: not a one-tile-per-CTA shape
        return None
    check(rc)
    return out


def multiply_rows_from(aq: IntgemmTensor, b: IntgemmTensor, bias: torch.Tensor | None, out: torch.Tensor, same_a: torch.Tensor,
                       same_b: torch.Tensor, rows_unchanged_below: int, relu: bool = False, scale: float = 1.0,
                       ws: Workspace | None = None, tile_m: int = 0) -> torch.Tensor:
    """mi8_multiply_i8_rows_from: when the device words same_a[0] and same_b[0] (int32/uint32 tensors) are equal, whole
    tiles of activation rows below `rows_unchanged_below` keep what `out` already holds."""
    m, k, n = aq.rows, aq.cols, b.rows
    if b.cols != k or out.dtype != torch.float32 or out.numel() != m * n or not out.is_contiguous():
        raise Mi8Error(1, "operand shapes / output layout do not match")
    ws = ws or default_workspace(aq.device)
    check(lib().mi8_multiply_i8_rows_from(aq.data.data_ptr(), b.data.data_ptr(), m, n, k, aq.quant_mult.data_ptr(),
                                          b.quant_mult.data_ptr(), float(scale), bias.data_ptr() if bias is not None else None,
                                          int(relu), out.data_ptr(), MI8_F32, ws.ptr, ws.nbytes, _stream_ptr(),
                                          same_a.data_ptr(), same_b.data_ptr(), int(rows_unchanged_below), tile_m))
    return out


def transpose(a: torch.Tensor) -> torch.Tensor:
    """The last two axes of a float32 tensor swapped by the library's transpose kernel (the node the reference puts in front
    of prepareA for transA, src/tensors/cpu/intgemm_interface.h:52)."""
    _require_cuda(a, "a")
    if a.dtype != torch.float32 or a.dim() < 2:
        raise Mi8Error(1, "transpose expects a float32 tensor with at least two axes")
    a = a.contiguous()
    r, c = a.shape[-2], a.shape[-1]
    out = torch.empty(a.shape[:-2] + (c, r), dtype=torch.float32, device=a.device)
    check(lib().mi8_transpose_f32(a.data_ptr(), a.numel() // (r * c), r, c, out.data_ptr(), _stream_ptr()))
    return out


def _affine_or_dot(a: torch.Tensor, b: IntgemmTensor, bias, transA: bool, transB: bool, scale: float, relu: bool,
                   out_dtype=torch.float32, ws: Workspace | None = None, aq: IntgemmTensor | None = None) -> torch.Tensor:
    if not isinstance(b, IntgemmTensor):
        raise Mi8Error(1, f"Intgemm expects type of B to be a variant of intgemm not {type(b).__name__}")
    if aq is None:
        if transA:
            a = transpose(a)
        aq = prepareA(a, ws=ws)
        lead = tuple(a.shape[:-1])
    else:
        lead = tuple(aq.shape[:-1])
    # The reference ignores transB on this path (intgemm_interface.h:47): B is stored as Bt[N,K]
    # either way.  A [N,K]-shaped weight used with transB (tied embeddings) carries logical shape
    # [K,N] after prepareB(w_is_nk=True), so the output width is b.shape[-1] in both cases.
    del transB
    return multiply(aq, b, bias, scale, relu, out_dtype=out_dtype, ws=ws, out_shape=lead + (b.shape[-1],))


def affine(a, b, bias, transA: bool = False, transB: bool = False, scale: float = 1.0, **kw) -> torch.Tensor:
    return _affine_or_dot(a, b, bias, transA, transB, scale, False, **kw)


def dot(a, b, transA: bool = False, transB: bool = False, scale: float = 1.0, **kw) -> torch.Tensor:
    return _affine_or_dot(a, b, None, transA, transB, scale, False, **kw)


def affineWithReluDropout(x, W, bias, dropProb: float = 0.0, **kw) -> torch.Tensor:
    """Inference only: dropout is the identity; the ReLU is fused into the GEMM's write-back."""
    if dropProb != 0.0:
        raise Mi8Error(3, "dropout is a training feature; the int8 path is inference-only")
    return _affine_or_dot(x, W, bias, False, False, 1.0, True, **kw)


def poll_status() -> int:
    """Device status word (0 = healthy); synchronises the device."""
    import ctypes
    v = ctypes.c_int(0)
    lib().mi8_poll_status(ctypes.byref(v))
    return int(v.value)


def clear_status() -> None:
    check(lib().mi8_clear_status(_stream_ptr()))
