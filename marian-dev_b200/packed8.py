"""Host side of the packed-int8 (packed8avx512) affine: the call shape of the reference's
marian::cpu::mjdgemm::gemmInt8Packed(A, B, bias, C, M, N, K) (src/tensors/cpu/mjdgemm/mjdgemm.h:38, reached from
fbgemmPacked8Gemm, src/tensors/cpu/fbgemm/packed_gemm.cpp:566-592) over the C ABI of include/marian_packed8.h.
There is no CPU fallback: everything runs in libmarian_i8.so on the GPU."""
from __future__ import annotations

import numpy as np
import torch

from .binding import check, lib
from .ops import Workspace, _require_cuda, _stream_ptr, default_workspace


class Packed8Weight:
    """A packed8avx512 item on the device: the block-ordered bytes as stored in the model file, and the Bt[N,K]
    row-major copy the GEMM reads (made once, here).  scale_b / zp_b / off_b are views into the item's tail."""

    def __init__(self, packed, K: int, N: int, device="cuda"):
        L = lib()
        nbytes = int(L.mi8p_packed_bytes(K, N))
        host = torch.from_numpy(np.array(packed, copy=True).view(np.int8)) if not isinstance(packed, torch.Tensor) else packed
        if host.numel() != nbytes or host.dtype != torch.int8:
            raise ValueError(f"a packed8avx512 item of a [{K},{N}] weight has {nbytes} bytes")
        self.K, self.N = K, N
        self.item = host.to(device).contiguous()
        self.bt = torch.empty((N, K), dtype=torch.int8, device=device)
        check(L.mi8p_unpack_b(self.item.data_ptr(), K, N, self.bt.data_ptr(), _stream_ptr()))
        tail = self.item[K * N:]
        self.scale_b = tail[:4 * N].view(torch.float32)
        self.zp_b = tail[4 * N:8 * N].view(torch.int32)
        self.off_b = tail[8 * N:].view(torch.int32)


def prepareB(w: torch.Tensor) -> Packed8Weight:
    """marian-conv --gemm-type packed8avx512 for one weight: fp32 [K,N] on the device -> Packed8Weight (item + Bt)."""
    _require_cuda(w, "W")
    w = w.contiguous().float()
    K, N = w.shape
    L = lib()
    item = torch.empty(int(L.mi8p_packed_bytes(K, N)), dtype=torch.int8, device=w.device)
    check(L.mi8p_prepare_b_f32(w.data_ptr(), K, N, item.data_ptr(), _stream_ptr()))
    return Packed8Weight(item, K, N, device=w.device)


def quantize_rows(a: torch.Tensor):
    """computeQuantizationParams + quantize per row (mjdgemm_avx512.cpp:195-276): (aq uint8, scaleA, zeroPointA, sumA)."""
    _require_cuda(a, "A")
    a2 = a.reshape(-1, a.shape[-1]).contiguous()
    M, K = a2.shape
    aq = torch.empty((M, K), dtype=torch.uint8, device=a.device)
    scale_a = torch.empty(M, dtype=torch.float32, device=a.device)
    zp_a = torch.empty(M, dtype=torch.int32, device=a.device)
    sum_a = torch.empty(M, dtype=torch.int32, device=a.device)
    check(lib().mi8p_quantize_rows(a2.data_ptr(), M, K, aq.data_ptr(), scale_a.data_ptr(), zp_a.data_ptr(), sum_a.data_ptr(),
                                   _stream_ptr()))
    return aq, scale_a, zp_a, sum_a


def multiply(aq, scale_a, zp_a, sum_a, w: Packed8Weight, bias=None, relu: bool = False, want_acc: bool = False,
             ws: Workspace | None = None, tile_m: int = 0, splits: int = 0):
    M, K = aq.shape
    if K != w.K:
        raise ValueError("inner dimensions differ")
    ws = ws or default_workspace(aq.device)
    c = torch.empty((M, w.N), dtype=torch.float32, device=aq.device)
    acc = torch.empty((M, w.N), dtype=torch.int32, device=aq.device) if want_acc else None
    check(lib().mi8p_multiply(aq.data_ptr(), scale_a.data_ptr(), zp_a.data_ptr(), sum_a.data_ptr(), w.bt.data_ptr(),
                              w.scale_b.data_ptr(), w.zp_b.data_ptr(), w.off_b.data_ptr(), M, w.N, K,
                              bias.data_ptr() if bias is not None else None, int(relu), c.data_ptr(),
                              acc.data_ptr() if acc is not None else None, ws.ptr, ws.nbytes, _stream_ptr(), tile_m, splits))
    return (c, acc) if want_acc else c


def gemmInt8Packed(a: torch.Tensor, w: Packed8Weight, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
                   scratch: torch.Tensor | None = None, ws: Workspace | None = None) -> torch.Tensor:
    """C[M,N] = A[M,K] . B + bias with the arithmetic of the reference's gemmInt8Packed, in one ABI call."""
    _require_cuda(a, "A")
    a2 = a.reshape(-1, a.shape[-1]).contiguous()
    M, K = a2.shape
    L = lib()
    need = int(L.mi8p_scratch_bytes(M, K))
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=a.device)
    ws = ws or default_workspace(a.device)
    c = out if out is not None else torch.empty((M, w.N), dtype=torch.float32, device=a.device)
    check(L.mi8p_gemm_int8_packed(a2.data_ptr(), w.bt.data_ptr(), w.scale_b.data_ptr(), w.zp_b.data_ptr(), w.off_b.data_ptr(),
                                  bias.data_ptr() if bias is not None else None, c.data_ptr(), M, w.N, K, scratch.data_ptr(),
                                  scratch.numel(), ws.ptr, ws.nbytes, _stream_ptr()))
    return c.reshape(tuple(a.shape[:-1]) + (w.N,))
