"""Marian's binary model container and the intgemm8 model conversion.

Container (src/common/binary.cpp:20-25,35-116,158-254): ``uint64 version = 1``, ``uint64 nItems``,
``Header{nameLength, type, shapeLength, dataLength}[nItems]`` (uint64 each), the NUL-terminated names,
the shapes (int32), ``uint64 offset`` + padding so that the payload starts on a 256-byte boundary, then
the payloads, each a multiple of 256 bytes.  ``special:model.yml`` carries the YAML model description as
an int8 item (src/common/io.cpp:230-252).

Conversion (marian-conv --gemm-type intgemm8, src/tensors/cpu/expression_graph_packable.h:153-253):
every float32 parameter named ``*_W?`` / ``*_W`` becomes an ``intgemm8`` item whose payload is the
transposed, quantised matrix ``Bt[N,K]`` followed by the fp32 multiplier, while ``item.shape`` stays the
logical ``[K,N]``.  The quantisation itself runs on the GPU (``ops.prepareB``).
"""
from __future__ import annotations

import struct

import numpy as np

BINARY_FILE_VERSION = 1

# Type tags (src/common/types.h:270-328): class bits + element size
TYPE_INT8 = 0x0100 + 1
TYPE_FLOAT32 = 0x0400 + 4
TYPE_INTGEMM8 = 0x10000 + 1
TYPE_INTGEMM16 = 0x10000 + 2
TYPE_PACKED8AVX512 = 0x0800 + 1 + 0x2000               # Type::packed8avx512 (src/common/types.h:315)
_HW_BITS = 0x1000 | 0x2000 | 0x4000 | 0x8000          # avx2 / avx512 / sse2 / ssse3 layouts
TYPE_NAMES = {TYPE_INT8: "int8", TYPE_FLOAT32: "float32", TYPE_INTGEMM8: "intgemm8", TYPE_INTGEMM16: "intgemm16",
              TYPE_PACKED8AVX512: "packed8avx512"}


class Item:
    """io::Item (src/common/io_item.h:11-31): name, shape, type tag, raw bytes (a multiple of 256)."""

    def __init__(self, name: str, shape, type_tag: int, data: bytes):
        self.name, self.shape, self.type, self.bytes = name, [int(s) for s in shape], int(type_tag), bytes(data)

    def elements(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def _pad256(b: bytes) -> bytes:
    return b + b"\0" * ((-len(b)) % 256)


def meta_item(yaml_text: str, name: str = "special:model.yml") -> Item:
    """addMetaToItems: the text plus NUL, padded with NULs to a 256-byte block, shape = [padded size]."""
    raw = _pad256(yaml_text.encode() + b"\0")
    return Item(name, [len(raw)], TYPE_INT8, raw)


def float_item(name: str, arr: np.ndarray) -> Item:
    a = np.ascontiguousarray(arr, dtype=np.float32)
    return Item(name, a.shape, TYPE_FLOAT32, _pad256(a.tobytes()))


def intgemm8_item(name: str, bt: np.ndarray, quant_mult: float, logical_shape) -> Item:
    """Payload = int8 Bt[N,K] then the fp32 multiplier (requiredBytes: elements + 4), padded to 256."""
    raw = np.ascontiguousarray(bt, dtype=np.int8).tobytes() + struct.pack("<f", float(quant_mult))
    return Item(name, logical_shape, TYPE_INTGEMM8, _pad256(raw))


def packed8_item(name: str, packed: np.ndarray, logical_shape) -> Item:
    """A packed8avx512 item: block-ordered int8 weights + scaleB + zeroPointB + colOffsetsB, logical shape [K,N]
    (src/tensors/cpu/expression_graph_packable.h:82-92; the payload is padded to the allocation's 256-byte multiple)."""
    return Item(name, logical_shape, TYPE_PACKED8AVX512, _pad256(np.ascontiguousarray(packed).view(np.uint8).tobytes()))


def save_items(path: str, items) -> None:
    """io::binary::saveItems."""
    head = struct.pack("<Q", BINARY_FILE_VERSION)
    body = struct.pack("<Q", len(items))
    for it in items:
        if len(it.bytes) % 256 != 0:
            raise ValueError(f"Binary item size ({len(it.bytes)}) is not 256-byte aligned for tensor {it.name}")
        body += struct.pack("<QQQQ", len(it.name) + 1, it.type, len(it.shape), len(it.bytes))
    for it in items:
        body += it.name.encode() + b"\0"
    for it in items:
        body += struct.pack(f"<{len(it.shape)}i", *it.shape)
    pos = len(head) + len(body)
    nextpos = ((pos + 8) // 256 + 1) * 256
    offset = nextpos - pos - 8
    with open(path, "wb") as f:
        f.write(head + body + struct.pack("<Q", offset) + b"\0" * offset)
        for it in items:
            f.write(it.bytes)


def load_items(path_or_bytes) -> list:
    """io::binary::loadItems (no hardware-specific re-tiling: the GPU engine consumes the generic layout)."""
    buf = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, buf, pos)
        pos += struct.calcsize(fmt)
        return v

    (version,) = take("<Q")
    if version != BINARY_FILE_VERSION:
        raise ValueError(f"Unknown binary file version {version}")
    (n,) = take("<Q")
    headers = [take("<QQQQ") for _ in range(n)]
    names = []
    for h in headers:
        names.append(buf[pos:pos + h[0] - 1].decode())
        pos += h[0]
    shapes = [list(take(f"<{h[2]}i")) for h in headers]
    (offset,) = take("<Q")
    pos += offset
    items = []
    for h, name, shape in zip(headers, names, shapes):
        items.append(Item(name, shape, h[1], buf[pos:pos + h[3]]))
        pos += h[3]
    return items


def is_intgemm_param(name: str) -> bool:
    p = name.find("_W")
    return p != -1 and p in (len(name) - 3, len(name) - 2)


def convert(params: dict, yaml_text: str, gemm_type: str = "intgemm8", device="cuda"):
    """marian-conv: float32 parameters -> items; ``intgemm8`` quantises the ``*_W*`` matrices on the GPU."""
    import torch

    from . import ops
    if gemm_type not in ("float32", "intgemm8", "packed8avx512"):
        raise ValueError(f"gemm-type {gemm_type} is not supported by this engine (float32, intgemm8 or packed8avx512)")
    items = []
    for name, val in params.items():
        val = np.asarray(val, dtype=np.float32)
        if gemm_type == "intgemm8" and val.ndim == 2 and is_intgemm_param(name):
            t = ops.prepareB(torch.from_numpy(np.ascontiguousarray(val)).to(device))
            torch.cuda.synchronize()
            items.append(intgemm8_item(name, t.data.cpu().numpy(), float(t.quant_mult.item()), val.shape))
        elif gemm_type == "packed8avx512" and val.ndim == 2 and is_intgemm_param(name):
            # the same parameter selection as the intgemm branch (expression_graph_packable.h:52-53); the blocks have no padding
            from . import packed8
            if val.shape[0] % 256 or val.shape[1] % 32:
                raise ValueError(f"{name}: packed8avx512 needs K % 256 == 0 and N % 32 == 0, got {val.shape}")
            t = packed8.prepareB(torch.from_numpy(np.ascontiguousarray(val)).to(device))
            torch.cuda.synchronize()
            items.append(packed8_item(name, t.item.cpu().numpy(), val.shape))
        else:
            items.append(float_item(name, val))
    items.append(meta_item(yaml_text))
    return items


def items_to_params(items, device="cuda"):
    """Items -> (yaml text, {name: float32 ndarray | ops.IntgemmTensor | packed8.Packed8Weight on the device})."""
    import torch

    from . import ops
    params, yaml_text = {}, ""
    for it in items:
        if it.name == "special:model.yml":
            yaml_text = it.bytes.split(b"\0", 1)[0].decode()
        elif it.type == TYPE_FLOAT32:
            params[it.name] = np.frombuffer(it.bytes, dtype=np.float32, count=it.elements()).reshape(it.shape).copy()
        elif it.type == TYPE_INTGEMM8:
            k, n = it.shape[-2], it.shape[-1]
            t = ops.IntgemmTensor(n, k, device, logical_shape=(k, n))
            need = n * k + 4
            t.storage[:need].copy_(torch.frombuffer(bytearray(it.bytes[:need]), dtype=torch.uint8))
            params[it.name] = t
        elif it.type == TYPE_PACKED8AVX512:
            from . import packed8
            k, n = it.shape[-2], it.shape[-1]
            need = k * n + 12 * n
            params[it.name] = packed8.Packed8Weight(np.frombuffer(it.bytes, dtype=np.int8, count=need), k, n, device=device)
        elif (it.type & 0x10000) and (it.type & _HW_BITS):
            raise ValueError(f"{it.name}: hardware-specific intgemm layout (type {it.type:#x}) cannot be used on the GPU; "
                             "convert the model with --gemm-type intgemm8")
        else:
            raise ValueError(f"{it.name}: unsupported item type {it.type:#x}")
    return yaml_text, params


def main(argv=None):
    """python -m marian_dev_b200.binary_io --from model.npz --to model.bin --gemm-type intgemm8
    (the flags of marian-conv, src/command/marian_conv.cpp:14-151)."""
    import argparse
    ap = argparse.ArgumentParser(description="Convert a Marian .npz model to the binary format, optionally quantising to intgemm8 on the GPU")
    ap.add_argument("--from", dest="src", required=True)
    ap.add_argument("--to", dest="dst", required=True)
    ap.add_argument("--gemm-type", "-g", default="float32")
    a = ap.parse_args(argv)
    npz = np.load(a.src)
    yaml_text = ""
    params = {}
    for name in npz.files:
        if name == "special:model.yml":
            yaml_text = bytes(npz[name].astype(np.uint8)).split(b"\0", 1)[0].decode()
        else:
            params[name] = npz[name]
    save_items(a.dst, convert(params, yaml_text, a.gemm_type))


if __name__ == "__main__":
    main()
