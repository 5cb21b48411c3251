"""GGUF: the file a model ships in, read for the device's weight formats.

The host-side counterpart of the engine's reader (inference/gguf.rs:1-246; the
metadata values of model/gguf.rs:95-213), with the one change a device that
multiplies k-quants needs: ``matrix`` hands Q4_K, Q6_K and Q8_0 tensors over
as their raw blocks (the engine re-quantizes Q6_K to Q8_0 at load,
inference/gguf.rs:224-229, and does not know Q4_K's type id 12 at all,
:28-33).

    "GGUF" | version (u32) | tensor count (u64) | key count (u64)
    keys:    name | type (u32) | value
    tensors: name | dimensions (u32, then u64 each, innermost first) | type (u32) | offset (u64)
    padding to the alignment | tensor data

Strings are a u64 length and the bytes.  Nothing here computes a product;
bytes are mapped and moved.  Where a split of a fused projection does not fall
on the format's 256-weight blocks (the 128-wide column groups of the linear
attention's output projection, inference/qwen35/mod.rs:845-847),
``column_groups`` decodes the matrix on the device, regroups its columns and
quantizes it again as Q8_0 on the device, which is what the engine does with
every Q6_K tensor.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from ._lib import BF16, Q4_K, Q6_K, Q8_0
from .tensor import FORMATS, Tensor

F32 = 0            # llama.cpp's numbering (inference/gguf.rs:28-33), and 12 for Q4_K
BLOCK_TYPES = {Q8_0, Q4_K, Q6_K}


def row_bytes(dtype: int, cols: int) -> int:
    """Bytes of a row of ``cols`` weights of a tensor type (inference/gguf.rs:36-53)."""
    if dtype == F32:
        return cols * 4
    if dtype not in FORMATS:
        raise ValueError(f"tensor type {dtype} is not supported")
    _, per, size = FORMATS[dtype]
    if cols % per:
        raise ValueError(f"a row of {cols} is not whole blocks of {per}")
    return cols // per * size


@dataclass
class Info:
    """Where a tensor is and what it holds; ``dims`` innermost first."""
    dims: tuple
    dtype: int
    offset: int

    def shape(self):
        return tuple(reversed(self.dims))

    def size(self) -> int:
        if not self.dims:
            raise ValueError("a tensor has dimensions")
        rows = int(np.prod(self.dims[1:], dtype=np.int64)) if len(self.dims) > 1 else 1
        return rows * row_bytes(self.dtype, self.dims[0])


class _Reader:
    def __init__(self, data, at=0):
        self.data, self.at = data, at

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.at + size > len(self.data):
            raise ValueError("the file ends inside its header")
        (v,) = struct.unpack_from(fmt, self.data, self.at)
        self.at += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.at + n > len(self.data):
            raise ValueError("the file ends inside a string")
        s = bytes(self.data[self.at:self.at + n]).decode("utf-8", "replace")
        self.at += n
        return s

    _SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}

    def value(self, kind: int):
        """model/gguf.rs:186-211."""
        if kind in self._SCALARS:
            return self.take(self._SCALARS[kind])
        if kind == 7:
            return self.take("<B") != 0
        if kind == 8:
            return self.string()
        if kind == 9:
            inner, n = self.take("<I"), self.take("<Q")
            return [self.value(inner) for _ in range(n)]
        raise ValueError(f"unknown metadata type {kind}")


class Gguf:
    """A GGUF file mapped into memory (``Gguf::open``, inference/gguf.rs:120-158)."""

    def __init__(self, path):
        self.path = Path(path)
        self.map = np.memmap(self.path, dtype=np.uint8, mode="r")
        r = _Reader(self.map)
        if bytes(self.map[:4]) != b"GGUF":
            raise ValueError(f"{self.path}: not a GGUF file")
        r.at = 4
        self.version = r.take("<I")
        n_tensors, n_keys = r.take("<Q"), r.take("<Q")
        self.meta = {}
        for _ in range(n_keys):
            key = r.string()
            self.meta[key] = r.value(r.take("<I"))
        self.tensors = {}
        for _ in range(n_tensors):
            name = r.string()
            dims = tuple(r.take("<Q") for _ in range(r.take("<I")))
            dtype, offset = r.take("<I"), r.take("<Q")
            self.tensors[name] = Info(dims, dtype, offset)
        alignment = int(self.meta.get("general.alignment", 32))
        self.data_start = -(-r.at // alignment) * alignment

    def info(self, name: str) -> Info:
        try:
            return self.tensors[name]
        except KeyError:
            raise KeyError(f"missing tensor '{name}'") from None

    def bytes(self, name: str) -> np.ndarray:
        info = self.info(name)
        start, size = self.data_start + info.offset, info.size()
        if start + size > self.map.size:
            raise ValueError(f"tensor '{name}' runs past the end of the file")
        return self.map[start:start + size]

    def f32s(self, name: str) -> np.ndarray:
        if self.info(name).dtype != F32:
            raise ValueError(f"tensor '{name}' is not f32")
        return np.frombuffer(self.bytes(name), dtype="<f4").copy()

    def matrix(self, name: str) -> Tensor:
        """A matrix in the form the device takes it in (``Gguf::matrix``,
        inference/gguf.rs:206-236): bf16 and the block formats as they are, f32
        rounded to bf16 (nearest even, gpu/float.rs:30-36)."""
        info = self.info(name)
        if len(info.dims) != 2:
            raise ValueError(f"tensor '{name}' is not a matrix")
        rows, cols = info.dims[1], info.dims[0]
        if info.dtype in BLOCK_TYPES or info.dtype == BF16:
            return Tensor(info.dtype, (rows, cols), np.array(self.bytes(name)))
        if info.dtype == F32:
            u = self.f32s(name).view(np.uint32)
            nan = (u & 0x7FFFFFFF) > 0x7F800000
            bits = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
            bits[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)      # a NaN stays one
            return Tensor(BF16, (rows, cols), bits)
        raise ValueError(f"tensor '{name}' is of type {info.dtype}, which this device does not take")


def column_groups(dev, tensor: Tensor, width: int, groups) -> Tensor:
    """``Tensor::select_column_groups`` (gpu/mod.rs:103-136) for any group width.
    Groups of whole blocks are byte moves.  Narrower ones (128-wide groups of a
    k-quant matrix) cannot be: the matrix is decoded on the device, its columns
    regrouped, and the result quantized on the device as Q8_0, whose 32-weight
    blocks any such width is whole blocks of."""
    _, per, _ = FORMATS[tensor.fmt]
    if width % per == 0:
        return tensor.select_column_groups(width, groups)
    if width % 32:
        raise ValueError("column groups must at least be whole 32-weight blocks")
    idx = np.asarray(groups, dtype=np.int64)
    full = dev.dequantize(dev.upload(tensor)).reshape(tensor.rows, tensor.cols // width, width)
    regrouped = np.ascontiguousarray(full[:, idx, :]).reshape(tensor.rows, idx.size * width)
    return dev.quantize(Q8_0, regrouped)


def write(path, meta: dict, tensors) -> None:
    """Writes a GGUF file, for tests (the ``write`` of inference/gguf.rs:248-325):
    ``meta`` maps keys to ``(kind, value)``; ``tensors`` is a list of ``(name, dims
    innermost first, type, bytes)``."""
    out = bytearray(b"GGUF")
    out += struct.pack("<IQQ", 3, len(tensors), len(meta))

    def string(s):
        b = s.encode()
        return struct.pack("<Q", len(b)) + b

    def value(kind, v):
        if kind in _Reader._SCALARS:
            return struct.pack(_Reader._SCALARS[kind], v)
        if kind == 7:
            return struct.pack("<B", 1 if v else 0)
        if kind == 8:
            return string(v)
        inner, items = v
        return struct.pack("<IQ", inner, len(items)) + b"".join(value(inner, i) for i in items)

    for key, (kind, v) in meta.items():
        out += string(key) + struct.pack("<I", kind) + value(kind, v)
    offset = 0
    for name, dims, dtype, data in tensors:
        out += string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", dtype, offset)
        offset += -(-len(bytes(data)) // 32) * 32
    out += b"\0" * (-len(out) % 32)
    for _, _, _, data in tensors:
        out += bytes(data)
        out += b"\0" * (-len(out) % 32)
    Path(path).write_bytes(out)
