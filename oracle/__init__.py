"""ctypes front end of the CPU oracle (``oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared with.  Only
the tests, the smoke check and the benchmark's CPU-baseline legs import this
package; the shipped library never does.

Every function works on numpy arrays and returns numpy arrays.  Weight
matrices are bytes in GGUF block order, row-major, ``row_bytes(fmt, cols)``
per row.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "liboracle.so"

# GGUF type ids
Q8_0, Q4_K, Q6_K = 8, 12, 14
FORMATS = {"q8_0": Q8_0, "q4_k": Q4_K, "q6_k": Q6_K}


def build(force: bool = False) -> Path:
    """Compiles ``oracle.c`` with the recipe in ``oracle/Makefile``."""
    src = _DIR / "oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "liboracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            build()
        _lib = C.CDLL(str(_SO))
        _declare(_lib)
    return _lib


_u8p, _i8p = C.POINTER(C.c_uint8), C.POINTER(C.c_int8)
_u16p, _f32p = C.POINTER(C.c_uint16), C.POINTER(C.c_float)


def _declare(L):
    sz = C.c_size_t
    L.orc_bf16.restype = C.c_float
    L.orc_bf16.argtypes = [C.c_uint16]
    L.orc_to_bf16.restype = C.c_uint16
    L.orc_to_bf16.argtypes = [C.c_float]
    L.orc_from_f16.restype = C.c_float
    L.orc_from_f16.argtypes = [C.c_uint16]
    L.orc_to_f16.restype = C.c_uint16
    L.orc_to_f16.argtypes = [C.c_float]
    for name, a, b in [("orc_to_f16_array", _f32p, _u16p), ("orc_from_f16_array", _u16p, _f32p),
                       ("orc_to_bf16_array", _f32p, _u16p), ("orc_bf16_array", _u16p, _f32p)]:
        getattr(L, name).restype = None
        getattr(L, name).argtypes = [a, sz, b]
    L.orc_lcg_floats.restype = None
    L.orc_lcg_floats.argtypes = [C.POINTER(C.c_uint64), sz, _f32p]
    L.orc_quantize_block.restype = C.c_uint16
    L.orc_quantize_block.argtypes = [_f32p, _i8p]
    L.orc_quantize_q8_0_row_split.argtypes = [_f32p, sz, _u16p, _i8p]
    L.orc_dequantize_q8_0_row_split.argtypes = [_u16p, _i8p, sz, _f32p]
    L.orc_dot_q8_0_split.restype = C.c_float
    L.orc_dot_q8_0_split.argtypes = [_u16p, _i8p, _f32p, sz]
    L.orc_quantize_q4_0_row_split.argtypes = [_f32p, sz, _u16p, _u8p]
    L.orc_dequantize_q4_0_row_split.argtypes = [_u16p, _u8p, sz, _f32p]
    L.orc_dot_q4_0_split.restype = C.c_float
    L.orc_dot_q4_0_split.argtypes = [_u16p, _u8p, _f32p, sz]
    for name in ("orc_dequantize_q8_0", "orc_dequantize_q4_1", "orc_dequantize_q6_k", "orc_dequantize_q4_k"):
        getattr(L, name).restype = None
        getattr(L, name).argtypes = [_u8p, sz, _f32p]
    for name in ("orc_quantize_q8_0", "orc_quantize_q6_k", "orc_quantize_q4_k"):
        getattr(L, name).restype = None
        getattr(L, name).argtypes = [_f32p, sz, _u8p]
    for name in ("orc_dot_q8_0", "orc_dot_q6_k", "orc_dot_q4_k"):
        getattr(L, name).restype = C.c_float
        getattr(L, name).argtypes = [_u8p, _f32p, sz]
    L.orc_q8_0_split_to_file.argtypes = [_u16p, _i8p, sz, _u8p]
    L.orc_q8_0_file_to_split.argtypes = [_u8p, sz, _u16p, _i8p]
    L.orc_q4k_unpack_scales.argtypes = [_u8p, _u8p, _u8p]
    L.orc_q4k_pack_scales.argtypes = [_u8p, _u8p, _u8p]
    L.orc_row_bytes.restype = sz
    L.orc_row_bytes.argtypes = [C.c_int, sz]
    L.orc_matmul.argtypes = [C.c_int, _u8p, sz, sz, _f32p, sz, _f32p]
    L.orc_matmul_add.argtypes = [C.c_int, _u8p, sz, sz, _f32p, sz, _f32p]
    L.orc_swiglu.argtypes = [C.c_int, _u8p, _u8p, sz, sz, _f32p, sz, _f32p]
    L.orc_dequantize.argtypes = [C.c_int, _u8p, sz, sz, _f32p]
    L.orc_quantize.argtypes = [C.c_int, _f32p, sz, sz, _u8p]
    L.orc_threads.restype = C.c_int
    L.orc_set_threads.argtypes = [C.c_int]


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1) if a.dtype != np.uint8 else a.reshape(-1)


def _fmt(fmt) -> int:
    return FORMATS[fmt] if isinstance(fmt, str) else int(fmt)


# ---- scalars / arrays -------------------------------------------------
def to_f16(x) -> np.ndarray:
    x = _f32(x).reshape(-1)
    out = np.empty(x.size, np.uint16)
    lib().orc_to_f16_array(_p(x, _f32p), x.size, _p(out, _u16p))
    return out


def from_f16(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16).reshape(-1)
    out = np.empty(h.size, np.float32)
    lib().orc_from_f16_array(_p(h, _u16p), h.size, _p(out, _f32p))
    return out


def to_bf16(x) -> np.ndarray:
    x = _f32(x).reshape(-1)
    out = np.empty(x.size, np.uint16)
    lib().orc_to_bf16_array(_p(x, _f32p), x.size, _p(out, _u16p))
    return out


def bf16(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16).reshape(-1)
    out = np.empty(h.size, np.float32)
    lib().orc_bf16_array(_p(h, _u16p), h.size, _p(out, _f32p))
    return out


class Lcg:
    """The reference tests' generator (gpu/tests.rs:45-54): floats in [-1, 1)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def floats(self, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib().orc_lcg_floats(C.byref(self.state), n, _p(out, _f32p))
        return out


# ---- 32-blocks, split layout (gpu/quant.rs) ---------------------------
def quantize_block(block):
    block = _f32(block)
    assert block.size == 32
    q = np.empty(32, np.int8)
    bits = lib().orc_quantize_block(_p(block, _f32p), _p(q, _i8p))
    return int(bits), q


def quantize_q8_0_row_split(x):
    x = _f32(x).reshape(-1)
    scales, quants = np.empty(x.size // 32, np.uint16), np.empty(x.size, np.int8)
    lib().orc_quantize_q8_0_row_split(_p(x, _f32p), x.size, _p(scales, _u16p), _p(quants, _i8p))
    return scales, quants


def dequantize_q8_0_row_split(scales, quants):
    out = np.empty(quants.size, np.float32)
    lib().orc_dequantize_q8_0_row_split(_p(scales, _u16p), _p(quants, _i8p), quants.size, _p(out, _f32p))
    return out


def dot_q8_0_split(scales, quants, x) -> float:
    x = _f32(x)
    return float(lib().orc_dot_q8_0_split(_p(scales, _u16p), _p(quants, _i8p), _p(x, _f32p), x.size))


def quantize_q4_0_row_split(x):
    x = _f32(x).reshape(-1)
    scales, quants = np.empty(x.size // 32, np.uint16), np.empty(x.size // 2, np.uint8)
    lib().orc_quantize_q4_0_row_split(_p(x, _f32p), x.size, _p(scales, _u16p), _p(quants, _u8p))
    return scales, quants


def dequantize_q4_0_row_split(scales, quants):
    out = np.empty(quants.size * 2, np.float32)
    lib().orc_dequantize_q4_0_row_split(_p(scales, _u16p), _p(quants, _u8p), out.size, _p(out, _f32p))
    return out


def dot_q4_0_split(scales, quants, x) -> float:
    x = _f32(x)
    return float(lib().orc_dot_q4_0_split(_p(scales, _u16p), _p(quants, _u8p), _p(x, _f32p), x.size))


def q8_0_split_to_file(scales, quants) -> np.ndarray:
    out = np.empty(scales.size * 34, np.uint8)
    lib().orc_q8_0_split_to_file(_p(scales, _u16p), _p(quants, _i8p), scales.size, _p(out, _u8p))
    return out


def q8_0_file_to_split(data):
    data = _u8(data)
    n = data.size // 34
    scales, quants = np.empty(n, np.uint16), np.empty(n * 32, np.int8)
    lib().orc_q8_0_file_to_split(_p(data, _u8p), n, _p(scales, _u16p), _p(quants, _i8p))
    return scales, quants


def dequantize_q4_1(row, cols: int) -> np.ndarray:
    row = _u8(row)
    out = np.empty(cols, np.float32)
    lib().orc_dequantize_q4_1(_p(row, _u8p), cols, _p(out, _f32p))
    return out


def q4k_unpack_scales(b12):
    b12 = _u8(b12)
    sc, m = np.empty(8, np.uint8), np.empty(8, np.uint8)
    lib().orc_q4k_unpack_scales(_p(b12, _u8p), _p(sc, _u8p), _p(m, _u8p))
    return sc, m


def q4k_pack_scales(sc, m) -> np.ndarray:
    sc, m = np.ascontiguousarray(sc, np.uint8), np.ascontiguousarray(m, np.uint8)
    out = np.empty(12, np.uint8)
    lib().orc_q4k_pack_scales(_p(sc, _u8p), _p(m, _u8p), _p(out, _u8p))
    return out


# ---- whole matrices in GGUF layout ------------------------------------
def row_bytes(fmt, cols: int) -> int:
    n = int(lib().orc_row_bytes(_fmt(fmt), cols))
    if n == 0:
        raise ValueError(f"unknown format {fmt}")
    return n


def quantize(fmt, w) -> np.ndarray:
    """f32 [rows, cols] -> GGUF blocks, uint8 [rows * row_bytes]."""
    w = _f32(w)
    rows, cols = w.shape
    out = np.empty(rows * row_bytes(fmt, cols), np.uint8)
    rc = lib().orc_quantize(_fmt(fmt), _p(w, _f32p), rows, cols, _p(out, _u8p))
    assert rc == 0
    return out


def dequantize(fmt, blocks, rows: int, cols: int) -> np.ndarray:
    blocks = _u8(blocks)
    assert blocks.size == rows * row_bytes(fmt, cols)
    out = np.empty((rows, cols), np.float32)
    rc = lib().orc_dequantize(_fmt(fmt), _p(blocks, _u8p), rows, cols, _p(out, _f32p))
    assert rc == 0
    return out


def dot(fmt, row, x) -> float:
    row, x = _u8(row), _f32(x)
    fn = {Q8_0: lib().orc_dot_q8_0, Q4_K: lib().orc_dot_q4_k, Q6_K: lib().orc_dot_q6_k}[_fmt(fmt)]
    return float(fn(_p(row, _u8p), _p(x, _f32p), x.size))


def matmul(fmt, blocks, rows: int, cols: int, x) -> np.ndarray:
    """out[t, r] = w[r] . x[t]  (gpu/cpu.rs:110-149); x is [n, cols]."""
    blocks, x = _u8(blocks), _f32(x).reshape(-1, cols)
    n = x.shape[0]
    assert blocks.size == rows * row_bytes(fmt, cols)
    out = np.empty((n, rows), np.float32)
    rc = lib().orc_matmul(_fmt(fmt), _p(blocks, _u8p), rows, cols, _p(x, _f32p), n, _p(out, _f32p))
    assert rc == 0
    return out


def matmul_add(fmt, blocks, rows: int, cols: int, inp, x) -> np.ndarray:
    """Returns x + w . inp  (gpu/mod.rs:256-268)."""
    blocks, inp = _u8(blocks), _f32(inp).reshape(-1, cols)
    n = inp.shape[0]
    out = _f32(x).reshape(n, rows).copy()
    rc = lib().orc_matmul_add(_fmt(fmt), _p(blocks, _u8p), rows, cols, _p(inp, _f32p), n, _p(out, _f32p))
    assert rc == 0
    return out


def swiglu(fmt, gate, up, rows: int, cols: int, x) -> np.ndarray:
    """silu(gate . x) * (up . x)  (gpu/mod.rs:270-285)."""
    gate, up, x = _u8(gate), _u8(up), _f32(x).reshape(-1, cols)
    n = x.shape[0]
    out = np.empty((n, rows), np.float32)
    rc = lib().orc_swiglu(_fmt(fmt), _p(gate, _u8p), _p(up, _u8p), rows, cols, _p(x, _f32p), n, _p(out, _f32p))
    assert rc == 0
    return out


def threads() -> int:
    return int(lib().orc_threads())


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


# ---- the operators either side of the product ---------------------------
def rmsnorm(x, weight, eps: float) -> np.ndarray:
    """Rows of ``x`` normalized by their root mean square, times ``weight``
    (gpu/cpu.rs:157-166; ``Device::normalize`` is a copy followed by this)."""
    weight = _f32(weight).reshape(-1)
    out = _f32(x).reshape(-1, weight.size).copy()
    lib().orc_rmsnorm.restype = None
    lib().orc_rmsnorm.argtypes = [_f32p, C.c_size_t, _f32p, C.c_size_t, C.c_float]
    lib().orc_rmsnorm(_p(out, _f32p), out.shape[0], _p(weight, _f32p), weight.size, eps)
    return out


def matmul_bf16(w_bits, rows: int, cols: int, x) -> np.ndarray:
    """out[t, r] = bf16 weights w[r] . x[t]  (gpu/cpu.rs:124-128, 370-384)."""
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16).reshape(-1)
    x = _f32(x).reshape(-1, cols)
    assert w_bits.size == rows * cols
    out = np.empty((x.shape[0], rows), np.float32)
    lib().orc_matmul_bf16.argtypes = [_u16p, C.c_size_t, C.c_size_t, _f32p, C.c_size_t, _f32p]
    lib().orc_matmul_bf16(_p(w_bits, _u16p), rows, cols, _p(x, _f32p), x.shape[0], _p(out, _f32p))
    return out


def argmax(logits) -> int:
    """First index of the largest value (inference/qwen35/mod.rs:702-710)."""
    logits = _f32(logits).reshape(-1)
    lib().orc_argmax.restype = C.c_uint32
    lib().orc_argmax.argtypes = [_f32p, C.c_size_t]
    return int(lib().orc_argmax(_p(logits, _f32p), logits.size))
