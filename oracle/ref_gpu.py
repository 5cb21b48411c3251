"""TEST INFRASTRUCTURE ONLY: the reference engine's own CUDA tile kernel
(matmul_tile.cu:94-258), run on this box as the same-hardware baseline.

``make -C oracle ref_gpu`` compiles the reference's sources where they lie into
``oracle/_ref/dwim_tile.cubin`` (nothing of them is kept in this repository).
This module restates the host side that feeds the kernel, which is Rust in the
reference and cannot be built here:

* ``tile_q4_0``: the weight layout of ``tile`` / ``q4_0_words``
  (gpu/cuda/mod.rs:642-704): 128-row by 64-column tiles, a row's two blocks
  as eight words ``[b[2i], b[2i+8], b[2i+1], b[2i+9]]``, the tile's scales a
  block of columns at a time;
* ``RefTile.matmul``: the launches of ``matmul_tiles`` (gpu/cuda/mod.rs:402-442):
  whole 64-token tiles through ``matmul_tile64_q4_0``, the rest in 16-token
  tiles through ``matmul_tile16_q4_0``, grid ``(ceil(count / tokens),
  ceil(rows / 128))``, 128 threads, ``tile_shared`` bytes of shared memory
  (gpu/cuda/mod.rs:625-631), mode FLOATS.

Q4_0 has the density of Q4_K (18 bytes per 32 weights), so bytes and flops
per second compare directly.  Only the tests and the benchmark's baseline legs
import this.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
CUBIN = _DIR / "_ref" / "dwim_tile.cubin"
TILE_ROWS, TILE_COLS, STAGES = 128, 64, 3


def build(reference: str = "/root/reference") -> bool:
    """Builds the cubin when the reference's sources are present (they are not
    on a GPU box, which uses the file built beforehand)."""
    if CUBIN.exists():
        return True
    if not (Path(reference) / "gpu" / "cuda" / "kernels" / "matmul_tile.cu").exists():
        return False
    subprocess.run(["make", "-C", str(_DIR), "ref_gpu", f"REF={reference}"], check=True, capture_output=True)
    return CUBIN.exists()


def available() -> bool:
    return CUBIN.exists()


def quantize_q4_0(w: np.ndarray):
    """Rows of f32 to the reference's split Q4_0 (gpu/quant.rs:85-126) through
    the oracle: scales u16 [rows, blocks], quants u8 [rows, blocks, 16]."""
    import oracle
    rows, cols = w.shape
    scales = np.empty((rows, cols // 32), np.uint16)
    quants = np.empty((rows, cols // 32, 16), np.uint8)
    for r in range(rows):
        s, q = oracle.quantize_q4_0_row_split(w[r])
        scales[r], quants[r] = s, q.reshape(-1, 16)
    return scales, quants


def tile_q4_0(scales: np.ndarray, quants: np.ndarray):
    """gpu/cuda/mod.rs:642-704.  Returns (tiled u32 [groups, tiles, 128, 8],
    tiled_scales u16 [groups, tiles, 2, 128]); rows and blocks past the
    matrix's are zeros with a scale of zero."""
    rows, blocks = scales.shape
    tiles, groups = -(-blocks // 2), -(-rows // TILE_ROWS)
    q = np.zeros((groups * TILE_ROWS, tiles * 2, 16), np.uint8)
    s = np.zeros((groups * TILE_ROWS, tiles * 2), np.uint16)
    q[:rows, :blocks], s[:rows, :blocks] = quants, scales
    i = np.arange(4)
    # word i of a block: bytes 2i, 2i+8, 2i+1, 2i+9, little-endian
    order = np.stack([2 * i, 2 * i + 8, 2 * i + 1, 2 * i + 9], axis=1).reshape(-1)      # [4 words x 4 bytes]
    words = np.ascontiguousarray(q[:, :, order]).view(np.uint32)                         # [R, tiles*2, 4]
    words = words.reshape(groups, TILE_ROWS, tiles, 2, 4)                                # [g, r, t, v, i]
    tiled = np.ascontiguousarray(words.transpose(0, 2, 1, 4, 3))                         # [g, t, r, i, v]: word i*2 + v
    ts = np.ascontiguousarray(s.reshape(groups, TILE_ROWS, tiles, 2).transpose(0, 2, 3, 1))   # [g, t, v, r]
    return tiled.reshape(groups, tiles, TILE_ROWS, 8), ts


class TileParams(C.Structure):      # prelude.cu:37-47
    _fields_ = [("rows", C.c_uint32), ("cols", C.c_uint32), ("tiles", C.c_uint32), ("first", C.c_uint32),
                ("count", C.c_uint32), ("mode", C.c_uint32)]


class RefTile:
    """The loaded kernels.  CUDA must be initialised (torch has a context) first."""

    def __init__(self):
        from cuda.bindings import driver as cu
        self.cu = cu
        err, self.module = cu.cuModuleLoadData(CUBIN.read_bytes())
        self._ok(err, "cuModuleLoadData")
        self.fn = {}
        for name in ("matmul_tile64_q4_0", "matmul_tile16_q4_0"):
            err, f = cu.cuModuleGetFunction(self.module, name.encode())
            self._ok(err, name)
            self.fn[name] = f

    def _ok(self, err, what):
        if int(err) != 0:
            raise RuntimeError(f"{what}: CUDA driver error {int(err)}")

    @staticmethod
    def shared_bytes(tokens: int) -> int:     # tile_shared, gpu/cuda/mod.rs:625-631, one byte to a pair
        return STAGES * (tokens * TILE_COLS * 2 + TILE_ROWS * TILE_COLS // 2 + 2 * TILE_ROWS * 2)

    def matmul(self, out_ptr: int, w_ptr: int, s_ptr: int, x16_ptr: int, rows: int, cols: int, n: int, stream: int) -> int:
        """out f32 [n, rows] = tiled Q4_0 weights . halves x [n, cols]; returns the launches made."""
        whole, launches = n // 64 * 64, 0
        for name, tokens, first, count in (("matmul_tile64_q4_0", 64, 0, whole), ("matmul_tile16_q4_0", 16, whole, n - whole)):
            if count == 0:
                continue
            p = TileParams(rows, cols, -(-cols // TILE_COLS), first, count, 0)
            args = [C.c_void_p(out_ptr), C.c_void_p(w_ptr), C.c_void_p(s_ptr), C.c_void_p(x16_ptr), C.c_void_p(0), p]
            ptrs = (C.c_void_p * len(args))(*[C.addressof(a) for a in args])
            err, = self.cu.cuLaunchKernel(self.fn[name], -(-count // tokens), -(-rows // TILE_ROWS), 1, 128, 1, 1,
                                          self.shared_bytes(tokens), stream, C.addressof(ptrs), 0)
            self._ok(err, f"launching {name}")
            launches += 1
        return launches
