"""Host-side weight matrices: the counterpart of the engine's ``Tensor``
(gpu/mod.rs:43-168) for GGUF block formats.

A ``Tensor`` is a ``[rows, cols]`` matrix held as raw GGUF blocks, row-major.
Only byte moves happen here (selecting rows or column groups, as the loader
does when it splits fused projections); decoding and arithmetic are the
device's job (``B200.dequantize``, ``B200.matmul``).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ._lib import BF16, Q4_K, Q6_K, Q8_0

# format id -> (name, weights per block, bytes per block)
FORMATS = {
    Q8_0: ("Q8_0", 32, 34),
    Q4_K: ("Q4_K", 256, 144),
    Q6_K: ("Q6_K", 256, 210),
    BF16: ("BF16", 1, 2),       # plain bf16 weights (Tensor::Bf16, gpu/mod.rs:46-50)
}
BY_NAME = {name.lower(): fmt for fmt, (name, _, _) in FORMATS.items()}


def format_id(fmt) -> int:
    if isinstance(fmt, str):
        try:
            return BY_NAME[fmt.lower()]
        except KeyError:
            raise ValueError(f"unknown weight format {fmt!r}") from None
    if int(fmt) not in FORMATS:
        raise ValueError(f"unknown weight format {fmt!r}")
    return int(fmt)


def row_bytes(fmt, cols: int) -> int:
    """Bytes of a row of ``cols`` weights (inference/gguf.rs:36-53)."""
    _, per, size = FORMATS[format_id(fmt)]
    if cols % per:
        raise ValueError("rows must be a whole number of blocks")   # gpu/quant.rs:22-29
    return cols // per * size


@dataclass
class Tensor:
    fmt: int
    shape: tuple
    data: np.ndarray   # uint8, rows * row_bytes

    def __post_init__(self):
        self.fmt = format_id(self.fmt)
        self.shape = (int(self.shape[0]), int(self.shape[1]))
        self.data = np.ascontiguousarray(self.data).view(np.uint8).reshape(-1)
        want = self.shape[0] * row_bytes(self.fmt, self.shape[1])
        if self.data.size != want:
            raise ValueError(f"a {self.shape} {FORMATS[self.fmt][0]} matrix is {want} bytes, not {self.data.size}")

    @property
    def rows(self) -> int:
        return self.shape[0]

    @property
    def cols(self) -> int:
        return self.shape[1]

    def _by_row(self) -> np.ndarray:
        return self.data.reshape(self.rows, -1) if self.rows else self.data.reshape(0, row_bytes(self.fmt, self.cols))

    def select_rows(self, rows) -> "Tensor":
        """The matrix made of the given rows, in the given order; a row may be
        taken more than once or not at all (gpu/mod.rs:72-101)."""
        idx = np.asarray(rows, dtype=np.int64)
        return Tensor(self.fmt, (idx.size, self.cols), self._by_row()[idx].copy())

    def select_column_groups(self, width: int, groups) -> "Tensor":
        """The matrix with its columns taken in groups of ``width``, in the
        given order of groups; the groups must be whole blocks of the format
        (gpu/mod.rs:103-136)."""
        _, per, size = FORMATS[self.fmt]
        if self.cols % width:
            raise ValueError("cols must be a whole number of groups")
        if width % per:
            raise ValueError("the groups must be whole blocks of the format")
        idx = np.asarray(groups, dtype=np.int64)
        gb = width // per * size
        by_group = self._by_row().reshape(self.rows, self.cols // width, gb)
        return Tensor(self.fmt, (self.rows, idx.size * width), by_group[:, idx, :].copy())

    def slice_rows(self, begin: int, end: int) -> "Tensor":
        """Rows [begin, end): what one rank holds of a row-sharded matrix."""
        return Tensor(self.fmt, (end - begin, self.cols), self._by_row()[begin:end].copy())
