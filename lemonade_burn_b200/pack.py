"""Packed ternary layout and absmean ternariser: the host side of lb-ternary's `pack` module.

Mirrors crates/lb-ternary/src/pack.rs (names and argument meaning kept): rows are packed
row-major; each 128-weight block is 32 bytes; byte j of a block holds in bits 2k..2k+1 the
code (w + 1) of column block*128 + k*32 + j; columns are padded to a multiple of 128 with
code 1 (weight 0). These run offline (the converter, crates/lb-convert/src/main.rs:62-87),
so they are plain vectorised numpy on the host; the kernels only ever read the result.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

BLOCK = 128        # pack.rs:18
BLOCK_BYTES = 32   # pack.rs:19


def padded_cols(cols: int) -> int:
    """pack.rs:22-24"""
    return (cols + BLOCK - 1) // BLOCK * BLOCK


def row_bytes(cols: int) -> int:
    """pack.rs:83-85"""
    return padded_cols(cols) // 4


def pack_rows(values: np.ndarray) -> np.ndarray:
    """pack_row (pack.rs:88-103) for every row of an int8 [rows, cols] matrix of {-1,0,1}."""
    values = np.asarray(values)
    if values.ndim != 2:
        raise ValueError("expected a [rows, cols] matrix")
    if values.size and (values.min() < -1 or values.max() > 1):
        raise ValueError("non-ternary value")  # pack.rs:97 debug_assert
    rows, cols = values.shape
    kp = padded_cols(cols)
    codes = np.ones((rows, kp), dtype=np.uint8)          # pad = code 1
    codes[:, :cols] = (values.astype(np.int16) + 1).astype(np.uint8) & 3
    c = codes.reshape(rows, kp // BLOCK, 4, 32)          # [row, block, k, j]
    out = c[:, :, 0] | (c[:, :, 1] << 2) | (c[:, :, 2] << 4) | (c[:, :, 3] << 6)
    return np.ascontiguousarray(out.reshape(rows, kp // 4))


def pack_row(values: np.ndarray) -> np.ndarray:
    """pack.rs:88-103 for one row."""
    return pack_rows(np.asarray(values).reshape(1, -1))[0]


def unpack_row(row: np.ndarray, padded: int) -> np.ndarray:
    """pack.rs:106-116: packed row -> int8 values of the padded length."""
    row = np.asarray(row, dtype=np.uint8).reshape(padded // BLOCK, 1, 32)
    shifts = np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 4, 1)
    return (((row >> shifts) & 3).astype(np.int8) - 1).reshape(padded)


def absmean_f32(w: np.ndarray) -> np.float32:
    """pack.rs:135-138: f64 sum of |w|, rounded once to f32."""
    w = np.asarray(w, dtype=np.float32)
    return np.float32(np.abs(w.astype(np.float64)).sum() / w.size)


def ternarize_with_scale(w: np.ndarray, scale) -> np.ndarray:
    """pack.rs:140-142: round_ties_even(w*scale).clamp(-1,1) as i8 (np.rint is ties-to-even)."""
    w = np.asarray(w, dtype=np.float32)
    r = np.rint(w * np.float32(scale))
    r = np.where(np.isnan(r), np.float32(0), np.clip(r, -1, 1))
    return r.astype(np.int8)


def ternarize_absmean(w: np.ndarray):
    """pack.rs:129-133 -> (values, scale) with scale = 1/max(mean|w|, 1e-5)."""
    mean = absmean_f32(w)
    scale = np.float32(1.0) / np.maximum(mean, np.float32(1e-5))
    return ternarize_with_scale(w, scale), np.float32(scale)


@dataclass
class TernaryView:
    """Borrowed view of a packed matrix (pack.rs:28-56)."""
    rows: int
    cols: int
    data: np.ndarray  # uint8, rows * row_bytes(cols)
    scale: float

    def __post_init__(self):
        self.data = np.ascontiguousarray(self.data, dtype=np.uint8).reshape(-1)
        if self.data.size != self.rows * row_bytes(self.cols):  # pack.rs:40
            raise ValueError("packed data length mismatch")

    def row_bytes(self) -> int:
        return row_bytes(self.cols)

    def row(self, r: int) -> np.ndarray:
        rb = self.row_bytes()
        return self.data[r * rb:(r + 1) * rb]

    def unpack_row(self, r: int) -> np.ndarray:
        return unpack_row(self.row(r), padded_cols(self.cols))[: self.cols]


@dataclass
class PackedTernary:
    """Owned packed matrix (pack.rs:58-81)."""
    rows: int
    cols: int
    data: np.ndarray
    scale: float

    @classmethod
    def from_ternary(cls, rows: int, cols: int, values, scale: float) -> "PackedTernary":
        values = np.asarray(values, dtype=np.int8)
        if values.size != rows * cols:  # pack.rs:70
            raise ValueError("values length mismatch")
        return cls(rows, cols, pack_rows(values.reshape(rows, cols)).reshape(-1), float(scale))

    def view(self) -> TernaryView:
        return TernaryView(self.rows, self.cols, self.data, self.scale)
