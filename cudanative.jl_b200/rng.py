"""Counter-based synthetic matrices: the numpy statement of csrc/rng.cuh plus device fills.

Element (i, j) of a rows x cols column-major matrix is a pure function of (seed, matrix_id,
j*rows + i), so any window of any matrix can be regenerated in isolation -- which is how the
tests check tiles of outputs whose full CPU product would take minutes.

The reference draws its test matrices from Julia's unseeded ``rand`` (test/device/wmma.jl:196-199
of CUDAnative.jl) and has no generator to follow; this one is specific to this library.
"""
from __future__ import annotations

import numpy as np

from . import _lib

UNIFORM, NORMAL, ZEROS = 0, 1, 2

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return x ^ (x >> np.uint64(31))


def synth_values(seed: int, matrix_id: int, index: np.ndarray, dist: int) -> np.ndarray:
    """float32 values for linear indices ``index`` (any shape, uint64-compatible)."""
    with np.errstate(over="ignore"):
        base = (np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)
                + np.uint64(matrix_id) * np.uint64(0xD1B54A32D192ED03))
        u = splitmix64(base + index.astype(np.uint64))
    if dist == UNIFORM:
        return ((u >> np.uint64(40)).astype(np.float64) * (1.0 / 8388608.0) - 1.0).astype(np.float32)
    if dist == NORMAL:
        u1 = ((u >> np.uint64(40)).astype(np.float64) + 1.0) * (1.0 / 16777216.0)
        u2 = ((u >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float64) * (1.0 / 16777216.0)
        return (np.sqrt(-2.0 * np.log(u1)) * np.cos(6.283185307179586476925 * u2)).astype(np.float32)
    if dist == ZEROS:
        return np.zeros(index.shape, dtype=np.float32)
    raise ValueError("dist must be UNIFORM, NORMAL or ZEROS")


def window(seed: int, matrix_id: int, rows: int, row0: int, row1: int, col0: int, col1: int,
           dist: int, scale: float, dtype=np.float32) -> np.ndarray:
    """Rows [row0,row1) x cols [col0,col1) of the rows-tall synthetic matrix, as a
    Fortran-ordered array of ``dtype`` (float16 rounds to nearest even, like the device)."""
    i = np.arange(row0, row1, dtype=np.uint64)[:, None]
    j = np.arange(col0, col1, dtype=np.uint64)[None, :]
    v = synth_values(seed, matrix_id, j * np.uint64(rows) + i, dist) * np.float32(scale)
    return np.asfortranarray(v.astype(dtype))


def matrix(seed: int, matrix_id: int, rows: int, cols: int, dist: int, scale: float = 1.0,
           dtype=np.float32) -> np.ndarray:
    return window(seed, matrix_id, rows, 0, rows, 0, cols, dist, scale, dtype)


def fill_device(ptr: int, rows: int, cols: int, ld: int, seed: int, matrix_id: int, dist: int,
                scale: float, f16: bool, stream=None, col0: int = 0) -> None:
    """Fill a column-major device matrix in place through the C ABI (b200_fill_f16/_f32).
    ``col0`` makes the buffer columns [col0, col0 + cols) of a wider synthetic matrix."""
    L = _lib.lib()
    fn = L.b200_fill_f16 if f16 else L.b200_fill_f32
    _lib.check(fn(stream, ptr, rows, cols, ld, seed, matrix_id, col0 * rows, dist, scale), "fill")
