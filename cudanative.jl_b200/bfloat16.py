"""bfloat16 on the host.

numpy has no bfloat16 dtype, so host arrays hold the 16-bit patterns in ``uint16`` and carry the
element type beside them as the ``BFloat16`` tag (the role ``Float16`` plays in the reference's
``WMMA.Config{16,16,16,d_type}``, src/device/cuda/wmma.jl:394; bfloat16 itself has no counterpart
there).  A bfloat16 is the upper half of an IEEE binary32: 1 sign, 8 exponent, 7 fraction bits.
"""
from __future__ import annotations

import numpy as np


class BFloat16:
    """Element-type tag for ``Handle.gemm_ex`` / ``gemm_strided_batched``; never instantiated."""

    itemsize = 2


def round_to_bf16(x) -> np.ndarray:
    """float32 values -> bfloat16 bit patterns (uint16), round to nearest, ties to even; NaN stays
    NaN (quiet), overflow rounds to infinity as IEEE rounding does."""
    f = np.ascontiguousarray(x, dtype=np.float32) if not isinstance(x, np.ndarray) else x.astype(np.float32, copy=False)
    bits = f.view(np.uint32) if f.flags.c_contiguous or f.flags.f_contiguous else np.ascontiguousarray(f).view(np.uint32)
    bits = bits.astype(np.uint64)
    lsb = (bits >> np.uint64(16)) & np.uint64(1)
    rounded = ((bits + np.uint64(0x7FFF) + lsb) >> np.uint64(16)).astype(np.uint16)
    nan = np.isnan(f)
    if np.any(nan):
        rounded = np.where(nan, ((bits >> np.uint64(16)) | np.uint64(0x0040)).astype(np.uint16), rounded)
    return rounded.reshape(f.shape, order="F" if f.flags.f_contiguous and not f.flags.c_contiguous else "C")


def widen_bf16(bits) -> np.ndarray:
    """bfloat16 bit patterns (uint16) -> the float32 values they stand for (exact)."""
    b = np.asarray(bits, dtype=np.uint16)
    order = "F" if b.flags.f_contiguous and not b.flags.c_contiguous else "C"
    out = (b.astype(np.uint32) << np.uint32(16)).view(np.float32)
    return out.reshape(b.shape, order=order)
