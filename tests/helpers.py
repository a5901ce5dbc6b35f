"""Shared helpers of the GPU parity tests: synthetic operands on the device and oracle checks."""
from __future__ import annotations

import numpy as np

from cudanative_jl_b200 import _lib, rng
from cudanative_jl_b200.array import Array, CuArray


def operands(M, N, K, transA, transB, seed, *, a_scale=None, c_dist=rng.UNIFORM, lda=None, ldb=None):
    """Host float16 A, B (in STORED orientation) and float32 C drawn from the counter-based
    generator: A ~ normal/sqrt(K), B ~ normal, C ~ c_dist."""
    a_shape = (K, M) if transA else (M, K)
    b_shape = (N, K) if transB else (K, N)
    a = rng.matrix(seed, 0, *a_shape, rng.NORMAL, (K ** -0.5 if K else 1.0) if a_scale is None else a_scale, np.float16)
    b = rng.matrix(seed, 1, *b_shape, rng.NORMAL, 1.0, np.float16)
    c = rng.matrix(seed, 2, M, N, c_dist, 1.0, np.float32)
    return a, b, c


def padded(host: np.ndarray, ld: int, fill=np.nan) -> np.ndarray:
    """Copy a Fortran matrix into a taller one (leading dimension ld); the padding rows hold
    ``fill`` so that a kernel writing outside its window is caught."""
    out = np.full((ld, host.shape[1]), fill, dtype=host.dtype, order="F")
    out[:host.shape[0], :] = host
    return out


def run_gemm(handle, transA, transB, M, N, K, alpha, a, b, beta, c, *, ldd=None, d_init=None):
    """Upload, launch through the C ABI, check the device status word, download D."""
    ldd = M if ldd is None else ldd
    a_dev, b_dev = CuArray(a), CuArray(b)
    c_dev = CuArray(c) if c is not None else None
    d_host = np.full((ldd, N), np.float32(-7.25), dtype=np.float32, order="F") if d_init is None else d_init
    d_dev = CuArray(d_host)
    handle.gemm(transA, transB, M, N, K, alpha, a_dev, a.shape[0], b_dev, b.shape[0], beta, c_dev,
                c.shape[0] if c is not None else max(M, 1), d_dev, ldd)
    _lib.check(_lib.lib().b200_stream_sync(None), "sync")
    code, block, detail = handle.device_status()
    assert code == 0, f"device wait {code} ran out in block {block} (detail {detail})"
    return Array(d_dev)
