"""numpy / ctypes front end of the CPU oracle.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the CPU legs of
``bench.py``; never by the product package.  PARITY UNPINNED for the arithmetic (see oracle.c): the
reference delegates D = A*B + C to the wmma.mma instruction, has no golden vectors, and cannot be run
here (no Julia), so the benchmark specification's tolerances are the contract.

Two statements of the same product are kept side by side and checked against each other:

* ``gemm_ref``     -- float32 ``sgemm`` through numpy (OpenBLAS) on the Float16-rounded inputs.  This
  is the stand-in for Julia's ``LinearAlgebra.mul!`` on ``Matrix{Float32}``, which dispatches to
  OpenBLAS sgemm as well; Julia itself is not installed here.  It is also the timed CPU baseline.
* ``gemm_c``       -- the plain triple loop of oracle.c (float or double accumulation), for small
  cases and for checking gemm_ref itself.

``wmma_unit_ref`` follows the CPU side of the reference's 16x16x16 tests
(test/device/wmma.jl:223-246 of CUDAnative.jl).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"

# the benchmark specification's tolerances for the tiled GEMM
REL_FRO_TOL = 1e-3
ELEM_TOL = 1e-2
# the reference's own tolerance for the 16x16x16 unit: rtol = sqrt(eps(Float16))
UNIT_RTOL = float(np.sqrt(np.finfo(np.float16).eps))


def build() -> Path:
    """Compile oracle.c with the Makefile beside it (gcc)."""
    subprocess.run(["make", "-C", str(HERE), "liboracle.so"], check=True, capture_output=True)
    return LIB


_lib = None


def clib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists() or LIB.stat().st_mtime < (HERE / "oracle.c").stat().st_mtime:
            build()
        L = C.CDLL(str(LIB))
        fp = C.POINTER(C.c_float)
        L.oracle_f32_to_f16_bits.restype = C.c_uint16
        L.oracle_f32_to_f16_bits.argtypes = [C.c_float]
        L.oracle_f16_bits_to_f32.restype = C.c_float
        L.oracle_f16_bits_to_f32.argtypes = [C.c_uint16]
        L.oracle_round_f16.restype = C.c_float
        L.oracle_round_f16.argtypes = [C.c_float]
        u16p = C.POINTER(C.c_uint16)
        L.oracle_round_bf16_array.restype = None
        L.oracle_round_bf16_array.argtypes = [fp, u16p, C.c_int64]
        L.oracle_widen_bf16_array.restype = None
        L.oracle_widen_bf16_array.argtypes = [u16p, fp, C.c_int64]
        L.oracle_synth_value.restype = C.c_float
        L.oracle_synth_value.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_int]
        L.oracle_fill.restype = None
        L.oracle_fill.argtypes = [fp, C.c_int64, C.c_int64, C.c_int64, C.c_uint64, C.c_uint64, C.c_int64, C.c_int,
                                  C.c_float, C.c_int]
        L.oracle_gemm.restype = None
        L.oracle_gemm.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_float, fp, C.c_int64, fp,
                                  C.c_int64, C.c_float, fp, C.c_int64, fp, C.c_int64, C.c_int]
        L.oracle_gemm_f16acc.restype = None
        L.oracle_gemm_f16acc.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_float, fp, C.c_int64, fp,
                                         C.c_int64, C.c_float, fp, C.c_int64, fp, C.c_int64, C.c_int]
        L.oracle_wmma_unit.restype = None
        L.oracle_wmma_unit.argtypes = [C.c_int] * 8 + [C.c_float, C.c_int, C.c_float, fp, fp, fp, fp]
        _lib = L
    return _lib


def _fptr(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def fill(rows: int, cols: int, seed: int, matrix_id: int, dist: int, scale: float, f16: bool,
         col0: int = 0) -> np.ndarray:
    """The C generator: rows x cols window (from column col0) as a Fortran float32 array;
    ``f16`` rounds the values to binary16 (they stay stored as float32)."""
    out = np.empty((rows, cols), dtype=np.float32, order="F")
    clib().oracle_fill(_fptr(out), rows, cols, rows, seed, matrix_id, col0, dist, scale, int(f16))
    return out


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 array -> bfloat16 bit patterns (uint16, same shape and memory order), round to nearest even."""
    order = "F" if x.flags.f_contiguous and not x.flags.c_contiguous else "C"
    src = np.array(x, dtype=np.float32, order=order)
    out = np.empty(src.shape, dtype=np.uint16, order=order)
    clib().oracle_round_bf16_array(_fptr(src), out.ctypes.data_as(C.POINTER(C.c_uint16)), src.size)
    return out


def bf16_widen(bits: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) -> the float32 values they stand for."""
    order = "F" if bits.flags.f_contiguous and not bits.flags.c_contiguous else "C"
    src = np.array(bits, dtype=np.uint16, order=order)
    out = np.empty(src.shape, dtype=np.float32, order=order)
    clib().oracle_widen_bf16_array(src.ctypes.data_as(C.POINTER(C.c_uint16)), _fptr(out), src.size)
    return out


def gemm_c(transA: bool, transB: bool, alpha: float, A: np.ndarray, B: np.ndarray, beta: float, Cm, acc64: bool):
    """Triple loop of oracle.c.  A, B: Fortran float32 arrays holding binary16-representable
    values in STORED orientation (A is K x M when transA)."""
    A = np.asfortranarray(A, dtype=np.float32)
    B = np.asfortranarray(B, dtype=np.float32)
    M, K = (A.shape[1], A.shape[0]) if transA else A.shape
    N = B.shape[0] if transB else B.shape[1]
    D = np.zeros((M, N), dtype=np.float32, order="F")
    Cf = np.asfortranarray(Cm, dtype=np.float32) if Cm is not None else D
    clib().oracle_gemm(int(transA), int(transB), M, N, K, alpha, _fptr(A), A.shape[0], _fptr(B), B.shape[0],
                       beta if Cm is not None else 0.0, _fptr(Cf), M, _fptr(D), M, int(acc64))
    return D


def gemm_ref_f32(transA: bool, transB: bool, alpha: float, A: np.ndarray, B: np.ndarray, beta: float, Cm):
    """The float32 product itself (what mul!(D, A32, B32, alpha, beta) computes): operands are
    float32 arrays in STORED orientation.  This is the part the CPU baseline times."""
    opA = A.T if transA else A
    opB = B.T if transB else B
    D = np.float32(alpha) * (opA @ opB)
    if Cm is not None and beta != 0.0:
        D += np.float32(beta) * Cm
    return D


def gemm_ref(transA: bool, transB: bool, alpha: float, A16: np.ndarray, B16: np.ndarray, beta: float, Cm):
    """float32 sgemm on the Float16 inputs converted to float32: alpha*(op(A)*op(B)) + beta*C."""
    D = gemm_ref_f32(transA, transB, alpha, A16.astype(np.float32), B16.astype(np.float32), beta,
                     Cm.astype(np.float32) if Cm is not None else None)
    return np.asfortranarray(D.astype(np.float32))


def gemm_ref_f16acc(transA: bool, transB: bool, alpha: float, A16: np.ndarray, B16: np.ndarray, beta: float, C16,
                    block: int = 16):
    """The product with a binary16 accumulator, as the reference's ``Config{16, 16, 16, Float16}`` with a
    Float16 accumulator fragment computes it when a caller loops over K (the .f16.f16 mma variants,
    src/device/cuda/wmma.jl:222-257 of CUDAnative.jl; its test accepts rtol = sqrt(eps(Float16)),
    test/device/wmma.jl:243-246): the running sum is rounded to binary16 after every ``block`` (= the
    instruction's K, 16) products; inside a block the products are summed in binary32.  alpha and beta
    are applied in binary32 and the result is rounded to binary16 once.  Hardware may round inside a
    block differently, hence the tolerance the tests state."""
    opA = (A16.T if transA else A16).astype(np.float32)
    opB = (B16.T if transB else B16).astype(np.float32)
    M, K = opA.shape
    N = opB.shape[1]
    acc = np.zeros((M, N), dtype=np.float16)
    for k0 in range(0, K, block):
        part = opA[:, k0:k0 + block] @ opB[k0:k0 + block, :]
        acc = (acc.astype(np.float32) + part).astype(np.float16)
    D = np.float32(alpha) * acc.astype(np.float32)
    if C16 is not None and beta != 0.0:
        D = D + np.float32(beta) * C16.astype(np.float32)
    return np.asfortranarray(D.astype(np.float16))


def gemm_c_f16acc(transA: bool, transB: bool, alpha: float, A: np.ndarray, B: np.ndarray, beta: float, Cm, block: int = 16):
    """The triple loop of oracle.c with a binary16 accumulator (oracle_gemm_f16acc): the second statement
    ``gemm_ref_f16acc`` is checked against.  Operands as for ``gemm_c``; returns float32 holding binary16 values."""
    A = np.asfortranarray(A, dtype=np.float32)
    B = np.asfortranarray(B, dtype=np.float32)
    M, K = (A.shape[1], A.shape[0]) if transA else A.shape
    N = B.shape[0] if transB else B.shape[1]
    D = np.zeros((M, N), dtype=np.float32, order="F")
    Cf = np.asfortranarray(Cm, dtype=np.float32) if Cm is not None else D
    clib().oracle_gemm_f16acc(int(transA), int(transB), M, N, K, alpha, _fptr(A), A.shape[0], _fptr(B), B.shape[0],
                              beta if Cm is not None else 0.0, _fptr(Cf), M, _fptr(D), M, block)
    return D


def errors(D: np.ndarray, ref: np.ndarray) -> tuple[float, float]:
    """(relative Frobenius error, max over elements of |D-ref| / (|ref|+1))."""
    D64 = D.astype(np.float64)
    R64 = ref.astype(np.float64)
    diff = D64 - R64
    denom = np.linalg.norm(R64)
    rel = float(np.linalg.norm(diff) / denom) if denom > 0 else float(np.linalg.norm(diff))
    elem = float(np.max(np.abs(diff) / (np.abs(R64) + 1.0))) if diff.size else 0.0
    return rel, elem


def assert_close(D: np.ndarray, ref: np.ndarray, what: str = "") -> tuple[float, float]:
    """Acceptance of the benchmark specification: rel-Frobenius <= 1e-3 and |D-ref| <= 1e-2*(|ref|+1) elementwise."""
    assert D.shape == ref.shape, f"{what}: shape {D.shape} vs {ref.shape}"
    assert np.all(np.isfinite(D)), f"{what}: non-finite output"
    rel, elem = errors(D, ref)
    assert rel <= REL_FRO_TOL, f"{what}: relative Frobenius error {rel:.3e} > {REL_FRO_TOL}"
    assert elem <= ELEM_TOL, f"{what}: per-element error {elem:.3e} > {ELEM_TOL}"
    return rel, elem


def wmma_unit_ref(a16: np.ndarray, b16: np.ndarray, c, *, a_layout=0, b_layout=0, c_layout=0, d_layout=0,
                  d_type=np.float32, alpha=None, beta=None) -> np.ndarray:
    """The 16x16x16 unit: a16, b16 are the STORED 16x16 float16 arrays (Fortran order), c the
    stored float16/float32 array or None (fill_c(0)).  Returns the STORED d array of d_type."""
    a = np.asfortranarray(a16.astype(np.float32))
    b = np.asfortranarray(b16.astype(np.float32))
    c_is_f16 = int(c is not None and c.dtype == np.float16) if c is not None else int(np.dtype(d_type) == np.float16)
    cf = np.asfortranarray(c.astype(np.float32)) if c is not None else np.zeros((16, 16), np.float32, order="F")
    d = np.zeros((16, 16), dtype=np.float32, order="F")
    clib().oracle_wmma_unit(a_layout, b_layout, c_layout, d_layout, c_is_f16, int(np.dtype(d_type) == np.float16),
                            int(c is not None), int(alpha is not None), 0.0 if alpha is None else float(alpha),
                            int(beta is not None), 0.0 if beta is None else float(beta), _fptr(a), _fptr(b),
                            _fptr(cf), _fptr(d))
    return np.asfortranarray(d.astype(d_type))


def unit_close(d: np.ndarray, ref: np.ndarray) -> bool:
    """The reference's acceptance for the unit: all(isapprox.(ref, d; rtol=sqrt(eps(Float16))))
    (test/device/wmma.jl:243-246).  Julia's isapprox(x, y; rtol) is |x-y| <= rtol*max(|x|,|y|)."""
    x = ref.astype(np.float64)
    y = d.astype(np.float64)
    return bool(np.all(np.abs(x - y) <= UNIT_RTOL * np.maximum(np.abs(x), np.abs(y))))
