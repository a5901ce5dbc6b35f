"""ctypes binding of libb200wmma.so: one Python callable per symbol of include/b200wmma.h.

There is no fallback.  If the shared library has not been built (``python -m`` style:
``build.build()`` in this package, which shells out to nvcc) loading raises, and every entry
point of the package raises with it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200wmma.so"

OK, INVALID_ARG, UNSUPPORTED, CUDA_ERROR, DEVICE_TIMEOUT, NO_DEVICE, PEER_TIMEOUT = range(7)
COL_MAJOR, ROW_MAJOR = 0, 1
F16, F32, BF16 = 0, 1, 2
MATRIX_A, MATRIX_B, ACCUMULATOR = 0, 1, 2
LOWER_WARP, LOWER_TCGEN05 = 0, 1
KERNEL_AUTO, KERNEL_TCGEN05, KERNEL_SIMPLE = 0, 1, 2
(OPT_FORCE_KERNEL, OPT_MAX_CTAS, OPT_WAIT_BUDGET_NS, OPT_TILE_N, OPT_SPLIT_K, OPT_CTA_PAIR,
 OPT_RASTER_GROUP, OPT_CHECK_ON_CALL, OPT_PDL, OPT_F16_ACCUMULATE) = range(10)
SHARDED_GATED, SHARDED_NO_TRANSFER, SHARDED_NO_COMPUTE = 1, 2, 4
SHARDED_OPT_SCATTER_LANES, SHARDED_OPT_GATHER_LANES, SHARDED_OPT_FIRST_GROUP = 0, 1, 2
SHARDED_MAX_RANKS, SHARDED_MAX_PANELS, SHARDED_BLOB_BYTES = 64, 32, 128

_i, _i64, _u64, _f, _p, _sz = C.c_int, C.c_int64, C.c_uint64, C.c_float, C.c_void_p, C.c_size_t
_pp = C.POINTER(C.c_void_p)
_ip = C.POINTER(C.c_int)

# symbol -> (restype, argtypes); the single source the loader and the export test both read
SIGNATURES = {
    "b200_last_error": (C.c_char_p, []),
    "b200_status_string": (C.c_char_p, [_i]),
    "b200_version": (_i, []),
    "b200_device_count": (_i, []),
    "b200_create": (_i, [_pp, _i]),
    "b200_destroy": (_i, [_p]),
    "b200_set_option": (_i, [_p, _i, _i64]),
    "b200_get_option": (_i, [_p, _i, C.POINTER(_i64)]),
    "b200_device_status": (_i, [_p, _ip, _ip, _ip]),
    "b200_selftest_bounded_wait": (_i, [_p, _p, _i64]),
    "b200_last_launch": (_i, [_p, _ip, _ip, _ip, _ip, _ip]),
    "b200_gemm_f16f32": (_i, [_p, _p, _i, _i, _i64, _i64, _i64, _f, _p, _i64, _p, _i64, _f, _p, _i64, _p, _i64]),
    "b200_gemm_f16_typed": (_i, [_p, _p, _i, _i, _i64, _i64, _i64, _f, _p, _i64, _p, _i64, _f, _p, _i64, _i, _p, _i64, _i]),
    "b200_gemm_ex": (_i, [_p, _p, _i, _i, _i64, _i64, _i64, _f, _p, _i64, _p, _i64, _i, _f, _p, _i64, _i, _p, _i64, _i]),
    "b200_gemm_strided_batched": (_i, [_p, _p, _i, _i, _i64, _i64, _i64, _f, _p, _i64, _i64, _p, _i64, _i64, _i, _f, _p, _i64,
                                       _i64, _i, _p, _i64, _i64, _i, _i64]),
    "b200_gemm_f16f32_gated": (_i, [_p, _p, _i, _i, _i64, _i64, _i64, _f, _p, _i64, _p, _i64, _f, _p, _i64, _p, _i64, _p, _i64]),
    "b200_stream_write_u32": (_i, [_p, _p, C.c_uint32]),
    "b200_stream_wait_u32": (_i, [_p, _p, C.c_uint32]),
    "b200_gemm_f16f32_host": (_i, [_p, _i, _i, _i64, _i64, _i64, _f, _p, _i64, _p, _i64, _f, _p, _i64, _p, _i64]),
    "b200_gemm_f16f32_splitk_static": (_i, [_p, _i, _i, _i64, _i64, _i64, _f, _p, _i64, _p, _i64, _f, _p, _i64, _p, _i64, _i, _i]),
    "b200_wmma_16x16x16": (_i, [_p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _f, _p, _i64, _p, _i64, _p, _i64, _p, _i64]),
    "b200_wmma_load": (_i, [_p, _i, _i, _i, _p, _i64, _p]),
    "b200_wmma_fill_c": (_i, [_p, _i, _f, _p]),
    "b200_wmma_bcast": (_i, [_p, _i, _i, _i, _f, _p, _p]),
    "b200_wmma_mma": (_i, [_p, _i, _i, _p, _p, _p, _p]),
    "b200_wmma_store_d": (_i, [_p, _i, _i, _p, _p, _i64]),
    "b200_malloc": (_i, [_pp, _sz]),
    "b200_free": (_i, [_p]),
    "b200_host_alloc": (_i, [_pp, _sz]),
    "b200_host_free": (_i, [_p]),
    "b200_memcpy_h2d": (_i, [_p, _p, _sz, _p]),
    "b200_memcpy_d2h": (_i, [_p, _p, _sz, _p]),
    "b200_static_warmup": (_i, []),
    "b200_static_status": (_i, [_ip, _ip, _ip]),
    "b200_static_selftest_bounded_wait": (_i, [_p, _i64]),
    "b200_sharded_create": (_i, [_pp, _p, _i, _i, _i64, _i64, _i64, _i]),
    "b200_sharded_destroy": (_i, [_p]),
    "b200_sharded_set_option": (_i, [_p, _i, _i64]),
    "b200_sharded_set_groups": (_i, [_p, _ip, _i]),
    "b200_sharded_info": (_i, [_p, C.POINTER(_i64), C.POINTER(_i64), _pp, _pp, _ip, _ip]),
    "b200_sharded_ipc_blob": (_i, [_p, _p]),
    "b200_sharded_attach": (_i, [_p, _p]),
    "b200_sharded_attach_local": (_i, [_p, _pp, _pp]),
    "b200_sharded_run": (_i, [_p, _p, _f, _p, _i64, _f, _p, _i64, _p, _i64, _i]),
    "b200_sharded_wait": (_i, [_p, _i64]),
    "b200_sharded_layout": (_i, [_i, _i64, _i64, _i, C.POINTER(_i64), C.POINTER(_i64), _ip, _ip, _ip, C.POINTER(_i64)]),
    "b200_ipc_get_handle": (_i, [_p, _p]),
    "b200_ipc_open_handle": (_i, [_p, _pp]),
    "b200_ipc_close_handle": (_i, [_p]),
    "b200_memcpy_d2d": (_i, [_p, _p, _sz, _p]),
    "b200_memset": (_i, [_p, _i, _sz, _p]),
    "b200_stream_sync": (_i, [_p]),
    "b200_stream_create": (_i, [_pp]),
    "b200_stream_destroy": (_i, [_p]),
    "b200_fill_f16": (_i, [_p, _p, _i64, _i64, _i64, _u64, _u64, _u64, _i, _f]),
    "b200_fill_f32": (_i, [_p, _p, _i64, _i64, _i64, _u64, _u64, _u64, _i, _f]),
    "b200_fill_bf16": (_i, [_p, _p, _i64, _i64, _i64, _u64, _u64, _u64, _i, _f]),
}


class B200Error(RuntimeError):
    """A non-zero status from the C ABI; ``status`` holds the B200_* code."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """The loaded shared library (loads it on first use; raises if it is not built)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with nvcc first (cudanative.jl_b200/build.py, or "
                "__graft_entry__.build()).  This package has no CPU or PyTorch fallback.")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, what: str = "") -> None:
    """Raise B200Error for a non-zero status, with the library's own error text."""
    if status != OK:
        L = lib()
        name = L.b200_status_string(status).decode()
        text = L.b200_last_error().decode()
        raise B200Error(status, f"{what + ': ' if what else ''}{name}: {text}")
