"""The tiled GEMM ``D = alpha * op(A) * op(B) + beta * C`` and its N-sharded multi-GPU form.

Reference: CUDAnative.jl has no multi-tile GEMM; its WMMA examples compute one 16x16x16 product
per launch (examples/wmma/high-level.jl:30-46).  This module is that same load_a/load_b/load_c ->
mma -> store_d sequence (src/device/cuda/wmma.jl:507-632) scaled to whole matrices, with the
column-major ``CuArray`` layout (src/device/array.jl:104) and the asynchronous, stream-ordered
launch convention of ``@cuda`` (src/execution.jl:158-166) kept.

Everything here hands pointers to ``libb200wmma.so`` and imports neither PyTorch nor any other GPU
library; ``nccl_broadcast.py`` holds the one variant of the sharded product that moves A with
``torch.distributed``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .array import CuHostArray, DevicePtr
from .bfloat16 import BFloat16


def _type_code(t) -> int:
    """numpy dtype (float16 / float32) or the ``BFloat16`` tag -> the library's element tag."""
    if t is BFloat16:
        return _lib.BF16
    dt = np.dtype(t)
    if dt == np.float16:
        return _lib.F16
    if dt == np.float32:
        return _lib.F32
    raise TypeError(f"invalid element type {t!r}: Float16, BFloat16 or Float32")


class Handle:
    """Per-device library handle (status word, host-path workspace, split-K scratch)."""

    def __init__(self, device: int = 0):
        L = _lib.lib()
        h = C.c_void_p()
        _lib.check(L.b200_create(C.byref(h), int(device)), "b200_create")
        self._h = h
        self.device = int(device)

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().b200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def set_option(self, option: int, value: int) -> None:
        _lib.check(_lib.lib().b200_set_option(self._h, option, int(value)), "set_option")

    def get_option(self, option: int) -> int:
        v = C.c_int64()
        _lib.check(_lib.lib().b200_get_option(self._h, option, C.byref(v)), "get_option")
        return v.value

    def device_status(self) -> tuple[int, int, int]:
        """(code, block, detail) of the device status word; call after synchronising."""
        code, block, detail = C.c_int(), C.c_int(), C.c_int()
        _lib.check(_lib.lib().b200_device_status(self._h, C.byref(code), C.byref(block), C.byref(detail)),
                   "device_status")
        return code.value, block.value, detail.value

    def last_launch(self) -> dict:
        v = [C.c_int() for _ in range(5)]
        _lib.check(_lib.lib().b200_last_launch(self._h, *[C.byref(x) for x in v]), "last_launch")
        return dict(zip(("kernel", "tile_n", "split_k", "ctas", "cta_pair"), (x.value for x in v)))

    # -- device pointers ---------------------------------------------------------------------
    def gemm(self, transA: bool, transB: bool, M: int, N: int, K: int, alpha: float, A, lda: int, B, ldb: int,
             beta: float, Cm, ldc: int, D, ldd: int, stream=None) -> None:
        """Raw form: A, B, C, D are device addresses (ints), DevicePtr, CuHostArray or CUDA tensors."""
        a, b, d = _addr(A), _addr(B), _addr(D)
        c = _addr(Cm) if Cm is not None else None
        _lib.check(_lib.lib().b200_gemm_f16f32(self._h, stream, int(bool(transA)), int(bool(transB)), M, N, K,
                                               float(alpha), a, lda, b, ldb, float(beta), c, ldc, d, ldd), "gemm")

    def gemm_typed(self, transA: bool, transB: bool, M: int, N: int, K: int, alpha: float, A, lda: int, B, ldb: int,
                   beta: float, Cm, ldc: int, c_type, D, ldd: int, d_type, stream=None) -> None:
        """``gemm`` with Float16 or Float32 C and D (b200_gemm_f16_typed); types are numpy dtypes."""
        code = {np.dtype(np.float16): _lib.F16, np.dtype(np.float32): _lib.F32}
        a, b, d = _addr(A), _addr(B), _addr(D)
        c = _addr(Cm) if Cm is not None else None
        _lib.check(_lib.lib().b200_gemm_f16_typed(self._h, stream, int(bool(transA)), int(bool(transB)), M, N, K,
                                                  float(alpha), a, lda, b, ldb, float(beta), c, ldc, code[np.dtype(c_type)],
                                                  d, ldd, code[np.dtype(d_type)]), "gemm_typed")

    def gemm_ex(self, transA: bool, transB: bool, M: int, N: int, K: int, alpha: float, A, lda: int, B, ldb: int,
                ab_type, beta: float, Cm, ldc: int, c_type, D, ldd: int, d_type, stream=None) -> None:
        """``gemm`` with A and B both Float16 or both ``BFloat16`` and C, D each Float16, ``BFloat16`` or
        Float32 (b200_gemm_ex); accumulation is binary32 throughout."""
        self.gemm_strided_batched(transA, transB, M, N, K, alpha, A, lda, 0, B, ldb, 0, ab_type, beta, Cm, ldc, 0,
                                  c_type, D, ldd, 0, d_type, 1, stream=stream)

    def gemm_strided_batched(self, transA: bool, transB: bool, M: int, N: int, K: int, alpha: float, A, lda: int,
                             stride_a: int, B, ldb: int, stride_b: int, ab_type, beta: float, Cm, ldc: int,
                             stride_c: int, c_type, D, ldd: int, stride_d: int, d_type, batch: int, stream=None) -> None:
        """``batch`` products of one shape, matrix i of X starting ``stride_x * i`` elements after X
        (b200_gemm_strided_batched); a stride of 0 repeats A, B or C."""
        a, b, d = _addr(A), _addr(B), _addr(D)
        c = _addr(Cm) if Cm is not None else None
        _lib.check(_lib.lib().b200_gemm_strided_batched(
            self._h, stream, int(bool(transA)), int(bool(transB)), M, N, K, float(alpha), a, lda, stride_a, b, ldb,
            stride_b, _type_code(ab_type), float(beta), c, ldc, stride_c, _type_code(c_type), d, ldd, stride_d,
            _type_code(d_type), batch), "gemm_strided_batched")

    def gemm_gated(self, transA: bool, transB: bool, M: int, N: int, K: int, alpha: float, A, lda: int, B, ldb: int,
                   beta: float, Cm, ldc: int, D, ldd: int, panel_flags, panel_k: int, stream=None) -> None:
        """``gemm`` whose main loop reads columns [j*panel_k, (j+1)*panel_k) of op(A) only once the
        32-bit device word ``panel_flags[j]`` is non-zero (b200_gemm_f16f32_gated)."""
        a, b, d = _addr(A), _addr(B), _addr(D)
        c = _addr(Cm) if Cm is not None else None
        _lib.check(_lib.lib().b200_gemm_f16f32_gated(self._h, stream, int(bool(transA)), int(bool(transB)), M, N, K,
                                                     float(alpha), a, lda, b, ldb, float(beta), c, ldc, d, ldd,
                                                     _addr(panel_flags), panel_k), "gemm_gated")

    # -- host buffers (numpy, ideally page-locked) ---------------------------------------------
    def gemm_host(self, transA: bool, transB: bool, M: int, N: int, K: int, alpha: float, A: np.ndarray, lda: int,
                  B: np.ndarray, ldb: int, beta: float, Cm, ldc: int, D: np.ndarray, ldd: int) -> None:
        """Host-buffer form: upload, multiply, download, synchronise (b200_gemm_f16f32_host)."""
        if A.dtype != np.float16 or B.dtype != np.float16 or D.dtype != np.float32:
            raise TypeError("A and B must be float16, D float32")
        if Cm is not None and Cm.dtype != np.float32:
            raise TypeError("C must be float32")
        _lib.check(_lib.lib().b200_gemm_f16f32_host(
            self._h, int(bool(transA)), int(bool(transB)), M, N, K, float(alpha), A.ctypes.data, lda,
            B.ctypes.data, ldb, float(beta), Cm.ctypes.data if Cm is not None else None, ldc, D.ctypes.data, ldd),
            "gemm_host")


def _addr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return DevicePtr.of(x).addr


def _dtype(x) -> np.dtype:
    return DevicePtr.of(x).dtype


def _dims(x):
    """(rows, cols, ld) of a column-major 2-D operand: CuHostArray, or a torch tensor holding
    the matrix transposed (shape (cols, rows), contiguous), which is how row-major torch stores a
    column-major matrix."""
    if isinstance(x, CuHostArray):
        return x.shape[0], x.shape[1], x.shape[0]
    cols, rows = x.shape
    if x.stride(1) != 1:
        raise ValueError("tensor must be contiguous in its last dimension")
    return rows, cols, x.stride(0)


def gemm_f16f32(handle: Handle, D, A, B, Cm=None, *, alpha: float = 1.0, beta: float = 0.0, transA: bool = False,
                transB: bool = False, stream=None) -> None:
    """``D = alpha*op(A)*op(B) + beta*C`` on column-major device matrices.

    Operands are ``CuHostArray`` (shape (rows, cols)) or CUDA tensors whose torch shape is
    (cols, rows) -- the transposed view of the same column-major memory.  C and D may be Float16 or
    Float32 independently (the reference's four Config / load_c type combinations); A and B are Float16."""
    ar, ac, lda = _dims(A)
    br, bc, ldb = _dims(B)
    M, K = (ac, ar) if transA else (ar, ac)
    K2, N = (bc, br) if transB else (br, bc)
    if K != K2:
        raise ValueError(f"inner dimensions differ: {K} vs {K2}")
    dr, dc, ldd = _dims(D)
    if (dr, dc) != (M, N):
        raise ValueError(f"D is {dr}x{dc}, expected {M}x{N}")
    ldc = ldd
    if Cm is not None:
        cr, cc, ldc = _dims(Cm)
        if (cr, cc) != (M, N):
            raise ValueError(f"C is {cr}x{cc}, expected {M}x{N}")
    elif beta != 0.0:
        raise ValueError("beta != 0 needs C")
    c_type = _dtype(Cm) if Cm is not None else np.dtype(np.float32)
    d_type = _dtype(D)
    if c_type == np.float32 and d_type == np.float32:
        handle.gemm(transA, transB, M, N, K, alpha, A, lda, B, ldb, beta if Cm is not None else 0.0, Cm, ldc, D, ldd,
                    stream=stream)
    else:
        handle.gemm_typed(transA, transB, M, N, K, alpha, A, lda, B, ldb, beta if Cm is not None else 0.0, Cm, ldc, c_type,
                          D, ldd, d_type, stream=stream)


# --------------------------------------------------------------------------------------------------
# N-sharded multi-GPU GEMM (b200_sharded_*)
# --------------------------------------------------------------------------------------------------
class ShardLayout:
    """What b200_sharded_layout says about a product: column slabs of B / C / D per rank, K panels in
    which A travels, GEMM launches as groups of panels, and per panel the columns of A every rank
    forwards.  Pure host arithmetic (no GPU needed)."""

    def __init__(self, world: int, N: int, K: int, panels: int = 16):
        L = _lib.lib()
        slab = (C.c_int64 * (_lib.SHARDED_MAX_RANKS + 1))()
        panel = (C.c_int64 * (_lib.SHARDED_MAX_PANELS + 1))()
        group = (C.c_int * (_lib.SHARDED_MAX_PANELS + 1))()
        sub = (C.c_int64 * (2 * max(world, 1) * _lib.SHARDED_MAX_PANELS))()
        n_p, n_g = C.c_int(), C.c_int()
        _lib.check(L.b200_sharded_layout(world, N, K, panels, slab, panel, C.byref(n_p), group, C.byref(n_g), sub),
                   "sharded_layout")
        self.world = world
        self.slabs = [(slab[r], slab[r + 1]) for r in range(world)]
        self.panels = [(panel[p], panel[p + 1]) for p in range(n_p.value)]
        self.groups = [(group[g], group[g + 1]) for g in range(n_g.value)]
        self.sub_cols = [[(sub[(p * world + g) * 2], sub[(p * world + g) * 2 + 1]) for g in range(world)]
                         for p in range(n_p.value)]


class DeviceView:
    """A device address range exposed through ``__cuda_array_interface__`` so that array libraries
    (torch.as_tensor, cupy.asarray) can view it without copying.  Owns nothing."""

    def __init__(self, ptr: int, count: int, typestr: str = "<f2"):
        self.ptr = ptr
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 2,
                                         "strides": None}


class ShardedGemm:
    """``D[:, slab_r] = alpha * A * B[:, slab_r] + beta * C[:, slab_r]`` on every rank r: a thin
    caller of the b200_sharded_* entry points, one object per rank, one rank per GPU.

    B, C and D are split into contiguous column slabs that never move.  A (M x K column-major,
    lda = M, Float16) lives in a buffer the library owns on every rank (``a_ptr``): valid on rank 0
    before a product, everywhere after it.  It travels over NVLink on the copy engines in K panels
    while the GEMM on the panels that have arrived is already running.

    ``exchange`` moves the ranks' 128-byte IPC blobs: a callable taking this rank's ``bytes`` and
    returning every rank's, in rank order (MPI allgather, torch.distributed.all_gather_object, files
    -- anything).  Ranks that live in one process pass ``exchange=None`` and call
    ``attach_local`` with each other's objects instead.
    """

    def __init__(self, handle: Handle, M: int, N: int, K: int, *, rank: int = 0, world: int = 1, panels: int = 16,
                 exchange=None):
        L = _lib.lib()
        self.handle, self.M, self.N, self.K = handle, M, N, K
        self.rank, self.world = rank, world
        s = C.c_void_p()
        _lib.check(L.b200_sharded_create(C.byref(s), handle._h, rank, world, M, N, K, panels), "sharded_create")
        self._s = s
        n0, n1 = C.c_int64(), C.c_int64()
        a, f = C.c_void_p(), C.c_void_p()
        n_p, n_g = C.c_int(), C.c_int()
        _lib.check(L.b200_sharded_info(s, C.byref(n0), C.byref(n1), C.byref(a), C.byref(f), C.byref(n_p), C.byref(n_g)),
                   "sharded_info")
        self.n0, self.n1 = n0.value, n1.value
        self.a_ptr, self.flags_ptr = a.value, f.value
        self.n_panels, self.n_groups = n_p.value, n_g.value
        if world > 1 and exchange is not None:
            blob = C.create_string_buffer(_lib.SHARDED_BLOB_BYTES)
            _lib.check(L.b200_sharded_ipc_blob(s, blob), "sharded_ipc_blob")
            blobs = exchange(bytes(blob.raw))
            if len(blobs) != world or any(len(b) != _lib.SHARDED_BLOB_BYTES for b in blobs):
                raise ValueError("exchange must return one 128-byte blob per rank, in rank order")
            _lib.check(L.b200_sharded_attach(s, b"".join(blobs)), "sharded_attach")

    @property
    def slab_cols(self) -> int:
        return self.n1 - self.n0

    def a_view(self) -> DeviceView:
        """This rank's A buffer (M * K Float16, column-major) as a zero-copy view for array libraries."""
        return DeviceView(self.a_ptr, self.M * self.K)

    def attach_local(self, peers: "list[ShardedGemm]") -> None:
        """Peers that live in this process (``peers[r]`` = the object of rank r, this one included)."""
        a = (C.c_void_p * self.world)(*[p.a_ptr for p in peers])
        f = (C.c_void_p * self.world)(*[p.flags_ptr for p in peers])
        _lib.check(_lib.lib().b200_sharded_attach_local(self._s, a, f), "sharded_attach_local")

    def set_option(self, option: int, value: int) -> None:
        """One of _lib.SHARDED_OPT_* (b200_sharded_set_option); the same on every rank, between products."""
        _lib.check(_lib.lib().b200_sharded_set_option(self._s, option, int(value)), "sharded_set_option")
        n_p, n_g = C.c_int(), C.c_int()
        _lib.check(_lib.lib().b200_sharded_info(self._s, None, None, None, None, C.byref(n_p), C.byref(n_g)), "sharded_info")
        self.n_panels, self.n_groups = n_p.value, n_g.value

    def set_groups(self, sizes) -> None:
        """Panels per GEMM launch (b200_sharded_set_groups); must add up to ``n_panels``."""
        arr = (C.c_int * len(sizes))(*[int(x) for x in sizes])
        _lib.check(_lib.lib().b200_sharded_set_groups(self._s, arr, len(sizes)), "sharded_set_groups")
        self.n_groups = len(sizes)

    def run(self, alpha: float, B_slab, beta: float, C_slab, D_slab, *, stream=None, gated: bool = False,
            no_transfer: bool = False, no_compute: bool = False, ldb: int | None = None, ldc: int | None = None, ldd: int | None = None) -> None:
        """Enqueue one product (b200_sharded_run).  B_slab: K x slab_cols, C_slab / D_slab: M x
        slab_cols, column-major device matrices (addresses, DevicePtr, CuHostArray or CUDA tensors).
        Every rank must make the call, also one whose slab is empty."""
        flags = ((_lib.SHARDED_GATED if gated else 0) | (_lib.SHARDED_NO_TRANSFER if no_transfer else 0) |
                 (_lib.SHARDED_NO_COMPUTE if no_compute else 0))
        _lib.check(_lib.lib().b200_sharded_run(self._s, stream, float(alpha), _addr(B_slab), ldb or self.K, float(beta),
                                               _addr(C_slab) if C_slab is not None else None, ldc or self.M,
                                               _addr(D_slab), ldd or self.M, flags), "sharded_run")

    def wait(self, timeout_ms: int = 60000) -> None:
        """Host-side wait with a deadline (b200_sharded_wait): raises B200Error with status
        PEER_TIMEOUT when a peer never wrote its flags (the object is unusable afterwards) or
        DEVICE_TIMEOUT when a bounded wait ran out inside a kernel."""
        _lib.check(_lib.lib().b200_sharded_wait(self._s, int(timeout_ms)), "sharded_wait")

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's.  Call it on every rank after the last
        product has been synchronised everywhere."""
        if getattr(self, "_s", None):
            _lib.lib().b200_sharded_destroy(self._s)
            self._s = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
