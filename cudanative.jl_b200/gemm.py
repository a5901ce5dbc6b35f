"""The tiled GEMM ``D = alpha * op(A) * op(B) + beta * C`` and its N-sharded multi-GPU form.

Reference: CUDAnative.jl has no multi-tile GEMM; its WMMA examples compute one 16x16x16 product
per launch (examples/wmma/high-level.jl:30-46).  This module is that same load_a/load_b/load_c ->
mma -> store_d sequence (src/device/cuda/wmma.jl:507-632) scaled to whole matrices, with the
column-major ``CuArray`` layout (src/device/array.jl:104) and the asynchronous, stream-ordered
launch convention of ``@cuda`` (src/execution.jl:158-166) kept.

Everything here hands pointers to ``libb200wmma.so``; PyTorch appears only as an owner of device
memory, as the source of the current CUDA stream and, in ``ShardedGemm``, as the NCCL front end.
"""
from __future__ import annotations

import ctypes as C
import os

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
# N-sharded multi-GPU GEMM
# --------------------------------------------------------------------------------------------------
def slab_bounds(n: int, world_size: int, rank: int, align: int = 256) -> tuple[int, int]:
    """Columns [n0, n1) of rank ``rank``: contiguous slabs, multiples of ``align`` columns except
    possibly the last non-empty one, as even as that allows."""
    blocks = -(-n // align)
    per, extra = divmod(blocks, world_size)
    b0 = rank * per + min(rank, extra)
    b1 = b0 + per + (1 if rank < extra else 0)
    return min(b0 * align, n), min(b1 * align, n)


def panel_bounds(k: int, panels: int, align: int = 64) -> list[tuple[int, int]]:
    """Split [0, k) into at most ``panels`` contiguous ranges whose starts are multiples of
    ``align`` (a K panel must start on a shared-memory stage boundary)."""
    blocks = -(-k // align)
    panels = max(1, min(panels, blocks))
    per, extra = divmod(blocks, panels)
    out, b = [], 0
    for p in range(panels):
        nb = per + (1 if p < extra else 0)
        out.append((min(b * align, k), min((b + nb) * align, k)))
        b += nb
    return out


class _RawCudaBuffer:
    """A b200_malloc'ed device buffer exposed through ``__cuda_array_interface__`` so that torch can
    view it without copying (the IPC handle of a cudaMalloc'ed block is what peers can map)."""

    def __init__(self, nbytes: int, typestr: str = "<f2", itemsize: int = 2):
        p = C.c_void_p()
        _lib.check(_lib.lib().b200_malloc(C.byref(p), nbytes), "b200_malloc")
        self.ptr, self.nbytes = p.value, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes // itemsize,), "typestr": typestr, "data": (self.ptr, False),
                                         "version": 2, "strides": None}

    def free(self):
        if self.ptr:
            _lib.lib().b200_free(self.ptr)
            self.ptr = None


def launch_groups(n_panels: int, first: int = 1, growth: float = 2.5) -> list[tuple[int, int]]:
    """Group n transfer panels into GEMM launches [p0, p1) of geometrically growing size: the first
    launch starts as soon as little of A has arrived, later launches are long enough that their
    fixed cost and their extra pass over D do not matter.  While launch i computes, the panels of
    launch i+1 arrive: with compute slower than the transfer, growth up to 1 + compute/transfer
    keeps every launch fed."""
    out, p, size = [], 0, float(max(1, first))
    while p < n_panels:
        q = min(n_panels, p + max(1, int(round(size))))
        out.append((p, q))
        size *= growth
        p = q
    if len(out) > 1 and out[-1][1] - out[-1][0] < (out[-2][1] - out[-2][0]) // 2:
        last = out.pop()
        out[-1] = (out[-1][0], last[1])
    return out


def subblock_cols(panels: list[tuple[int, int]], world: int) -> list[list[tuple[int, int]]]:
    """For every K panel [k0, k1) the column range of A each rank owns during the transfer:
    ``out[p][g] = (c0, c1)``.  A panel is cut into world - 1 sub-blocks, one per receiving rank, so
    that rank 0 sends every byte of A exactly once (its link is the bottleneck of the scatter) and
    forwards nothing; rank 0's own range is empty."""
    out = []
    for (k0, k1) in panels:
        row = [(k0, k0)]
        for g in range(1, world):
            c0, c1 = slab_bounds(k1 - k0, world - 1, g - 1, align=8)
            row.append((k0 + c0, k0 + c1))
        out.append(row)
    return out


class ShardedGemm:
    """``D[:, slab_r] = alpha * A * B[:, slab_r] + beta * C[:, slab_r]`` on every rank r.

    One process per GPU.  B, C and D are split into contiguous column slabs that never move; A
    (M x K column-major, lda = M) starts on rank 0 and reaches every rank in K panels, while the
    GEMM on the panels that have already arrived is running.  There is no output collective: D
    stays sharded like C.

    Two transports for A:

    ``"nccl"``  ``broadcast(panel, src=0)`` per panel through torch.distributed (NCCL on GPUs, gloo in
                the CPU tests).  NCCL's broadcast is an SM kernel: the persistent GEMM grid leaves
                ``reserve_ctas`` SMs to it, and its bandwidth follows the CTAs it is given.
    ``"p2p"``   copy engines over NVLink, no SMs and no kernels at all: per panel, rank 0 copies
                sub-block g of the panel into rank g's A (scatter), then every rank copies its
                sub-block into every other rank's A (all-gather), so no GPU sends more than the
                panel's size.  Arrival is signalled by stream memory operations: behind each copy the
                sender's stream writes the call's epoch into a flag word in the receiver's memory,
                and the receiver's streams wait for that word before they forward the data or launch
                the GEMM that reads it.  Needs A in the buffer from ``alloc_a()`` (peers map it and
                the flag words through CUDA IPC).

    The product itself is a sequence of GEMM launches over growing K ranges (``launch_groups``), each
    accumulating into D and ordered behind the arrival of its own panels only; with ``fused=True``
    (p2p) it is instead ONE launch of the gated GEMM, whose TMA producer waits for per-panel flag
    words itself -- that form overlaps transfer and main loop inside one kernel and writes D once,
    but its first wave of tiles cannot finish before all of A has arrived.
    """

    MAX_PANELS = 32

    def __init__(self, handle: Handle, M: int, N: int, K: int, *, panels: int = 16, reserve_ctas: int | None = None,
                 group=None, sm_count: int | None = None, transport: str = "nccl", fused: bool = False,
                 grouping: str | None = None):
        import torch
        import torch.distributed as dist

        if transport not in ("nccl", "p2p"):
            raise ValueError("transport must be 'nccl' or 'p2p'")
        self.torch, self.dist = torch, dist
        self.handle = handle
        self.M, self.N, self.K = M, N, K
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.transport = transport if self.world > 1 else "nccl"
        self.fused = bool(fused) and self.world > 1
        if self.fused and self.transport != "p2p":
            raise ValueError("fused=True needs the p2p transport")
        self.n0, self.n1 = slab_bounds(N, self.world, self.rank)
        # transfer panels: equal ranges of whole 64-wide k-blocks
        panels = max(1, min(panels if self.world > 1 else 1, self.MAX_PANELS))
        self.panel_k = -(-(-(-K // panels)) // 64) * 64  # ceil(ceil(K / panels) / 64) * 64
        self.panels = [(k0, min(K, k0 + self.panel_k)) for k0 in range(0, K, self.panel_k)]
        # GEMM launches: groups of consecutive panels
        if grouping is None:
            grouping = "geometric" if self.transport == "p2p" else "each"
        if grouping == "geometric":
            self.groups = launch_groups(len(self.panels))
        elif grouping == "each":
            self.groups = [(p, p + 1) for p in range(len(self.panels))]
        else:
            raise ValueError("grouping must be 'geometric' or 'each'")
        if reserve_ctas is None:
            reserve_ctas = 0 if self.transport == "p2p" else 8
        self.reserve_ctas = reserve_ctas if self.world > 1 else 0
        if sm_count is None:
            sm_count = torch.cuda.get_device_properties(handle.device).multi_processor_count
        self.sm_count = sm_count
        self._raw = None
        self._raw_flags = None
        self._peers = {}
        self._peer_flags = {}
        self._scatter_stream = None
        self._gather_stream = None
        self._gate_words = None
        self._epoch = 0
        self.A = None

    @property
    def slab_cols(self) -> int:
        return self.n1 - self.n0

    _FLAG_BYTES = 4 * (128 + 32 * 64)  # B200_P2P_FLAG_BYTES

    # ------------------------------------------------------------------------------------------
    def alloc_a(self):
        """The M*K float16 buffer that holds A on this rank (flat torch tensor, column-major data).
        With the p2p transport it is a cudaMalloc'ed block which, like the block of flag words
        beside it, every peer maps through CUDA IPC."""
        torch, dist = self.torch, self.dist
        if self.A is not None:
            return self.A
        n = self.M * self.K
        dev = torch.device("cuda", self.handle.device)
        if self.transport != "p2p":
            self.A = torch.empty(n, dtype=torch.float16, device=dev)
            return self.A
        if self.world > 64:
            raise ValueError("the p2p transport supports at most 64 ranks")
        L = _lib.lib()
        self._raw = _RawCudaBuffer(2 * n)
        self._raw_flags = _RawCudaBuffer(self._FLAG_BYTES)
        _lib.check(L.b200_memset(self._raw_flags.ptr, 0, self._FLAG_BYTES, None), "clear flags")
        _lib.check(L.b200_stream_sync(None), "clear flags")
        self.A = torch.as_tensor(self._raw, device=dev)
        mine = []
        for buf in (self._raw, self._raw_flags):
            hnd = C.create_string_buffer(64)
            _lib.check(L.b200_ipc_get_handle(buf.ptr, hnd), "ipc_get_handle")
            mine.append(bytes(hnd.raw))
        handles = [None] * self.world
        dist.all_gather_object(handles, mine, group=self.group)  # also orders the clears above before any use
        for g, (ha, hf) in enumerate(handles):
            if g == self.rank:
                continue
            pa, pf = C.c_void_p(), C.c_void_p()
            _lib.check(L.b200_ipc_open_handle(ha, C.byref(pa)), f"ipc_open_handle(A of rank {g})")
            _lib.check(L.b200_ipc_open_handle(hf, C.byref(pf)), f"ipc_open_handle(flags of rank {g})")
            self._peers[g], self._peer_flags[g] = pa.value, pf.value
        self._scatter_stream = torch.cuda.Stream()
        self._gather_stream = torch.cuda.Stream()
        self._gate_words = torch.zeros(self.MAX_PANELS, dtype=torch.int32, device=dev)
        # tables the C side walks: every rank's A and flag block, and the sub-block column ranges
        G, P = self.world, len(self.panels)
        self._a_table = (C.c_void_p * G)(*[self._raw.ptr if g == self.rank else self._peers[g] for g in range(G)])
        self._flag_table = (C.c_void_p * G)(*[self._raw_flags.ptr if g == self.rank else self._peer_flags[g] for g in range(G)])
        cols = [c for panel in subblock_cols(self.panels, G) for rng_ in panel for c in rng_]
        self._sub_cols = (C.c_int64 * (2 * G * P))(*cols)
        return self.A

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's A and flags (p2p transport).  Call it on
        every rank after the last product has been synchronised everywhere."""
        L = _lib.lib()
        for p in list(self._peers.values()) + list(self._peer_flags.values()):
            L.b200_ipc_close_handle(p)
        self._peers, self._peer_flags = {}, {}
        self.A = None
        for buf in (self._raw, self._raw_flags):
            if buf is not None:
                buf.free()
        self._raw = self._raw_flags = None

    # ------------------------------------------------------------------------------------------
    def _p2p_begin(self, cur_stream) -> int:
        """Start a product: new epoch, 'done with my A' handshake with every peer (b200_p2p_begin)."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        self._scatter_stream.wait_stream(cur)
        self._gather_stream.wait_stream(cur)
        self._epoch += 1
        _lib.check(_lib.lib().b200_p2p_begin(self.rank, self.world, self._flag_table, self._epoch, cur_stream,
                                             self._scatter_stream.cuda_stream, self._gather_stream.cuda_stream), "p2p_begin")
        return self._epoch

    def _p2p_exchange(self, cur_stream, p0: int, p1: int, gates=None) -> None:
        """Enqueue the transfer of panels [p0, p1) and order `cur_stream` behind their arrival here."""
        _lib.check(_lib.lib().b200_p2p_exchange(self.rank, self.world, self.M, self._sub_cols, p0, p1, self._a_table,
                                                self._flag_table, self._epoch, cur_stream,
                                                self._scatter_stream.cuda_stream, self._gather_stream.cuda_stream,
                                                gates), "p2p_exchange")

    def run(self, alpha: float, A, B_slab, beta: float, C_slab, D_slab, stream=None) -> None:
        """A: device buffer of M*K float16 on every rank (contents valid on rank 0 only before the
        call, on every rank after it; with the p2p transport it must be ``alloc_a()``'s buffer).
        B_slab: K x slab_cols (ldb = K).  C_slab / D_slab: M x slab_cols (ld = M).  All column-major
        torch tensors (flat or 2-D, any shape with the right number of elements).  Every rank must
        make the call, also one whose slab is empty."""
        torch, dist = self.torch, self.dist
        M, K, ns = self.M, self.K, self.slab_cols
        a_flat = A.view(-1)
        a_addr = a_flat.data_ptr()
        if stream is not None:
            s = stream
        else:
            s = torch.cuda.current_stream().cuda_stream if a_flat.is_cuda else None
        works = []
        p2p = self.world > 1 and self.transport == "p2p"
        if p2p:
            if self._raw is None or a_addr != self._raw.ptr:
                raise ValueError("the p2p transport needs A in the buffer returned by alloc_a()")
            self._p2p_begin(s)
        elif self.world > 1:
            for (k0, k1) in self.panels:
                view = a_flat[k0 * M:k1 * M]
                works.append(dist.broadcast(view, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                                            group=self.group, async_op=True))
        h = self.handle
        saved = h.get_option(_lib.OPT_MAX_CTAS)
        b_addr = B_slab.data_ptr()
        c_addr = C_slab.data_ptr() if C_slab is not None else None
        d_addr = D_slab.data_ptr()
        reserved = max(2, (self.sm_count - self.reserve_ctas) // 2 * 2) if self.reserve_ctas else saved
        try:
            if self.fused and p2p:
                # one launch: the producer warps wait for the panel gates themselves; the transfers are
                # enqueued behind the launch so that the waits they put on this stream follow it
                L = _lib.lib()
                gates = self._gate_words.data_ptr()
                _lib.check(L.b200_memset(gates, 1 if self.rank == 0 else 0, 4 * self.MAX_PANELS, s), "arm gates")
                self._gather_stream.wait_stream(torch.cuda.current_stream())
                if ns:
                    h.set_option(_lib.OPT_MAX_CTAS, reserved)
                    h.gemm_gated(False, False, M, ns, K, alpha, a_addr, M, b_addr, K, beta, c_addr, M, d_addr, M,
                                 gates, self.panel_k, stream=s)
                self._p2p_exchange(s, 0, len(self.panels), gates)
                return
            for i, (p0, p1) in enumerate(self.groups):
                last = i == len(self.groups) - 1
                if p2p:
                    self._p2p_exchange(s, p0, p1)  # transfers of this group, then the waits for them
                else:
                    for w in works[p0:p1]:
                        w.wait()  # stream-level: the GEMM below is ordered after these panels
                if not ns:
                    continue
                # while transfers that need SMs are still in flight, leave them a few
                h.set_option(_lib.OPT_MAX_CTAS, saved if last else reserved)
                k0, k1 = self.panels[p0][0], self.panels[p1 - 1][1]
                h.gemm(False, False, M, ns, k1 - k0, alpha, a_addr + 2 * k0 * M, M, b_addr + 2 * k0, K,
                       beta if i == 0 else 1.0, c_addr if i == 0 else d_addr, M, d_addr, M, stream=s)
        finally:
            h.set_option(_lib.OPT_MAX_CTAS, saved)


def init_nccl_env(max_ctas: int = 8) -> None:
    """Environment NCCL reads at communicator creation: cap its CTAs so that a broadcast fits
    beside the persistent GEMM grid.  Call before ``torch.distributed.init_process_group``."""
    os.environ.setdefault("NCCL_MAX_CTAS", str(max_ctas))
