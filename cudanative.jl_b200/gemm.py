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
    (cols, rows) -- the transposed view of the same column-major memory."""
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
    handle.gemm(transA, transB, M, N, K, alpha, A, lda, B, ldb, beta if Cm is not None else 0.0, Cm, ldc, D, ldd,
                stream=stream)


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

    def __init__(self, nbytes: int):
        p = C.c_void_p()
        _lib.check(_lib.lib().b200_malloc(C.byref(p), nbytes), "b200_malloc")
        self.ptr, self.nbytes = p.value, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes // 2,), "typestr": "<f2", "data": (self.ptr, False),
                                         "version": 2, "strides": None}

    def free(self):
        if self.ptr:
            _lib.lib().b200_free(self.ptr)
            self.ptr = None


class ShardedGemm:
    """``D[:, slab_r] = alpha * A * B[:, slab_r] + beta * C[:, slab_r]`` on every rank r.

    One process per GPU.  B, C and D are split into contiguous column slabs that never move; A
    (M x K column-major, lda = M) starts on rank 0 and reaches every rank in K panels.  Panel p's
    GEMM (accumulating into D) runs while later panels are still in flight, so only the first
    panel's transfer is exposed.  There is no output collective: D stays sharded like C.

    Two transports for A:

    ``"nccl"``  ``broadcast(panel, src=0)`` per panel through torch.distributed (NCCL on GPUs, gloo in
                the CPU tests).  NCCL's broadcast is an SM kernel: the persistent GEMM grid leaves
                ``reserve_ctas`` SMs to it, and its bandwidth follows the CTAs it is given.
    ``"p2p"``   copy engines over NVLink, no SMs: per panel, rank 0 sends sub-block g of the panel to
                rank g, then every rank sends its sub-block to all others (a scatter followed by an
                all-gather, so no GPU sends more than the panel's size), each step fenced by a
                4-byte NCCL all-reduce that every rank enqueues behind its own copies.  Needs A in
                a buffer from ``alloc_a()`` (peers map it through CUDA IPC).
    """

    def __init__(self, handle: Handle, M: int, N: int, K: int, *, panels: int = 8, reserve_ctas: int | None = None,
                 group=None, sm_count: int | None = None, transport: str = "nccl"):
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
        self.n0, self.n1 = slab_bounds(N, self.world, self.rank)
        self.panels = panel_bounds(K, panels if self.world > 1 else 1)
        if reserve_ctas is None:
            reserve_ctas = 4 if self.transport == "p2p" else 8
        self.reserve_ctas = reserve_ctas if self.world > 1 else 0
        if sm_count is None:
            sm_count = torch.cuda.get_device_properties(handle.device).multi_processor_count
        self.sm_count = sm_count
        self._raw = None
        self._peers = {}
        self._copy_stream = None
        self._flag = None
        self.A = None

    @property
    def slab_cols(self) -> int:
        return self.n1 - self.n0

    # ------------------------------------------------------------------------------------------
    def alloc_a(self):
        """The M*K float16 buffer that holds A on this rank (flat torch tensor, column-major data).
        With the p2p transport it is a cudaMalloc'ed block whose IPC handle every peer maps."""
        torch, dist = self.torch, self.dist
        if self.A is not None:
            return self.A
        n = self.M * self.K
        if self.transport != "p2p":
            self.A = torch.empty(n, dtype=torch.float16, device=torch.device("cuda", self.handle.device))
            return self.A
        L = _lib.lib()
        self._raw = _RawCudaBuffer(2 * n)
        self.A = torch.as_tensor(self._raw, device=torch.device("cuda", self.handle.device))
        hnd = C.create_string_buffer(64)
        _lib.check(L.b200_ipc_get_handle(self._raw.ptr, hnd), "ipc_get_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(hnd.raw), group=self.group)
        for g, raw in enumerate(handles):
            if g == self.rank:
                continue
            p = C.c_void_p()
            _lib.check(L.b200_ipc_open_handle(raw, C.byref(p)), f"ipc_open_handle(rank {g})")
            self._peers[g] = p.value
        self._copy_stream = torch.cuda.Stream()
        self._flag = torch.ones(1, dtype=torch.int32, device=self.A.device)
        return self.A

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's A (p2p transport).  Collective in spirit:
        call it on every rank, after the last product has been synchronised."""
        L = _lib.lib()
        for p in self._peers.values():
            L.b200_ipc_close_handle(p)
        self._peers = {}
        self.A = None
        if self._raw is not None:
            self._raw.free()
            self._raw = None

    # ------------------------------------------------------------------------------------------
    def _fence(self):
        """4-byte all-reduce enqueued behind everything on the current stream; its completion on a
        rank means every rank got that far.  Returns the async work handle."""
        return self.dist.all_reduce(self._flag, op=self.dist.ReduceOp.MAX, group=self.group, async_op=True)

    def _send_panels_p2p(self, a_addr: int):
        """Enqueue the scatter + all-gather of every K panel on the copy stream; returns one work
        handle per panel whose completion means the panel is complete on every rank."""
        torch, L = self.torch, _lib.lib()
        M, G, r = self.M, self.world, self.rank
        cs = self._copy_stream
        cs.wait_stream(torch.cuda.current_stream())  # what the caller enqueued so far comes first
        ready = []
        with torch.cuda.stream(cs):
            self._fence().wait()  # nobody still reads or fills the A of the previous call
            for (k0, k1) in self.panels:
                sub = [(k0 + c0, k0 + c1) for (c0, c1) in (slab_bounds(k1 - k0, G, g, align=8) for g in range(G))]
                if r == 0:  # scatter: sub-block g goes to rank g
                    for g in range(1, G):
                        c0, c1 = sub[g]
                        if c1 > c0:
                            _lib.check(L.b200_memcpy_d2d(self._peers[g] + 2 * c0 * M, a_addr + 2 * c0 * M,
                                                         2 * (c1 - c0) * M, cs.cuda_stream), "scatter copy")
                self._fence().wait()
                c0, c1 = sub[r]  # all-gather: my sub-block goes to everybody but rank 0, which has it all
                if c1 > c0:
                    for h in range(1, G):
                        if h != r:
                            _lib.check(L.b200_memcpy_d2d(self._peers[h] + 2 * c0 * M, a_addr + 2 * c0 * M,
                                                         2 * (c1 - c0) * M, cs.cuda_stream), "all-gather copy")
                ready.append(self._fence())
        return ready

    def run(self, alpha: float, A, B_slab, beta: float, C_slab, D_slab, stream=None) -> None:
        """A: device buffer of M*K float16 on every rank (contents valid on rank 0 only before the
        call, on every rank after it; with the p2p transport it must be ``alloc_a()``'s buffer).
        B_slab: K x slab_cols (ldb = K).  C_slab / D_slab: M x slab_cols (ld = M).  All column-major
        torch tensors (flat or 2-D, any shape with the right number of elements)."""
        torch, dist = self.torch, self.dist
        M, K, ns = self.M, self.K, self.slab_cols
        a_flat = A.view(-1)
        a_addr = a_flat.data_ptr()
        works = []
        if self.world > 1:
            if self.transport == "p2p":
                if self._raw is None or a_addr != self._raw.ptr:
                    raise ValueError("the p2p transport needs A in the buffer returned by alloc_a()")
                works = self._send_panels_p2p(a_addr)
            else:
                for (k0, k1) in self.panels:
                    view = a_flat[k0 * M:k1 * M]
                    works.append(dist.broadcast(view, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                                                group=self.group, async_op=True))
        if ns == 0:
            for w in works:
                w.wait()
            return
        h = self.handle
        saved = h.get_option(_lib.OPT_MAX_CTAS)
        b_addr = B_slab.data_ptr()
        c_addr = C_slab.data_ptr() if C_slab is not None else None
        d_addr = D_slab.data_ptr()
        if stream is not None:
            s = stream
        else:
            s = torch.cuda.current_stream().cuda_stream if a_flat.is_cuda else None
        try:
            for p, (k0, k1) in enumerate(self.panels):
                last = p == len(self.panels) - 1
                if works:
                    works[p].wait()  # stream-level: the GEMM below is ordered after panel p
                if self.reserve_ctas and not last:
                    # transfers (or their fences) are still in flight: leave them a few SMs
                    h.set_option(_lib.OPT_MAX_CTAS, max(2, (self.sm_count - self.reserve_ctas) // 2 * 2))
                else:
                    h.set_option(_lib.OPT_MAX_CTAS, saved)
                h.gemm(False, False, M, ns, k1 - k0, alpha, a_addr + 2 * k0 * M, M, b_addr + 2 * k0, K,
                       beta if p == 0 else 1.0, c_addr if p == 0 else d_addr, M, d_addr, M, stream=s)
        finally:
            h.set_option(_lib.OPT_MAX_CTAS, saved)


def init_nccl_env(max_ctas: int = 8) -> None:
    """Environment NCCL reads at communicator creation: cap its CTAs so that a broadcast fits
    beside the persistent GEMM grid.  Call before ``torch.distributed.init_process_group``."""
    os.environ.setdefault("NCCL_MAX_CTAS", str(max_ctas))
