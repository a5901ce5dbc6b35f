"""The N-sharded GEMM with A broadcast by a collective library: ``torch.distributed.broadcast`` per
K panel (NCCL over NVLink on GPUs, gloo in the CPU tests), one GEMM launch per panel ordered behind
its broadcast.

This is the transport the task statement names.  NCCL's broadcast is an SM kernel, so the
persistent GEMM grid leaves ``reserve_ctas`` SMs to it while panels are in flight, and its
bandwidth follows the CTAs it is given; the copy-engine transport behind ``gemm.ShardedGemm``
(b200_sharded_* in the C ABI) needs neither and is the default of ``bench.py``.  PyTorch appears
here as the front end of the collective library and as the owner of A only; the product itself is
``Handle.gemm``.

No counterpart in the reference (single device per task: src/init.jl:187-209 of CUDAnative.jl).
"""
from __future__ import annotations

import os

from . import _lib


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



class NcclBroadcastGemm:
    """``D[:, slab_r] = alpha * A * B[:, slab_r] + beta * C[:, slab_r]`` on every rank r, with A
    (M x K column-major, valid on rank 0 before the call, everywhere after it) broadcast in K panels."""

    MAX_PANELS = 32

    def __init__(self, handle, M: int, N: int, K: int, *, panels: int = 16, reserve_ctas: int = 8, group=None,
                 sm_count: int | None = None):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.handle = handle
        self.M, self.N, self.K = M, N, K
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n0, self.n1 = slab_bounds(N, self.world, self.rank)
        panels = max(1, min(panels if self.world > 1 else 1, self.MAX_PANELS))
        self.panel_k = -(-(-(-K // panels)) // 64) * 64  # ceil(ceil(K / panels) / 64) * 64
        self.panels = [(k0, min(K, k0 + self.panel_k)) for k0 in range(0, K, self.panel_k)]
        self.reserve_ctas = reserve_ctas if self.world > 1 else 0
        if sm_count is None:
            sm_count = torch.cuda.get_device_properties(handle.device).multi_processor_count
        self.sm_count = sm_count

    @property
    def slab_cols(self) -> int:
        return self.n1 - self.n0

    def run(self, alpha: float, A, B_slab, beta: float, C_slab, D_slab, stream=None) -> None:
        """A: M*K float16 tensor on every rank.  B_slab: K x slab_cols (ldb = K).  C_slab / D_slab:
        M x slab_cols (ld = M).  Column-major data in torch tensors of any shape with the right
        number of elements.  Every rank must make the call, also one whose slab is empty."""
        torch, dist = self.torch, self.dist
        M, K, ns = self.M, self.K, self.slab_cols
        a_flat = A.view(-1)
        a_addr = a_flat.data_ptr()
        if stream is not None:
            s = stream
        else:
            s = torch.cuda.current_stream().cuda_stream if a_flat.is_cuda else None
        works = []
        if self.world > 1:
            src = dist.get_global_rank(self.group, 0) if self.group else 0
            for (k0, k1) in self.panels:
                works.append(dist.broadcast(a_flat[k0 * M:k1 * M], src=src, group=self.group, async_op=True))
        h = self.handle
        saved = h.get_option(_lib.OPT_MAX_CTAS)
        b_addr = B_slab.data_ptr()
        c_addr = C_slab.data_ptr() if C_slab is not None else None
        d_addr = D_slab.data_ptr()
        reserved = max(2, (self.sm_count - self.reserve_ctas) // 2 * 2) if self.reserve_ctas else saved
        try:
            for i, (k0, k1) in enumerate(self.panels):
                last = i == len(self.panels) - 1
                if works:
                    works[i].wait()  # stream-level: the GEMM below is ordered after this panel
                if not ns:
                    continue
                # while broadcasts that need SMs are still in flight, leave them a few
                h.set_option(_lib.OPT_MAX_CTAS, saved if last else reserved)
                h.gemm(False, False, M, ns, k1 - k0, alpha, a_addr + 2 * k0 * M, M, b_addr + 2 * k0, K,
                       beta if i == 0 else 1.0, c_addr if i == 0 else d_addr, M, d_addr, M, stream=s)
        finally:
            h.set_option(_lib.OPT_MAX_CTAS, saved)


def init_nccl_env(max_ctas: int = 8) -> None:
    """Environment NCCL reads at communicator creation: cap its CTAs so that a broadcast fits
    beside the persistent GEMM grid.  Call before ``torch.distributed.init_process_group``."""
    os.environ.setdefault("NCCL_MAX_CTAS", str(max_ctas))
