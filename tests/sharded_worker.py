"""One rank of the N-sharded GEMM check; launched by test_sharded_gpu.py (one rank per GPU) and by
test_sharded_host.py (gloo on CPU with a stand-in for the GEMM call).

Transports: ``p2p`` = the b200_sharded_* entry points of the C ABI (copy engines over NVLink; torch
only carries the 128-byte IPC blobs between the ranks), ``nccl`` = NcclBroadcastGemm (broadcast of A
through torch.distributed, which is also what the gloo run exercises).

Every rank regenerates its own slabs from the counter-based generator, runs the product twice and
compares its D slab and (ranks other than 0) its copy of A with the CPU oracle.  Exit code 0 = this
rank's slab is right."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
oracle = entry.load_oracle()
from cudanative_jl_b200 import _lib, rng  # noqa: E402
from cudanative_jl_b200.gemm import ShardedGemm  # noqa: E402
from cudanative_jl_b200.nccl_broadcast import NcclBroadcastGemm, init_nccl_env  # noqa: E402


class OracleHandle:
    """Stand-in for gemm.Handle on machines without a GPU: same ``gemm`` signature, computes with
    the CPU oracle on the memory the addresses point to.  Used only by the gloo host-logic test."""

    device = 0

    def __init__(self):
        self.opts = {}
        self.calls = []

    def get_option(self, opt):
        return self.opts.get(opt, 0)

    def set_option(self, opt, value):
        self.opts[opt] = value

    def gemm(self, transA, transB, M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc, D, ldd, stream=None):
        import ctypes as C

        def view(addr, rows, cols, ld, ctype, dtype):
            buf = (ctype * (ld * cols)).from_address(addr)
            return np.frombuffer(buf, dtype=dtype).reshape((ld, cols), order="F")[:rows]

        a = view(A, M, K, lda, C.c_uint16, np.float16)
        b = view(B, K, N, ldb, C.c_uint16, np.float16)
        c = view(Cm, M, N, ldc, C.c_float, np.float32).copy() if beta != 0.0 else None
        d = view(D, M, N, ldd, C.c_float, np.float32)
        d[:] = oracle.gemm_ref(False, False, alpha, a, b, beta, c)
        self.calls.append((K, self.opts.get(_lib.OPT_MAX_CTAS, 0)))


def main():
    backend = sys.argv[1]
    M, N, K = (int(x) for x in sys.argv[2:5])
    panels = int(sys.argv[5]) if len(sys.argv) > 5 else 4
    transport = sys.argv[6] if len(sys.argv) > 6 else "nccl"
    fused = (sys.argv[7] == "fused") if len(sys.argv) > 7 else False
    seed, alpha, beta = 4, 1.0, 1.0
    rank = int(os.environ["RANK"])
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        init_nccl_env(8)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from cudanative_jl_b200.gemm import Handle

        handle = Handle(local)
        handle.set_option(_lib.OPT_WAIT_BUDGET_NS, 500_000_000)
        dev = torch.device("cuda", local)
    else:
        dist.init_process_group("gloo")
        handle = OracleHandle()
        dev = torch.device("cpu")
    p2p = backend == "nccl" and transport == "p2p"
    if p2p:
        def exchange(blob):
            blobs = [None] * dist.get_world_size()
            dist.all_gather_object(blobs, blob)
            return blobs
        sg = ShardedGemm(handle, M, N, K, rank=rank, world=dist.get_world_size(), panels=panels, exchange=exchange)
    else:
        sg = NcclBroadcastGemm(handle, M, N, K, panels=panels, reserve_ctas=8, sm_count=148)
    n0, ns = sg.n0, sg.slab_cols
    a_host = rng.matrix(seed, 0, M, K, rng.NORMAL, K ** -0.5, np.float16)
    b_host = rng.window(seed, 1, K, 0, K, n0, n0 + ns, rng.NORMAL, K ** -0.5, np.float16)
    c_host = rng.window(seed, 2, M, 0, M, n0, n0 + ns, rng.NORMAL, 1.0, np.float32)
    # torch holds the column-major matrices as their transposes
    if p2p:
        A = torch.as_tensor(sg.a_view(), device=dev)
    elif backend == "nccl":
        A = torch.empty(M * K, dtype=torch.float16, device=dev)
    if backend == "nccl":
        A.zero_()
        if rank == 0:
            A.copy_(torch.from_numpy(np.ascontiguousarray(a_host.T)).reshape(-1))
    else:
        A = torch.from_numpy(np.ascontiguousarray(a_host.T)).to(dev) if rank == 0 else torch.zeros((K, M), dtype=torch.float16, device=dev)
    B = torch.from_numpy(np.ascontiguousarray(b_host.T)).to(dev) if ns else torch.zeros((1,), dtype=torch.float16, device=dev)
    Cm = torch.from_numpy(np.ascontiguousarray(c_host.T)).to(dev) if ns else torch.zeros((1,), dtype=torch.float32, device=dev)
    D = torch.full((max(ns, 1), M), -3.0, dtype=torch.float32, device=dev)
    for _ in range(2):  # twice: the second call finds A already resident everywhere
        if p2p:
            torch.cuda.synchronize()
            sg.run(alpha, B, beta, Cm, D, stream=torch.cuda.current_stream().cuda_stream, gated=fused)
            sg.wait(20000)  # host-side deadline: a peer that never writes ends in an error, not in a hang
        else:
            sg.run(alpha, A, B, beta, Cm, D)
        if backend == "nccl":
            torch.cuda.synchronize()
            code, block, _ = handle.device_status()
            assert code == 0, f"rank {rank}: device wait {code} ran out in block {block}"
    if rank != 0:
        assert np.array_equal(A.cpu().numpy().reshape(K, M).T, a_host), f"rank {rank}: A did not arrive intact"
    if ns:
        d = D.cpu().numpy().T
        oracle.assert_close(d, oracle.gemm_ref(False, False, alpha, a_host, b_host, beta, c_host), f"rank {rank} slab [{n0},{n0 + ns})")
    if p2p and ns:
        # the compute-only form (A already everywhere) must give the same slab
        D.fill_(-5.0)
        sg.run(alpha, B, beta, Cm, D, stream=torch.cuda.current_stream().cuda_stream, no_transfer=True)
        torch.cuda.synchronize()
        oracle.assert_close(D.cpu().numpy().T, oracle.gemm_ref(False, False, alpha, a_host, b_host, beta, c_host), f"rank {rank} compute-only")
    if backend != "nccl" and ns:
        want = [k1 - k0 for (k0, k1) in sg.panels]
        got = [k for (k, _) in handle.calls[:len(want)]]
        assert got == want, (got, want)
        caps = [c for (_, c) in handle.calls[:len(want)]]
        assert all(c == 140 for c in caps[:-1]) and caps[-1] == 0, caps  # SMs left to NCCL except on the last panel
    dist.barrier()
    if p2p:
        torch.cuda.synchronize()
        del A
        sg.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok: slab [{n0},{n0 + ns}) of N={N}", flush=True)


if __name__ == "__main__":
    main()
