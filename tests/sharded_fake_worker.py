"""One gloo rank of the thin ``ShardedGemm`` caller against a stand-in for libb200wmma.so (launched by
test_sharded_host.py; no GPU).  The stand-in implements the b200_sharded_* entry points in Python: slab
bounds come from the real b200_sharded_layout (pure host arithmetic), "the transfer" is a gloo broadcast
of A, "the GEMM" is the CPU oracle on the memory the addresses point to, and "a peer wrote its flags" is a
key in the process group's store.  What is under test is what crosses the C ABI from real, separate
processes: the blob exchange in rank order, the slab pointers, the flags, and that a rank whose peer never
makes its call gets B200_PEER_TIMEOUT from ``wait`` instead of waiting for ever.

    sharded_fake_worker.py run      every rank makes its call: slabs against the oracle
    sharded_fake_worker.py silent   rank 1 never makes its call: rank 0 must see PEER_TIMEOUT
"""
import ctypes as C
import datetime
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
oracle = entry.load_oracle()
from cudanative_jl_b200 import B200Error, _lib, rng  # noqa: E402
from cudanative_jl_b200.gemm import ShardedGemm, ShardLayout  # noqa: E402

REAL = _lib.lib()


class FakeHandle:
    _h = C.c_void_p(0x42)
    device = 0


class FakeShardedLib:
    def __init__(self, rank, world, store):
        self.rank, self.world, self.store = rank, world, store
        self.epoch = 0
        self.error = b""

    def b200_sharded_create(self, out, h, rank, world, M, N, K, panels):
        assert (rank, world) == (self.rank, self.world)
        self.M, self.N, self.K = M, N, K
        self.lay = ShardLayout(world, N, K, panels)
        self.a = torch.zeros(M * K, dtype=torch.float16)  # "the buffer the library owns"
        C.cast(out, C.POINTER(C.c_void_p))[0] = 0x5000 + rank
        return _lib.OK

    def b200_sharded_info(self, s, n0, n1, a, f, n_p, n_g):
        lo, hi = self.lay.slabs[self.rank]
        for ptr, ty, val in ((n0, C.c_int64, lo), (n1, C.c_int64, hi), (a, C.c_void_p, self.a.data_ptr()), (f, C.c_void_p, 0xF000),
                             (n_p, C.c_int, len(self.lay.panels)), (n_g, C.c_int, len(self.lay.groups))):
            if ptr:
                C.cast(ptr, C.POINTER(ty))[0] = val
        return _lib.OK

    def b200_sharded_ipc_blob(self, s, blob):
        C.memmove(blob, bytes([self.rank + 1]) * 128, 128)
        return _lib.OK

    def b200_sharded_attach(self, s, blobs):
        assert bytes(blobs) == b"".join(bytes([r + 1]) * 128 for r in range(self.world)), "blobs not in rank order"
        return _lib.OK

    def b200_sharded_run(self, s, stream, alpha, b, ldb, beta, c, ldc, d, ldd, flags):
        self.epoch += 1
        self.store.set(f"done/{self.epoch}/{self.rank}", "1")  # what the 'done' flag words are across GPUs
        self.pending = (alpha, b, ldb, beta, c, ldc, d, ldd)
        return _lib.OK

    def b200_sharded_wait(self, s, timeout_ms):
        deadline = time.monotonic() + timeout_ms / 1e3
        for g in range(self.world):  # every peer must have made the call
            while not self.store.check([f"done/{self.epoch}/{g}"]):  # check() does not block, get() would
                if time.monotonic() > deadline:
                    self.error = f"sharded_wait: no word from a peer within {timeout_ms} ms; silent peers: {g}".encode()
                    return _lib.PEER_TIMEOUT
                time.sleep(0.01)
        dist.broadcast(self.a, src=0)  # "the transfer"
        alpha, b, ldb, beta, c, ldc, d, ldd = self.pending
        lo, hi = self.lay.slabs[self.rank]
        ns, M, K = hi - lo, self.M, self.K
        if ns:
            def view(addr, rows, cols, ld, ctype, dtype):
                return np.frombuffer((ctype * (ld * cols)).from_address(addr), dtype=dtype).reshape((ld, cols), order="F")[:rows]
            a = self.a.numpy().view(np.float16).reshape((M, K), order="F")
            view(d, M, ns, ldd, C.c_float, np.float32)[:] = oracle.gemm_ref(
                False, False, alpha, a, view(b, K, ns, ldb, C.c_uint16, np.float16), beta,
                view(c, M, ns, ldc, C.c_float, np.float32).copy() if beta != 0.0 else None)
        return _lib.OK

    def b200_sharded_destroy(self, s):
        return _lib.OK

    def b200_sharded_layout(self, *args):
        return REAL.b200_sharded_layout(*args)

    def b200_status_string(self, status):
        return REAL.b200_status_string(status)

    def b200_last_error(self):
        return self.error


def main():
    mode = sys.argv[1]
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    rank, world = dist.get_rank(), dist.get_world_size()
    store = dist.distributed_c10d._get_default_store()
    fake = FakeShardedLib(rank, world, store)
    _lib.lib = lambda: fake
    M, N, K = 96, 640, 200

    def exchange(blob):
        blobs = [None] * world
        dist.all_gather_object(blobs, blob)
        return blobs

    sg = ShardedGemm(FakeHandle(), M, N, K, rank=rank, world=world, panels=3, exchange=exchange)
    assert (sg.n0, sg.n1) == ShardLayout(world, N, K, 3).slabs[rank]
    a_host = rng.matrix(4, 0, M, K, rng.NORMAL, K ** -0.5, np.float16)
    ns = sg.slab_cols
    b_host = rng.window(4, 1, K, 0, K, sg.n0, sg.n1, rng.NORMAL, K ** -0.5, np.float16)
    c_host = rng.window(4, 2, M, 0, M, sg.n0, sg.n1, rng.NORMAL, 1.0, np.float32)
    if rank == 0:
        C.memmove(sg.a_ptr, a_host.ctypes.data, a_host.nbytes)
    D = np.full((M, max(ns, 1)), np.float32(-3.0), order="F")
    if mode == "silent" and rank == 1:
        time.sleep(1.0)  # this rank never makes its call; it only stays around until rank 0 has noticed
        print("rank 1 stayed silent", flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    sg.run(1.0, b_host.ctypes.data, 1.0, c_host.ctypes.data, D.ctypes.data)
    if mode == "silent":
        try:
            sg.wait(300)
            raise SystemExit("the wait returned although rank 1 never made its call")
        except B200Error as e:
            assert e.status == _lib.PEER_TIMEOUT and "silent peers: 1" in str(e), e
        print("rank 0 saw PEER_TIMEOUT", flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    sg.wait(20000)
    if ns:
        oracle.assert_close(D[:, :ns], oracle.gemm_ref(False, False, 1.0, a_host, b_host, 1.0, c_host), f"rank {rank}")
    dist.barrier()
    sg.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok: slab [{sg.n0},{sg.n1})", flush=True)


if __name__ == "__main__":
    main()
