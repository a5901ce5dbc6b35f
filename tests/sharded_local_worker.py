"""Several ranks of the N-sharded GEMM inside ONE process on ONE GPU (launched by
test_sharded_local_gpu.py): every rank is a b200_sharded object of its own with its own handle and
stream, the peers are attached by address (b200_sharded_attach_local).  The whole transfer schedule
-- scatter, staggered all-gather, epoch flags, launch groups -- then runs exactly as it does across
GPUs, only that every copy stays on this device.  No kernel ever waits for another one: the GEMM
launches sit behind stream-level waits, which is what makes this safe on a single GPU (the gated
single-launch form polls from inside a kernel and is therefore not run here).

    sharded_local_worker.py run <world> <M> <N> <K> <panels> [lanes]   every rank's slab and A against the oracle
    sharded_local_worker.py timeout                              a peer that never calls: deadline, error, context alive
"""
import ctypes as C
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
oracle = entry.load_oracle()
from cudanative_jl_b200 import B200Error, _lib, rng  # noqa: E402
from cudanative_jl_b200.array import Array, CuArray, CuHostArray  # noqa: E402
from cudanative_jl_b200.gemm import Handle, ShardedGemm  # noqa: E402

L = _lib.lib()


def new_stream():
    s = C.c_void_p()
    _lib.check(L.b200_stream_create(C.byref(s)), "stream_create")
    return s


def upload(dst_ptr, host):
    _lib.check(L.b200_memcpy_h2d(dst_ptr, host.ctypes.data, host.nbytes, None), "h2d")
    _lib.check(L.b200_stream_sync(None), "sync")


def download(src_ptr, shape, dtype):
    out = np.empty(shape, dtype=dtype, order="F")
    _lib.check(L.b200_memcpy_d2h(out.ctypes.data, src_ptr, out.nbytes, None), "d2h")
    _lib.check(L.b200_stream_sync(None), "sync")
    return out


def make_ranks(world, M, N, K, panels, lanes=1):
    handles = [Handle(0) for _ in range(world)]
    for h in handles:
        h.set_option(_lib.OPT_WAIT_BUDGET_NS, 500_000_000)
        if os.environ.get("B200_TEST_PDL") is not None:
            h.set_option(_lib.OPT_PDL, int(os.environ["B200_TEST_PDL"]))
    objs = [ShardedGemm(handles[r], M, N, K, rank=r, world=world, panels=panels) for r in range(world)]
    for o in objs:
        o.attach_local(objs)
        if lanes > 1:  # copies to different receivers side by side, and a two-panel first launch
            o.set_option(_lib.SHARDED_OPT_SCATTER_LANES, lanes)
            o.set_option(_lib.SHARDED_OPT_GATHER_LANES, lanes)
            o.set_option(_lib.SHARDED_OPT_FIRST_GROUP, 2)
    return handles, objs


def run(world, M, N, K, panels, lanes=1):
    seed, alpha, beta = 4, 1.0, 1.0
    handles, objs = make_ranks(world, M, N, K, panels, lanes)
    streams = [new_stream() for _ in range(world)]
    a_host = rng.matrix(seed, 0, M, K, rng.NORMAL, K ** -0.5, np.float16)
    upload(objs[0].a_ptr, a_host)
    for o in objs[1:]:
        _lib.check(L.b200_memset(o.a_ptr, 0, 2 * M * K, None), "memset")
    _lib.check(L.b200_stream_sync(None), "sync")
    slabs = []
    for o in objs:
        ns = o.slab_cols
        b = rng.window(seed, 1, K, 0, K, o.n0, o.n1, rng.NORMAL, K ** -0.5, np.float16)
        c = rng.window(seed, 2, M, 0, M, o.n0, o.n1, rng.NORMAL, 1.0, np.float32)
        slabs.append((b, c, CuArray(b) if ns else None, CuArray(c) if ns else None,
                      CuArray(np.full((M, max(ns, 1)), np.float32(-3.0), dtype=np.float32, order="F"))))
    for rep in range(2):  # the second product finds A resident everywhere and must still wait for the hand-shake
        for r, o in enumerate(objs):
            b, c, b_dev, c_dev, d_dev = slabs[r]
            o.run(alpha, b_dev.ptr if b_dev else 0, beta, c_dev.ptr if c_dev else 0, d_dev.ptr, stream=streams[r])
            print(f"product {rep}: rank {r} enqueued", flush=True)
        for r, o in enumerate(objs):
            o.wait(10000)
            print(f"product {rep}: rank {r} finished", flush=True)
    for r, o in enumerate(objs):
        if r:
            got = download(o.a_ptr, (M, K), np.float16)
            assert np.array_equal(got.view(np.uint16), a_host.view(np.uint16)), f"rank {r}: A did not arrive intact"
        b, c, b_dev, c_dev, d_dev = slabs[r]
        if o.slab_cols:
            oracle.assert_close(Array(d_dev)[:, :o.slab_cols], oracle.gemm_ref(False, False, alpha, a_host, b, beta, c),
                                f"rank {r} slab [{o.n0},{o.n1})")
        print(f"rank {r} ok: slab [{o.n0},{o.n1}) of N={N}, {o.n_panels} panels, {o.n_groups} launches", flush=True)
    for o in objs:
        o.close()


def timeout():
    """Rank 1 of 2 makes its call, rank 0 never does: rank 1's streams sit in stream-level waits (no kernel
    runs, nothing spins), the host-side deadline releases them and reports B200_PEER_TIMEOUT, and the
    context goes on working."""
    M, N, K = 256, 512, 256
    handles, objs = make_ranks(2, M, N, K, 2)
    o = objs[1]
    # argument checks come before anything is enqueued (a rank that gave up half-way would strand its peers)
    for bad in ([1], [1, 2], [0, 2]):
        try:
            o.set_groups(bad)
            raise SystemExit(f"launch groups {bad} were accepted for {o.n_panels} panels")
        except B200Error as e:
            assert e.status == _lib.INVALID_ARG, e
    o.set_groups([1, 1])
    try:
        o.run(1.0, 0x1000, 0.0, None, 0x2000, stream=None, ldb=K - 8)
        raise SystemExit("a leading dimension smaller than K was accepted")
    except B200Error as e:
        assert e.status == _lib.INVALID_ARG and "leading dimension" in str(e), e
    s = new_stream()
    b = rng.matrix(9, 1, K, o.slab_cols, rng.NORMAL, 1.0, np.float16)
    b_dev = CuArray(b)
    d_dev = CuHostArray(np.float32, shape=(M, o.slab_cols))
    o.run(1.0, b_dev.ptr, 0.0, None, d_dev.ptr, stream=s)
    try:
        o.wait(300)
        raise SystemExit("the wait returned although rank 0 never made its call")
    except B200Error as e:
        assert e.status == _lib.PEER_TIMEOUT, e
        assert "no word from a peer within 300 ms" in str(e), e
    try:
        o.run(1.0, b_dev.ptr, 0.0, None, d_dev.ptr, stream=s)
        raise SystemExit("a poisoned object accepted another product")
    except B200Error as e:
        assert e.status == _lib.PEER_TIMEOUT, e
    # the context is alive: an ordinary product on the same handle is right
    a = rng.matrix(9, 0, M, K, rng.NORMAL, K ** -0.5, np.float16)
    a_dev = CuArray(a)
    handles[1].gemm(False, False, M, o.slab_cols, K, 1.0, a_dev, M, b_dev, K, 0.0, None, M, d_dev, M, stream=s)
    _lib.check(L.b200_stream_sync(s), "sync")
    assert handles[1].device_status()[0] == 0
    oracle.assert_close(Array(d_dev), oracle.gemm_ref(False, False, 1.0, a, b, 0.0, None), "GEMM after the time-out")
    for x in objs:
        x.close()
    print("timeout ok", flush=True)


if __name__ == "__main__":
    if sys.argv[1] == "run":
        run(*(int(x) for x in sys.argv[2:8]))
    else:
        timeout()
