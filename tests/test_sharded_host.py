"""Host-side logic of the N-sharded GEMM, no GPU needed: the layout arithmetic of the C ABI
(b200_sharded_layout), the thin ctypes caller against a fake library, and the NCCL-broadcast variant
on gloo ranks on the CPU with the CPU oracle standing in for the GEMM call."""
import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import pytest

from cudanative_jl_b200 import B200Error, _lib
from cudanative_jl_b200 import gemm as gemm_mod
from cudanative_jl_b200.gemm import ShardedGemm, ShardLayout
from cudanative_jl_b200.nccl_broadcast import panel_bounds, slab_bounds

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("n,world", [(32768, 8), (32768, 1), (1000, 3), (256, 4), (100, 8), (0, 2), (8192, 5), (3000, 7)])
def test_slabs_partition_the_columns(lib, n, world):
    bounds = ShardLayout(world, n, 64, 4).slabs
    assert bounds == [slab_bounds(n, world, r) for r in range(world)]  # the C side and the Python helper agree
    assert bounds[0][0] == 0 and bounds[-1][1] == n
    for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
        assert a1 == b0 and a0 <= a1
    for (n0, n1) in bounds:
        assert n0 % 256 == 0 or n0 == n  # slabs start on tile boundaries
    sizes = [n1 - n0 for (n0, n1) in bounds]
    assert max(sizes) - min(sizes) <= 256 + 255  # as even as whole tiles allow


@pytest.mark.parametrize("k,panels", [(16384, 8), (16384, 1), (1000, 4), (64, 8), (130, 3), (1, 2), (16384, 32), (16384, 99)])
def test_panels_partition_k(lib, k, panels):
    b = ShardLayout(2, 512, k, panels).panels
    assert b[0][0] == 0 and b[-1][1] == k and len(b) <= min(panels, 32)
    for (a0, a1), (b0, b1) in zip(b, b[1:]):
        assert a1 == b0 and a1 > a0
    assert all(k0 % 64 == 0 for (k0, _) in b)
    assert ShardLayout(1, 512, k, panels).panels == [(0, k)]  # one rank: nothing travels, one panel
    p = panel_bounds(k, panels)
    assert p[0][0] == 0 and p[-1][1] == k and all(k0 % 64 == 0 for (k0, _) in p)


@pytest.mark.parametrize("n", [1, 2, 3, 8, 16, 32])
def test_launch_groups_cover_the_panels_and_grow(lib, n):
    lay = ShardLayout(2, 512, 64 * n, n)
    assert len(lay.panels) == n
    g = lay.groups
    assert g[0][0] == 0 and g[-1][1] == n
    assert all(a1 == b0 and a1 > a0 for (a0, a1), (b0, _) in zip(g, g[1:]))
    sizes = [b - a for (a, b) in g]
    assert sizes[0] == 1 and max(sizes) <= max(1, n // 4) + 1  # no launch waits for more than about a quarter of A
    assert all(y >= x for x, y in zip(sizes, sizes[1:-1]))       # growing, up to a merged or short last launch
    assert [b - a for (a, b) in ShardLayout(8, 32768, 16384, 16).groups] == [1, 2, 2, 3, 4, 4]


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("k,panels", [(16384, 16), (200, 4), (1000, 3)])
def test_transfer_subblocks_tile_every_panel(lib, world, k, panels):
    """Scatter / all-gather ownership: within each panel the receiving ranks' column ranges are
    disjoint, contiguous and cover the panel; rank 0 owns nothing (it only sends)."""
    lay = ShardLayout(world, 4096, k, panels)
    assert len(lay.sub_cols) == len(lay.panels)
    for (k0, k1), row in zip(lay.panels, lay.sub_cols):
        assert len(row) == world and row[0] == (k0, k0)
        edge = k0
        for (c0, c1) in row[1:]:
            assert c0 == edge and c1 >= c0 and (c0 - k0) % 8 == 0  # 16-byte columns of Float16 rows
            edge = c1
        assert edge == k1


def test_layout_refuses_bad_arguments(lib):
    for (world, n, k) in [(0, 10, 64), (65, 10, 64), (2, -1, 64), (2, 10, 0)]:
        with pytest.raises(B200Error) as e:
            ShardLayout(world, n, k, 4)
        assert e.value.status == _lib.INVALID_ARG


class FakeShardedLib:
    """Stands in for libb200wmma.so behind ShardedGemm: records what crosses the C ABI."""

    def __init__(self, rank, fail_wait=0):
        self.rank, self.calls, self.fail_wait = rank, [], fail_wait

    def b200_sharded_create(self, out, h, rank, world, M, N, K, panels):
        self.calls.append(("create", rank, world, M, N, K, panels))
        C.cast(out, C.POINTER(C.c_void_p))[0] = 0x1000 + rank
        return 0

    def b200_sharded_info(self, s, n0, n1, a, f, n_p, n_g):
        C.cast(n0, C.POINTER(C.c_int64))[0] = 256 * self.rank
        C.cast(n1, C.POINTER(C.c_int64))[0] = 256 * (self.rank + 1)
        C.cast(a, C.POINTER(C.c_void_p))[0] = 0xA000
        C.cast(f, C.POINTER(C.c_void_p))[0] = 0xF000
        C.cast(n_p, C.POINTER(C.c_int))[0] = 4
        C.cast(n_g, C.POINTER(C.c_int))[0] = 2
        return 0

    def b200_sharded_ipc_blob(self, s, blob):
        C.memmove(blob, bytes([self.rank + 1]) * 128, 128)
        return 0

    def b200_sharded_attach(self, s, blobs):
        self.calls.append(("attach", bytes(blobs)))
        return 0

    def b200_sharded_run(self, s, stream, alpha, b, ldb, beta, c, ldc, d, ldd, flags):
        self.calls.append(("run", alpha, b, ldb, beta, c, ldc, d, ldd, flags))
        return 0

    def b200_sharded_wait(self, s, timeout_ms):
        self.calls.append(("wait", timeout_ms))
        return self.fail_wait

    def b200_sharded_destroy(self, s):
        self.calls.append(("destroy",))
        return 0

    def b200_status_string(self, status):
        return {_lib.PEER_TIMEOUT: b"B200_PEER_TIMEOUT"}.get(status, b"B200_?")

    def b200_last_error(self):
        return b"sharded_wait: no word from a peer within 50 ms"


class FakeHandle:
    _h = C.c_void_p(0x42)
    device = 0


def test_thin_caller_crosses_the_abi_as_declared(monkeypatch):
    """create -> info -> ipc_blob -> (caller's exchange) -> attach, then run / wait / destroy with the
    arguments include/b200wmma.h declares; a peer time-out surfaces as B200Error(PEER_TIMEOUT)."""
    fake = FakeShardedLib(rank=1, fail_wait=_lib.PEER_TIMEOUT)
    monkeypatch.setattr(_lib, "lib", lambda: fake)
    seen = []

    def exchange(blob):
        seen.append(blob)
        return [bytes([1]) * 128, blob, bytes([3]) * 128]

    sg = ShardedGemm(FakeHandle(), 1024, 768, 512, rank=1, world=3, panels=4, exchange=exchange)
    assert seen == [bytes([2]) * 128]
    assert fake.calls[0] == ("create", 1, 3, 1024, 768, 512, 4)
    assert fake.calls[1] == ("attach", bytes([1]) * 128 + bytes([2]) * 128 + bytes([3]) * 128)
    assert (sg.n0, sg.n1, sg.slab_cols, sg.a_ptr, sg.n_panels, sg.n_groups) == (256, 512, 256, 0xA000, 4, 2)
    assert sg.a_view().__cuda_array_interface__["shape"] == (1024 * 512,)
    sg.run(1.0, 0xB000, 0.5, 0xC000, 0xD000, gated=True)
    assert fake.calls[-1] == ("run", 1.0, 0xB000, 512, 0.5, 0xC000, 1024, 0xD000, 1024, _lib.SHARDED_GATED)
    sg.run(2.0, 0xB000, 0.0, None, 0xD000, no_transfer=True, ldb=600, ldd=1100)
    assert fake.calls[-1] == ("run", 2.0, 0xB000, 600, 0.0, None, 1024, 0xD000, 1100, _lib.SHARDED_NO_TRANSFER)
    with pytest.raises(B200Error) as e:
        sg.wait(50)
    assert e.value.status == _lib.PEER_TIMEOUT and "no word from a peer" in str(e.value)
    sg.close()
    assert fake.calls[-1] == ("destroy",)
    with pytest.raises(ValueError):
        ShardedGemm(FakeHandle(), 1024, 768, 512, rank=1, world=3, exchange=lambda blob: [blob])


@pytest.mark.parametrize("world,shape", [(2, (96, 640, 200)), (3, (64, 512, 130))])
def test_broadcast_flow_on_gloo(world, shape):
    """world ranks on the CPU: broadcast of A in K panels (gloo), per-panel accumulate calls with the
    right pointer offsets, the SM reservation on all but the last panel, D slabs against the oracle."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + world), str(ROOT / "tests" / "sharded_worker.py"), "gloo", *map(str, shape), "3"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok: slab") == world


def _fake_ranks(mode, world=2):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29540 + world + (7 if mode == "silent" else 0)), str(ROOT / "tests" / "sharded_fake_worker.py"), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)


@pytest.mark.parametrize("world", [2, 3])
def test_thin_caller_from_separate_processes_on_gloo(world):
    """ShardedGemm in `world` real processes against a Python stand-in for the library: blobs exchanged in
    rank order, slab pointers and leading dimensions as declared, every slab against the oracle."""
    r = _fake_ranks("run", world)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok: slab") == world


def test_a_rank_that_never_calls_is_reported_on_the_host():
    """Failure detection made on the host: rank 1 of 2 never makes its call; rank 0's wait comes back with
    B200_PEER_TIMEOUT after its deadline and names the silent peer.  No GPU, nothing hangs."""
    r = _fake_ranks("silent")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 saw PEER_TIMEOUT" in r.stdout and "rank 1 stayed silent" in r.stdout
