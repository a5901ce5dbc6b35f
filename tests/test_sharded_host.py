"""Host-side logic of the N-sharded GEMM: slab / panel arithmetic, and the whole ShardedGemm.run
flow on two gloo ranks on the CPU with the CPU oracle standing in for the GEMM call."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from cudanative_jl_b200.gemm import launch_groups, panel_bounds, slab_bounds, subblock_cols

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("n,world", [(32768, 8), (32768, 1), (1000, 3), (256, 4), (100, 8), (0, 2), (8192, 5)])
def test_slabs_partition_the_columns(n, world):
    bounds = [slab_bounds(n, world, r) for r in range(world)]
    assert bounds[0][0] == 0 and bounds[-1][1] == n
    for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
        assert a1 == b0 and a0 <= a1
    for (n0, n1) in bounds:
        assert n0 % 256 == 0 or n0 == n  # slabs start on tile boundaries
    sizes = [n1 - n0 for (n0, n1) in bounds]
    assert max(sizes) - min(sizes) <= 256 + 255  # as even as whole tiles allow


@pytest.mark.parametrize("k,panels", [(16384, 8), (16384, 1), (1000, 4), (64, 8), (130, 3), (1, 2)])
def test_panels_partition_k(k, panels):
    b = panel_bounds(k, panels)
    assert b[0][0] == 0 and b[-1][1] == k and len(b) <= panels
    for (a0, a1), (b0, b1) in zip(b, b[1:]):
        assert a1 == b0 and a1 > a0
    assert all(k0 % 64 == 0 for (k0, _) in b)


@pytest.mark.parametrize("n", [1, 2, 3, 8, 16, 32])
def test_launch_groups_cover_the_panels_and_grow(n):
    g = launch_groups(n)
    assert g[0][0] == 0 and g[-1][1] == n
    assert all(a1 == b0 and a1 > a0 for (a0, a1), (b0, _) in zip(g, g[1:]))
    sizes = [b - a for (a, b) in g]
    assert sizes[0] == 1 and sizes == sorted(sizes) and len(g) <= 5


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("k,panel_k", [(16384, 1024), (200, 64), (1000, 320)])
def test_transfer_subblocks_tile_every_panel(world, k, panel_k):
    """Scatter / all-gather ownership: within each panel the receiving ranks' column ranges are
    disjoint, contiguous and cover the panel; rank 0 owns nothing (it only sends)."""
    panels = [(k0, min(k, k0 + panel_k)) for k0 in range(0, k, panel_k)]
    sub = subblock_cols(panels, world)
    assert len(sub) == len(panels)
    for (k0, k1), row in zip(panels, sub):
        assert len(row) == world and row[0] == (k0, k0)
        edge = k0
        for (c0, c1) in row[1:]:
            assert c0 == edge and c1 >= c0
            edge = c1
        assert edge == k1


@pytest.mark.parametrize("world,shape", [(2, (96, 640, 200)), (3, (64, 512, 130))])
def test_sharded_flow_on_gloo(world, shape):
    """world ranks on the CPU: broadcast of A in K panels (gloo), per-panel accumulate calls with the
    right pointer offsets, the SM reservation on all but the last panel, D slabs against the oracle."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + world), str(ROOT / "tests" / "sharded_worker.py"), "gloo", *map(str, shape), "3"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok: slab") == world
