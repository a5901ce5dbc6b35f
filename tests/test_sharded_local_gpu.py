"""The N-sharded GEMM's transfer schedule with 2 to 8 ranks on ONE GPU (the ranks are objects of one
process; see tests/sharded_local_worker.py), and its failure detection: a peer that never makes its
call ends in B200_PEER_TIMEOUT after the host-side deadline, with the context still usable.

Run as child processes: the child needs CUDA_DEVICE_MAX_CONNECTIONS before CUDA starts (every stream
of every rank must have a hardware queue of its own, or a stream that waits for a flag could sit in
front of the stream that writes it), and a child that went wrong is ended by the time-out here."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
WORKER = str(ROOT / "tests" / "sharded_local_worker.py")


def child(*args):
    env = dict(os.environ, CUDA_DEVICE_MAX_CONNECTIONS="32")
    return subprocess.run([sys.executable, WORKER, *map(str, args)], capture_output=True, text=True, timeout=180, env=env)


@pytest.mark.parametrize("world,shape,panels,lanes", [
    (2, (512, 1024, 768), 4, 1),
    (4, (256, 1024, 1160), 16, 2),     # two scatter and two gather lanes per rank, first launch over two panels
    (3, (256, 1000, 200), 3, 1),      # uneven slabs (1000 columns over 3 ranks), K not a multiple of panels x 64
    (4, (384, 1300, 1096), 16, 1),    # 16 panels -> 4 launch groups; the last rank's slab is ragged
    (5, (128, 600, 520), 5, 1),       # more ranks than column tiles: two ranks own nothing but still forward A
    (8, (128, 2304, 1160), 16, 1),    # the 8-rank schedule: 7 sub-blocks per panel, 16 panels, 4 launches
])
def test_ranks_on_one_gpu(lib, world, shape, panels, lanes):
    assert world * (1 + 2 * lanes) + 4 <= 32  # compute, scatter and gather streams per rank, each on a hardware queue of its own
    r = child("run", world, *shape, panels, lanes)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok: slab") == world


def test_peer_that_never_calls_ends_in_an_error_not_a_hang(lib):
    r = child("timeout")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "timeout ok" in r.stdout
