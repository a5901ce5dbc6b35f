"""The N-sharded GEMM on real GPUs, one rank per GPU: the b200_sharded_* entry points (copy engines
over NVLink, `p2p`), their gated single-launch form (`p2p-fused`) and the NCCL-broadcast variant."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def gpu_count(lib):
    return lib.b200_device_count()


def run_ranks(world, shape, panels, transport):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29611 + world), str(ROOT / "tests" / "sharded_worker.py"), "nccl", *map(str, shape), str(panels),
           transport.split("-")[0], "fused" if transport.endswith("fused") else "launches"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok: slab") == world


@pytest.mark.parametrize("transport", ["nccl", "p2p", "p2p-fused"])
@pytest.mark.parametrize("shape,panels", [((1024, 2048, 1536), 4), ((640, 1000, 200), 3)])
def test_sharded_gemm_two_gpus(lib, shape, panels, transport):
    if gpu_count(lib) < 2:
        pytest.skip("needs two GPUs")
    run_ranks(2, shape, panels, transport)


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("transport", ["p2p", "p2p-fused", "nccl"])
@pytest.mark.parametrize("shape,panels", [((1024, 4096 + 1000, 2048 + 200), 16), ((384, 1300, 1096), 5)])
def test_sharded_gemm_four_and_eight_gpus(lib, world, shape, panels, transport):
    """Uneven slabs (N is not a multiple of world x 256, the last slab is ragged) and a K that is not a
    multiple of panels x 64: the sub-block arithmetic of the scatter / all-gather differs per panel."""
    if gpu_count(lib) < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks(world, shape, panels, transport)


def test_handle_is_refused_on_another_current_device(lib, pkg):
    """A handle's status word and scratch live on its device, a launch goes to the calling thread's current
    device: the GEMM entry points refuse the call when the two differ instead of launching on the wrong GPU."""
    if gpu_count(lib) < 2:
        pytest.skip("needs two GPUs")
    import numpy as np

    from cudanative_jl_b200 import B200Error
    from cudanative_jl_b200.array import CuArray
    from cudanative_jl_b200.gemm import Handle

    h0 = Handle(0)
    buf = CuArray(np.zeros((64, 64), dtype=np.float16, order="F"))
    out = CuArray(np.zeros((64, 64), dtype=np.float32, order="F"))
    h1 = Handle(1)  # like device!(1): device 1 is now the calling thread's current device
    try:
        with pytest.raises(B200Error, match="belongs to device 0 but the calling thread's current device is 1"):
            h0.gemm(False, False, 64, 64, 64, 1.0, buf, 64, buf, 64, 0.0, None, 64, out, 64)
    finally:
        h1.close()
        Handle(0).close()  # back to device 0 for the tests that follow
        h0.close()
