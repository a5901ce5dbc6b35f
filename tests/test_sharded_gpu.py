"""The N-sharded GEMM on real GPUs (one rank per GPU, NCCL broadcast of A over NVLink)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def gpu_count(lib):
    return lib.b200_device_count()


@pytest.mark.parametrize("transport", ["nccl", "p2p", "p2p-fused"])
@pytest.mark.parametrize("shape,panels", [((1024, 2048, 1536), 4), ((640, 1000, 200), 3)])
def test_sharded_gemm_two_gpus(lib, shape, panels, transport):
    if gpu_count(lib) < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", str(ROOT / "tests" / "sharded_worker.py"), "nccl", *map(str, shape), str(panels), transport.split("-")[0], "fused" if transport.endswith("fused") else "launches"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok: slab") == 2
