"""Multi-GPU parity: launches one process per GPU (2, or 4 when present) and checks
column-sharded execution against the checker and against unsharded execution."""
import os
import subprocess
import sys

import pytest

from neon_b200 import runtime as rt

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_execution_matches_checker(world):
    if rt.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world),
           os.path.join(ROOT, "tests", "sharded_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "SHARDED-OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
