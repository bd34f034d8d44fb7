"""Expert-parallel parity on 2+ GPUs of one box: torchrun launches tests/ep_parity_worker.py, one rank per GPU.
Skipped on single-GPU machines."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), os.path.join(ROOT, "tests",
                                                                                              "ep_parity_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("ep parity ok") == 6   # 3 cases x 2 transports
    assert "ep overflow reported ok" in res.stdout


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_single_gpu(world):
    import __graft_entry__
    __graft_entry__.build()
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    _run(world)
