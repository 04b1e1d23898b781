"""ChunkTensors spanning several GPUs (cudaIpc peer mappings + shared host tail).
Needs at least two GPUs in the box; skipped otherwise."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "multi_rank_worker.py")]
    return subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_chunktensor_over_several_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    r = _run(world, 29500 + world)
    assert r.returncode == 0, r.stdout[-4000:]
    for rank in range(world):
        assert "RANK %d OK" % rank in r.stdout, r.stdout[-4000:]
