"""Tensor-parallel decoder on real GPUs (NCCL + the peer-buffer all-reduce): world sizes 2, 4 and 8."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# two_step: the all-reduce variant used from 8 ranks on (a row is summed by the rank that owns it and
# sent out finished), forced here on fewer ranks as well so that it is exercised wherever 2 GPUs exist
@pytest.mark.parametrize("world,two_step", [(2, False), (2, True), (4, False), (4, True), (8, True)])
def test_tensor_parallel_decoder_matches_oracle(world, two_step):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", LLMQRT_ALLREDUCE_TWO_STEP="1" if two_step else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + 2 * world + int(two_step)),
           os.path.join(ROOT, "tests", "tp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-9000:]
