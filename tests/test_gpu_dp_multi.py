"""Data-parallel training and column-sharded inference on 2 real GPUs (skipped on a box with one):
N-rank parameters against a single-GPU run of the same steps, replicas bit-identical, the loss
all-reduced, the sharded INT8 pipeline bit-equal to the unsharded oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_two_gpu_ranks():
    from vtl_b200 import capi
    capi.load()
    if capi.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(HERE, "dp_gpu_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    assert p.stdout.count(" ok") == 2
