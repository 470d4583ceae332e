"""world_size-2 gloo runs on CPU of the host-side logic behind the multi-GPU paths."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("case,port", [("plumbing", 29601), ("dp_gradients", 29602), ("dp_accumulate", 29604),
                                       ("int8_column_shards", 29603)])
def test_two_cpu_ranks(case, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "dist_cpu_worker.py"), case]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    assert p.stdout.count(" ok") == 2
