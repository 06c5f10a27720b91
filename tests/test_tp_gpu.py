"""Fused tensor-parallel kernels on 2 GPUs (skipped on boxes with fewer).  Runs with NVLS multicast and
with plain peer loads/stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("multicast", ["1", "0"])
def test_fused_tp_two_gpus(multicast):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, FB_TEST_MULTICAST=multicast)
    port = 29700 + os.getpid() % 100 + (1 if multicast == "1" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "tp_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_GPU_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
