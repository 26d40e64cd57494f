"""GPU, two devices: tensor-parallel results against the un-sharded run of the SAME weights (see
tests/tp_unsharded_worker.py).  Skipped on a single-GPU machine.  NVLS is switched off for the run: the ranks are
short-lived child processes."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tensor_parallel_matches_the_unsharded_model():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29541", os.path.join(root, "tests", "tp_unsharded_worker.py")],
                       capture_output=True, text=True, timeout=900, env=env, cwd=root)
    assert r.returncode == 0 and "TP_VS_SINGLE world=2 OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
