"""The fused exchange of the head-sharded decode on real peers: needs two GPUs with peer access (one process
per GPU, NCCL for the plumbing, symmetric memory for the gathered buffers).  Skipped on a single GPU, where
tests/test_peer_gpu.py covers the same kernels with local memory standing in for the peers'."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_stores_and_arrive_and_wait_equal_an_all_gather_on_two_gpus():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "peer_gather_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", "29541", worker],
        capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "PEER_GATHER_OK" in proc.stdout
