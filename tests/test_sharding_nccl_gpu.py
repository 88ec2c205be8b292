"""The sharded paths on NCCL: two ranks on two GPUs run the sharded Wavefunction Embedding and geometric attention
(by (batch, head) pairs and by query blocks) and compare the gathered / reduced results with the unsharded calls.
Skipped with fewer than two visible GPUs."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_sharded_calls_on_two_gpus_match_one_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "nccl_sharded_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "nccl sharded ok 2" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
