"""Tensor-parallel run of the fused kernel on 2+ GPUs of one box: in-kernel NVLS AllReduce
(multimem.ld_reduce / multimem.st), cross-rank readiness counters and the exit barrier,
many layers on one workspace with no host reset.  The body is tests/_mgpu_worker.py, run
as one process per GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_layers(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(__file__), "_mgpu_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), worker]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    tail = (res.stdout + res.stderr)[-4000:]
    assert res.returncode == 0, tail
    assert res.stdout.count("ALL OK") == world, tail
