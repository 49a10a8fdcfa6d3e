"""The sharded layer over NCCL on 2+ GPUs of one box (skipped on a single-GPU box)."""
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_layer_nccl(cuda, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = Path(__file__).with_name("sharded_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(worker)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                         env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    print(res.stdout[-3000:])
    assert res.returncode == 0 and "SHARDED_PASS" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
