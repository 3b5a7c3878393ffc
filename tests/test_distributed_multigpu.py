"""Native NVLink collectives and the fused DDP engine on 2+ real GPUs (one process per GPU)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(600)
def test_native_collectives_and_fused_ddp(tmp_path):
    n = min(torch.cuda.device_count(), 8)
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_mgpu_worker.py")
    env = dict(os.environ, FERRUM_DEVICE_WAIT_S="20")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(_port()), worker, str(tmp_path)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=540)
    tail = (r.stdout + r.stderr)[-4000:]
    assert r.returncode == 0, tail
    for rank in range(n):
        res = (tmp_path / f"rank{rank}.txt").read_text()
        assert res == "PASS", f"rank {rank}: {res}\n{tail}"
