"""Tensor-parallel generation on 2, 4 and 8 GPUs: fused peer-memory collectives vs NCCL vs single GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(world: int, port: int) -> None:
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    worker = os.path.join(os.path.dirname(__file__), "tp_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), worker],
                       capture_output=True, text=True, timeout=600, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "TP_OK" in out and "TP_FAIL" not in out, out[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_matches_single_gpu():
    _run(2, 29533)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp4_matches_single_gpu():
    _run(4, 29534)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_tp8_matches_single_gpu():
    _run(8, 29535)
