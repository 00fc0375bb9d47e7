"""Expert-parallel SERVING on 2+ GPUs: an Engine over partitioned lanes, MoE layers expert-parallel, ranks in lock step."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_engine_serves_requests_spread_over_two_expert_parallel_ranks():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    worker = os.path.join(os.path.dirname(__file__), "ep_serve_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29547", worker],
                       capture_output=True, text=True, timeout=300, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "EP_SERVE_OK" in out and "EP_SERVE_FAIL" not in out, out[-3000:]
