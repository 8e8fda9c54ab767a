"""Launches the multi-GPU kernel checks when at least two GPUs are visible."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_fused_collectives_two_ranks():
    from cornserve.services.process import free_port

    script = os.path.join(os.path.dirname(__file__), "multigpu_fused.py")
    n = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), script]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "MULTIGPU_FUSED_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
