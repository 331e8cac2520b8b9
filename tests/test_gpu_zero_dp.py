"""Optimizer-sharded data-parallel step (reduce-scatter, Adam on owned slices,
all-gather of the bf16 weights) equals the plain data-parallel step; needs two
GPUs (one process per GPU), skipped otherwise."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_sharded_adam_matches_replicated_adam():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(here, "zero_dp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ZERO_DP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
