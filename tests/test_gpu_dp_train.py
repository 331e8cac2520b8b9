"""Data-parallel training on real GPUs equals single-device training: 100 SGD
steps of one global batch of 8192 sharded over every power-of-two number of
GPUs the box has (2, 4, 8), against the CPU oracle on the whole batch (loss
curve within 1e-3, weights within 5e-4, replicas bit-identical).  One
process per GPU; skipped on a single-GPU box."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def _worlds():
    import torch
    n = torch.cuda.device_count()
    return [w for w in (2, 4, 8) if w <= n]


@pytest.mark.parametrize("mode", ["peer", "nccl"])
def test_sharded_training_follows_the_oracle(mode):
    worlds = _worlds()
    if not worlds:
        pytest.skip("needs at least 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    for i, world in enumerate(worlds):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
               "--master-port", str(29651 + i + (10 if mode == "nccl" else 0)), os.path.join(here, "dp_train_worker.py"), mode]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        assert "DP_TRAIN_OK" in r.stdout, "world %d: " % world + r.stdout[-2000:] + r.stderr[-2000:]
