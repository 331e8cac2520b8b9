"""The C++ host side (zigrad_b200/host: opspec structs, CudaDevice, MlpTrainer)
drives the same C ABI as the Python one: MLP training steps run by the C++
program, eagerly and from a captured graph, against the CPU oracle."""
import os
import struct
import subprocess

import numpy as np
import pytest

import oracle
from zigrad_b200 import build as zbuild
from zigrad_b200.mlp import kaiming_uniform

from .test_gpu_ops import rel_err


def test_cpp_host_example_builds_and_links():
    exe = zbuild.build_host_example()
    assert os.path.exists(exe) and os.access(exe, os.X_OK)


@pytest.mark.gpu
@pytest.mark.parametrize("use_graph,steps", [(0, 1), (0, 5), (1, 5)])
@pytest.mark.parametrize("dims,B", [([784, 128, 64, 10], 256), ([20, 16, 8, 5], 33)])
def test_cpp_mlp_steps_match_the_oracle(tmp_path, dims, B, use_graph, steps):
    """One step: every parameter within 1e-5 of the CPU path.  Five steps: the
    per-step loss within 1e-3 (the bound the hot path is held to over 100 steps);
    parameters are then compared loosely, because a ReLU unit whose
    pre-activation is ~0 may take the other branch on the two backends, which
    changes single gradient entries by O(lr / B)."""
    lr = 0.05
    g = np.random.Generator(np.random.PCG64(B + use_graph))
    Ws, bs = kaiming_uniform(dims, 7)
    bs = [g.standard_normal(b.size).astype(np.float32) * 0.1 for b in bs]
    X = g.uniform(0, 1, (B, dims[0])).astype(np.float32)
    lab = g.integers(0, dims[-1], B)
    T = np.eye(dims[-1], dtype=np.float32)[lab]
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(struct.pack("<Q", len(dims)))
        f.write(np.asarray(dims, np.uint64).tobytes())
        f.write(struct.pack("<QQQd", B, steps, use_graph, lr))
        for w, b in zip(Ws, bs):
            f.write(np.ascontiguousarray(w, np.float32).tobytes())
            f.write(np.ascontiguousarray(b, np.float32).tobytes())
        f.write(X.tobytes())
        f.write(T.tobytes())
    exe = zbuild.build_host_example()
    r = subprocess.run([exe, str(inp), str(out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    got = np.fromfile(out, np.float32)
    losses, params = got[:steps], got[steps:]
    model = oracle.MlpOracle(dims, Ws, bs, "sgd", lr=lr)
    want_losses = [model.step(X, T) for _ in range(steps)]
    want_params = np.concatenate([np.concatenate([model.W[l].ravel(), model.b[l].ravel()]) for l in range(len(dims) - 1)])
    assert params.size == want_params.size
    for a, b in zip(losses, want_losses):
        assert abs(a - b) <= (1e-5 if steps == 1 else 1e-3) * abs(b), (losses, want_losses)
    assert rel_err(params, want_params) <= (1e-5 if steps == 1 else 5e-3)
