"""Whole-step parity for the GCN (dense adjacency, 2708 nodes) and DQN
(4-128-128-2, batch 256) configurations against the CPU oracle."""
import numpy as np
import pytest

import oracle
from oracle.nets import DqnOracle, GcnOracle, GcnSparseOracle
from zigrad_b200 import opspec, synthetic
from zigrad_b200.dqn import DqnTrainer
from zigrad_b200.gcn import GcnTrainer
from zigrad_b200.mlp import kaiming_uniform

from .test_gpu_ops import rel_err

pytestmark = pytest.mark.gpu


def gcn_setup(N=2708, E=10556, F=1433, H=16, C=7, M=140):
    src, tgt = synthetic.gcn_graph(N, E, 81761)
    A = synthetic.gcn_dense_adjacency(src, tgt, N)
    X = synthetic.gcn_features(N, F)
    (W1, W2), (b1, b2) = kaiming_uniform([F, H, C], 11)
    g = np.random.Generator(np.random.PCG64(12))
    mask = np.sort(g.permutation(N)[:M]).astype(np.int64)  # a random (non-prefix) train mask
    T = np.eye(C, dtype=np.float32)[g.integers(0, C, M)]
    return A, X, W1, b1, W2, b2, mask, T


@pytest.mark.parametrize("size", ["cora", "small"])
def test_gcn_step_every_tensor_and_adam_steps(gpu, size):
    args = gcn_setup() if size == "cora" else gcn_setup(300, 1200, 97, 16, 7, 40)
    A, X, W1, b1, W2, b2, mask, T = args
    orc = GcnOracle(A, W1, b1, W2, b2, lr=0.01)
    tr = GcnTrainer(gpu, A, X, W1, b1, W2, b2, mask, lr=0.01)
    Td = gpu.from_numpy(T)
    for step in range(3):
        want = orc.step(X, T, mask)
        tr.step(Td)
        got = tr.read_loss()
        assert abs(got - want) <= 1e-4 * abs(want), (step, got, want)
        if step == 0:  # forward / backward tensors from identical parameters
            assert rel_err(tr.numpy("a1"), orc.a1) <= 1e-4
            assert rel_err(tr.numpy("logits"), orc.logits) <= 1e-4
            assert rel_err(tr.numpy("dlog"), orc.dlog) <= 1e-4
            assert rel_err(tr.numpy("da1"), orc.da1) <= 1e-4
            np.testing.assert_array_equal(np.argmax(tr.numpy("logits"), 1), np.argmax(orc.logits, 1))
        for name, want_g in zip(("dW1", "db1", "dW2", "db2"), orc.grads):
            assert rel_err(tr.numpy(name), want_g) <= 1e-4, (step, name, rel_err(tr.numpy(name), want_g))
    assert tr.t == orc.adam.t == 12
    # Adam amplifies rounding-level gradient noise on near-zero gradients (see test_gpu_mlp_step.py)
    for name, want_p in zip(("W1", "b1", "W2", "b2"), orc.tensors()):
        assert rel_err(tr.numpy(name), want_p) <= 2e-2, name
    tr.free()
    gpu.mem_cache_free(Td)


def test_dqn_update_steps(gpu):
    dims = [4, 128, 128, 2]
    Ws, bs = kaiming_uniform(dims, 21)
    orc = DqnOracle(dims, Ws, bs)
    tr = DqnTrainer(gpu, dims, 256, Ws, bs)
    for step in range(3):
        s, a, s2, r, done = synthetic.dqn_batch(256, 30 + step)
        dev = [gpu.from_numpy(x) for x in (s, a, s2, r, done)]
        want = orc.step(s, a, s2, r, done)
        tr.step(*dev)
        got = tr.read_loss()
        assert abs(got - want) <= 1e-4 * abs(want), (step, got, want)
        np.testing.assert_allclose(gpu.to_numpy(tr.targets), orc.targets, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(gpu.to_numpy(tr.q), orc.q, rtol=1e-4, atol=1e-5)
        gW, gb = tr.policy.get_grads()
        for l in range(3):
            assert rel_err(gW[l], orc.policy.dW[l]) <= 1e-4, (step, l)
            assert rel_err(gb[l], orc.policy.db[l]) <= 1e-4, (step, l)
        for x in dev:
            gpu.mem_cache_free(x)
    pW, _ = tr.policy.get_params()
    tW, _ = tr.target.get_params()
    for l in range(3):
        assert rel_err(pW[l], orc.policy.W[l]) <= 2e-2
        assert rel_err(tW[l], orc.target.W[l]) <= 1e-4  # soft update moves the target by tau = 0.005 of the difference
    tr.free()


def test_dqn_step_replays_as_one_graph(gpu):
    dims = [4, 128, 128, 2]
    Ws, bs = kaiming_uniform(dims, 22)
    s, a, s2, r, done = synthetic.dqn_batch(256, 5)
    dev = [gpu.from_numpy(x) for x in (s, a, s2, r, done)]
    eager, graph = DqnTrainer(gpu, dims, 256, Ws, bs), DqnTrainer(gpu, dims, 256, Ws, bs)
    for _ in range(4):
        eager.step(*dev)
    graph.step(*dev)
    gpu.capture.open()
    graph.step(*dev)
    gpu.capture.save()
    assert gpu.capture.kernel_count() > 10
    for _ in range(3):
        gpu.capture.run()
    gpu.sync()
    assert abs(graph.read_loss() - eager.read_loss()) <= 1e-4 * abs(eager.read_loss())
    gpu.capture.free()
    eager.free()
    graph.free()
    for x in dev:
        gpu.mem_cache_free(x)


def sparse_setup(N=2708, E=10556, F=1433, H=16, C=7, M=140, seed=81761):
    src, tgt = synthetic.gcn_graph(N, E, seed)
    deg = synthetic.gcn_degree_scale(tgt, N)
    X = synthetic.gcn_features(N, F)
    (W1, W2), (b1, b2) = kaiming_uniform([F, H, C], 11)
    g = np.random.Generator(np.random.PCG64(12))
    b1, b2 = (g.standard_normal(H) * 0.1).astype(np.float32), (g.standard_normal(C) * 0.1).astype(np.float32)
    mask = np.sort(g.permutation(N)[:M]).astype(np.int64)
    T = np.eye(C, dtype=np.float32)[g.integers(0, C, M)]
    return src, tgt, deg, X, W1, b1, W2, b2, mask, T


@pytest.mark.parametrize("stride", [1, 7, 16, 33])
def test_csr_propagate_is_bit_identical_to_the_edge_scatter(gpu, stride):
    """Forward and grad_h of scatter_gcn_deg_scaled (host loops over the edge
    list) against the CSR row walk: same products, same summation order."""
    N = 500
    src, tgt = synthetic.gcn_graph(N, 3000, 4)
    deg = synthetic.gcn_degree_scale(tgt, N)
    g = np.random.Generator(np.random.PCG64(stride))
    h = g.standard_normal((N, stride)).astype(np.float32)
    go = g.standard_normal((N, stride)).astype(np.float32)
    want = oracle.scatter_gcn_deg_scaled(np.zeros(N * stride, np.float32), h.ravel(), deg, src, tgt, stride).reshape(N, stride)
    want_gh, _ = oracle.scatter_gcn_deg_scaled_bwd(go.ravel(), h.ravel(), deg, src, tgt, np.zeros(N * stride, np.float32), np.zeros(N, np.float32), stride)
    rp, ci = synthetic.edges_to_csr(tgt, src, N)
    rpt, cit = synthetic.edges_to_csr(src, tgt, N)
    d = gpu
    bufs = [d.from_numpy(a) for a in (h, go, deg, rp, ci, rpt, cit, np.zeros((N, stride), np.float32))]
    H_, GO, DEG, RP, CI, RPT, CIT, OUT = bufs
    d.dispatch(opspec.csr_gcn_propagate(OUT, H_, DEG, RP, CI, N, stride, stride, stride))
    np.testing.assert_array_equal(d.to_numpy(OUT, (N, stride)), want)
    d.dispatch(opspec.csr_gcn_propagate(OUT, GO, DEG, RPT, CIT, N, stride, stride, stride, True))
    np.testing.assert_array_equal(d.to_numpy(OUT, (N, stride)), want_gh.reshape(N, stride))
    bias = d.from_numpy(g.standard_normal(stride).astype(np.float32))
    d.dispatch(opspec.csr_gcn_propagate(OUT, H_, DEG, RP, CI, N, stride, stride, stride, False, "bias_relu", bias))
    np.testing.assert_array_equal(d.to_numpy(OUT, (N, stride)), np.maximum(want + d.to_numpy(bias)[None, :], 0))
    for s in bufs + [bias]:
        d.mem_cache_free(s)


@pytest.mark.parametrize("size", ["cora", "small"])
def test_sparse_gcn_step_matches_the_reference_algorithm(gpu, size):
    """The reference's own GCN step (edge scatter) on the GPU with CSR
    propagation against the oracle that runs the host scatter loops."""
    src, tgt, deg, X, W1, b1, W2, b2, mask, T = sparse_setup() if size == "cora" else sparse_setup(300, 1200, 97, 16, 7, 40, 5)
    orc = GcnSparseOracle(src, tgt, deg, W1, b1, W2, b2, lr=0.01)
    tr = GcnTrainer(gpu, None, X, W1, b1, W2, b2, mask, lr=0.01, edges=(src, tgt, deg))
    Td = gpu.from_numpy(T)
    for step in range(3):
        want = orc.step(X, T, mask)
        tr.step(Td)
        got = tr.read_loss()
        assert abs(got - want) <= 1e-4 * abs(want), (step, got, want)
        if step == 0:
            assert rel_err(tr.numpy("a1"), orc.a1) <= 1e-4
            assert rel_err(tr.numpy("logits"), orc.logits) <= 1e-4
            assert rel_err(tr.numpy("da1"), orc.da1) <= 1e-4
            np.testing.assert_array_equal(np.argmax(tr.numpy("logits"), 1), np.argmax(orc.logits, 1))
        for name, want_g in zip(("dW1", "db1", "dW2", "db2"), orc.grads):
            assert rel_err(tr.numpy(name), want_g) <= 1e-4, (step, name, rel_err(tr.numpy(name), want_g))
    for name, want_p in zip(("W1", "b1", "W2", "b2"), orc.tensors()):
        assert rel_err(tr.numpy(name), want_p) <= 2e-2, name
    tr.free()
    gpu.mem_cache_free(Td)
