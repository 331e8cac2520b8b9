"""CPU checks of the oracle's step drivers (no GPU): internal consistency with
independent formulations, since the reference holds no golden vectors for them."""
import numpy as np
import torch

from oracle.nets import DqnOracle, GcnOracle
from zigrad_b200 import synthetic
from zigrad_b200.mlp import kaiming_uniform


def test_edge_scatter_equals_its_dense_matrix(orc):
    """scatter_gcn_deg_scaled (host_device.zig:1356-1370) over the edge list is the
    product with the dense matrix A'[t,s] = sum d[s] d[t] that it defines."""
    N, F = 300, 16
    src, tgt = synthetic.gcn_graph(N, 1200, 3)
    Ad, d = synthetic.gcn_scatter_equivalent(src, tgt, N)
    h = np.random.Generator(np.random.PCG64(1)).standard_normal((N, F)).astype(np.float32)
    got = orc.scatter_gcn_deg_scaled(np.zeros(N * F, np.float32), h.ravel(), d, src, tgt, F).reshape(N, F)
    want = (Ad.astype(np.float64) @ h.astype(np.float64))
    assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))


def test_synthetic_graph_has_the_requested_size_and_is_symmetric():
    src, tgt = synthetic.gcn_graph(2708, 10556, 81761)
    assert src.size == tgt.size == 10556
    pairs = set(zip(src.tolist(), tgt.tolist()))
    assert len(pairs) == 10556 and all((t, s) in pairs for s, t in pairs) and all(s != t for s, t in pairs)
    A = synthetic.gcn_dense_adjacency(src, tgt, 2708)
    assert np.array_equal(A, A.T) and abs(float(np.linalg.eigvalsh(A.astype(np.float64)).max()) - 1.0) < 1e-5


def test_mlp_oracle_step_matches_torch_autograd(orc):
    """SGD + Linear/ReLU/cross-entropy are torch-equivalent: one step of the
    oracle against torch autograd on the same numbers."""
    dims, B = [20, 16, 8, 5], 32
    g = np.random.Generator(np.random.PCG64(9))
    Ws, bs = kaiming_uniform(dims, 1)
    bs = [g.standard_normal(b.size).astype(np.float32) * 0.1 for b in bs]
    X = g.uniform(0, 1, (B, dims[0])).astype(np.float32)
    lab = g.integers(0, dims[-1], B)
    T = np.eye(dims[-1], dtype=np.float32)[lab]
    model = orc.MlpOracle(dims, Ws, bs, "sgd", lr=0.1)
    loss = model.step(X, T)
    tW = [torch.tensor(w, requires_grad=True) for w in Ws]
    tb = [torch.tensor(b, requires_grad=True) for b in bs]
    h = torch.tensor(X)
    for l in range(3):
        h = h @ tW[l].T + tb[l]
        if l < 2:
            h = torch.relu(h)
    tl = torch.nn.functional.cross_entropy(h, torch.tensor(lab))
    tl.backward()
    assert abs(loss - tl.item()) <= 1e-5 * abs(tl.item())
    for l in range(3):
        np.testing.assert_allclose(model.dW[l], tW[l].grad.numpy(), rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(model.db[l], tb[l].grad.numpy(), rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(model.W[l], (tW[l] - 0.1 * tW[l].grad).detach().numpy(), rtol=1e-5, atol=1e-6)


def test_gcn_oracle_gradients_match_torch_autograd(orc):
    N, F, H, C, M = 60, 23, 16, 7, 20
    src, tgt = synthetic.gcn_graph(N, 200, 5)
    A = synthetic.gcn_dense_adjacency(src, tgt, N)
    X = synthetic.gcn_features(N, F, 0.2)
    (W1, W2), (b1, b2) = kaiming_uniform([F, H, C], 2)
    g = np.random.Generator(np.random.PCG64(4))
    mask = np.sort(g.permutation(N)[:M])
    lab = g.integers(0, C, M)
    model = GcnOracle(A, W1, b1, W2, b2)
    loss = model.step(X, np.eye(C, dtype=np.float32)[lab], mask, update=False)
    t = lambda a: torch.tensor(a, requires_grad=True)
    tW1, tb1, tW2, tb2 = t(W1), t(b1), t(W2), t(b2)
    tA, tX = torch.tensor(A), torch.tensor(X)
    a1 = torch.relu(tA @ (tX @ tW1.T) + tb1)
    logits = tA @ (a1 @ tW2.T) + tb2
    tl = torch.nn.functional.cross_entropy(logits[torch.tensor(mask)], torch.tensor(lab))
    tl.backward()
    assert abs(loss - tl.item()) <= 1e-5 * abs(tl.item())
    for got, want in zip(model.grads, (tW1.grad, tb1.grad, tW2.grad, tb2.grad)):
        np.testing.assert_allclose(got, want.numpy(), rtol=1e-4, atol=1e-6)


def test_dqn_oracle_loss_and_gradients_match_torch(orc):
    dims, B = [4, 128, 128, 2], 256
    Ws, bs = kaiming_uniform(dims, 21)
    s, a, s2, r, done = synthetic.dqn_batch(B, 30)
    model = DqnOracle(dims, Ws, bs)
    loss = model.step(s, a, s2, r, done)
    tW = [torch.tensor(w, requires_grad=True) for w in Ws]
    tb = [torch.tensor(b, requires_grad=True) for b in bs]

    def net(x):
        h = torch.tensor(x)
        for l in range(3):
            h = h @ tW[l].T + tb[l]
            if l < 2:
                h = torch.relu(h)
        return h

    with torch.no_grad():
        tgt = torch.tensor(r) + 0.99 * net(s2).clamp(-100, 100).max(1).values * (1 - torch.tensor(done))
        tgt = tgt.clamp(-100, 100)
    q = net(s).gather(1, torch.tensor(a.astype(np.int64))[:, None])[:, 0]
    tl = torch.nn.functional.smooth_l1_loss(q, tgt, beta=1.0)
    tl.backward()
    assert abs(loss - tl.item()) <= 1e-5 * abs(tl.item())
    for l in range(3):
        np.testing.assert_allclose(model.policy.dW[l], tW[l].grad.numpy(), rtol=1e-4, atol=1e-7)
        np.testing.assert_allclose(model.policy.db[l], tb[l].grad.numpy(), rtol=1e-4, atol=1e-7)


def test_sparse_gcn_oracle_equals_dense_oracle_on_the_scatter_matrix(orc):
    """The reference's edge-scatter GCN step and the dense-adjacency step agree
    when the dense matrix is the one the scatter defines."""
    from oracle.nets import GcnSparseOracle
    N, F, H, C, M = 80, 31, 16, 7, 25
    src, tgt = synthetic.gcn_graph(N, 300, 9)
    Ad, d = synthetic.gcn_scatter_equivalent(src, tgt, N)
    np.testing.assert_array_equal(d, synthetic.gcn_degree_scale(tgt, N))
    X = synthetic.gcn_features(N, F, 0.2)
    (W1, W2), (b1, b2) = kaiming_uniform([F, H, C], 3)
    g = np.random.Generator(np.random.PCG64(5))
    mask = np.sort(g.permutation(N)[:M])
    T = np.eye(C, dtype=np.float32)[g.integers(0, C, M)]
    sp, de = GcnSparseOracle(src, tgt, d, W1, b1, W2, b2), GcnOracle(Ad, W1, b1, W2, b2)
    l1, l2 = sp.step(X, T, mask, update=False), de.step(X, T, mask, update=False)
    assert abs(l1 - l2) <= 1e-5 * abs(l2)
    for a, b in zip(sp.grads, de.grads):
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)
    # CSR built by a stable sort keeps the edges of a row in list order
    rp, ci = synthetic.edges_to_csr(tgt, src, N)
    assert rp[-1] == src.size
    for t in (0, N // 2, N - 1):
        np.testing.assert_array_equal(ci[int(rp[t]):int(rp[t + 1])], src[tgt == t])
