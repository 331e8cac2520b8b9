"""Seeded synthetic inputs with the shapes and value distributions of the
reference's example datasets (MNIST, Cora, CartPole replay), which are not
available offline.  One numpy PCG64 stream per tensor."""
from __future__ import annotations

import numpy as np


def _gen(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def mlp_batch(B: int, n_in: int, n_out: int, seed: int, normal: bool = False):
    """Inputs uniform [0,1) (or N(0,1)), labels uniform; returns X, one-hot T, labels."""
    g = _gen(seed)
    X = (g.standard_normal((B, n_in)) if normal else g.uniform(0.0, 1.0, (B, n_in))).astype(np.float32)
    lab = g.integers(0, n_out, B)
    T = np.zeros((B, n_out), np.float32)
    T[np.arange(B), lab] = 1.0
    return X, T, lab


def gcn_graph(n_nodes: int = 2708, n_directed_edges: int = 10556, seed: int = 81761, exponent: float = 2.5):
    """Random undirected graph with a power-law degree profile (Cora's size by
    default): returns (src, tgt) u64 arrays of the directed edge list (both
    directions of every undirected edge, no self loops, no duplicates)."""
    g = _gen(seed)
    want = n_directed_edges // 2
    # node weights ~ k^(-exponent) degree propensity (Chung-Lu style sampling)
    w = (np.arange(1, n_nodes + 1, dtype=np.float64)) ** (-1.0 / (exponent - 1.0))
    g.shuffle(w)
    p = w / w.sum()
    edges = set()
    while len(edges) < want:
        a = g.choice(n_nodes, size=want, p=p)
        b = g.choice(n_nodes, size=want, p=p)
        for i, j in zip(a, b):
            if i != j:
                edges.add((min(i, j), max(i, j)))
                if len(edges) == want:
                    break
    e = np.array(sorted(edges), dtype=np.uint64)
    src = np.concatenate([e[:, 0], e[:, 1]])
    tgt = np.concatenate([e[:, 1], e[:, 0]])
    return np.ascontiguousarray(src), np.ascontiguousarray(tgt)


def gcn_dense_adjacency(src, tgt, n_nodes: int) -> np.ndarray:
    """A_hat = D^-1/2 (A + I) D^-1/2 with D = rowsum(A + I), dense fp32."""
    A = np.zeros((n_nodes, n_nodes), np.float64)
    A[tgt.astype(np.int64), src.astype(np.int64)] = 1.0
    A[np.arange(n_nodes), np.arange(n_nodes)] = 1.0
    d = 1.0 / np.sqrt(A.sum(1))
    return (A * d[:, None] * d[None, :]).astype(np.float32)


def gcn_scatter_equivalent(src, tgt, n_nodes: int) -> np.ndarray:
    """The dense matrix that the reference's edge scatter computes
    (examples/gcn/src/model.zig:207-248): A'[t, s] = sum over edges s->t of
    d[s] d[t], d = (1 + indegree)^-1/2 -- no self message although the +1 is in
    the degree."""
    deg = np.ones(n_nodes, np.float32)
    np.add.at(deg, tgt.astype(np.int64), np.float32(1.0))
    d = (np.float32(1.0) / np.sqrt(np.maximum(deg, np.float32(1e-12)))).astype(np.float32)
    A = np.zeros((n_nodes, n_nodes), np.float32)
    np.add.at(A, (tgt.astype(np.int64), src.astype(np.int64)), d[src.astype(np.int64)] * d[tgt.astype(np.int64)])
    return A, d


def gcn_features(n_nodes: int = 2708, n_feat: int = 1433, density: float = 0.013, seed: int = 7):
    g = _gen(seed)
    return (g.random((n_nodes, n_feat)) < density).astype(np.float32)


def dqn_batch(B: int = 256, seed: int = 3):
    """Replay transitions: states N(0,1) [B,4], actions {0,1}, reward 1, done ~ Bernoulli(0.05)."""
    g = _gen(seed)
    s = g.standard_normal((B, 4)).astype(np.float32)
    s2 = g.standard_normal((B, 4)).astype(np.float32)
    a = g.integers(0, 2, B).astype(np.uint64)
    r = np.ones(B, np.float32)
    done = (g.random(B) < 0.05).astype(np.float32)
    return s, a, s2, r, done


def gcn_degree_scale(tgt, n_nodes: int) -> np.ndarray:
    """d = (1 + in-degree)^-1/2, as the reference's GCN layer computes it
    (examples/gcn/src/model.zig:207-224)."""
    deg = np.ones(n_nodes, np.float32)
    np.add.at(deg, np.asarray(tgt).astype(np.int64), np.float32(1.0))
    return (np.float32(1.0) / np.sqrt(np.maximum(deg, np.float32(1e-12)))).astype(np.float32)


def edges_to_csr(rows, cols, n_nodes: int):
    """CSR of an edge list grouped by `rows` with a STABLE sort (edges of one row
    keep their list order): returns (row_ptr u64 [n+1], col_idx u64 [n_edge])."""
    rows = np.asarray(rows).astype(np.int64)
    order = np.argsort(rows, kind="stable")
    counts = np.bincount(rows, minlength=n_nodes)
    row_ptr = np.zeros(n_nodes + 1, np.uint64)
    row_ptr[1:] = np.cumsum(counts)
    return row_ptr, np.ascontiguousarray(np.asarray(cols)[order].astype(np.uint64))
