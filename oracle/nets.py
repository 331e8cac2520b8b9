"""Step drivers of the CPU oracle for the DQN and GCN configurations, composed
from the oracle's device ops in the order the reference's code issues them.
TEST INFRASTRUCTURE ONLY (see oracle/__init__.py)."""
from __future__ import annotations

import ctypes as C

import numpy as np

import oracle as O
from oracle import _f, _pp, _shape, f32, len_t, lib


class MlpNet:
    """Linear(+ReLU) stack: parameters, gradients, activations (numpy)."""

    def __init__(self, dims, weights, biases):
        self.dims, self.L = [int(d) for d in dims], len(dims) - 1
        self.W = [f32(w).copy() for w in weights]
        self.b = [f32(x).copy() for x in biases]
        self.dW = [np.zeros_like(w) for w in self.W]
        self.db = [np.zeros_like(x) for x in self.b]
        self.act = self.dact = None

    def _buffers(self, B):
        if self.act is None or self.act[0].shape[0] != B:
            self.act = [np.zeros((B, self.dims[l + 1]), np.float32) for l in range(self.L)]
            self.dact = [np.zeros((B, self.dims[l + 1]), np.float32) for l in range(self.L)]

    def forward(self, X):
        X = f32(X)
        self._buffers(X.shape[0])
        lib().orc_mlp_forward(self.L, _shape(self.dims), _pp(self.W), _pp(self.b), _f(X), len_t(X.shape[0]), _pp(self.act))
        return self.act[-1]

    def backward(self, X, d_out):
        X = f32(X)
        self.dact[-1][...] = f32(d_out).reshape(self.dact[-1].shape)
        lib().orc_mlp_backward(self.L, _shape(self.dims), _pp(self.W), _pp(self.dW), _pp(self.db), _f(X),
                               len_t(X.shape[0]), _pp(self.act), _pp(self.dact))

    def tensors(self):  # attach order: W0, b0, W1, b1, ...
        return [t for pair in zip(self.W, self.b) for t in pair]

    def grads(self):
        return [t for pair in zip(self.dW, self.db) for t in pair]


class AdamState:
    """Adam with the reference's optimizer-wide counter that advances once per
    parameter tensor (src/nn/optim.zig:189) and per-tensor clipping."""

    def __init__(self, tensors, lr, beta1=0.9, beta2=0.999, eps=1e-8, clip=True, max_norm=10.0, delta=1e-6):
        self.m = [np.zeros(t.size, np.float32) for t in tensors]
        self.v = [np.zeros(t.size, np.float32) for t in tensors]
        self.lr, self.b1, self.b2, self.eps = lr, beta1, beta2, eps
        self.clip, self.max_norm, self.delta = clip, max_norm, delta
        self.t = 0

    def step(self, tensors, grads):
        for j, (p, g) in enumerate(zip(tensors, grads)):
            self.t += 1
            O.adam_update(p.reshape(-1), g.reshape(-1), self.m[j], self.v[j], self.lr, self.b1, self.b2, self.eps, self.t,
                          self.clip, self.max_norm, self.delta)


class DqnOracle:
    """One DQN update, examples/dqn/src/dqn_agent.zig:125-228 (+ the soft target
    update of :111-123 that dqn_train.zig:83 runs after it)."""

    def __init__(self, dims, weights, biases, lr=1e-4, gamma=0.99, tau=0.005, q_clip=100.0):
        self.policy = MlpNet(dims, weights, biases)
        self.target = MlpNet(dims, weights, biases)
        self.adam = AdamState(self.policy.tensors(), lr, clip=True)
        self.gamma, self.tau, self.q_clip = gamma, tau, q_clip
        self.C = dims[-1]

    def step(self, states, actions, next_states, rewards, dones):
        B, Cn, qc = states.shape[0], self.C, self.q_clip
        # targets, no gradient (:153-187)
        qn = self.target.forward(next_states).ravel().copy()
        qn = O.clamp_fwd(qn, -qc, qc)
        mx = O.max_along(qn, [B, Cn], 1)
        disc = O.elwise("mul", mx, np.array([self.gamma], np.float32))
        comp = O.elwise("sub", np.array([1.0], np.float32), f32(dones))
        targets = O.elwise("add", f32(rewards), O.elwise("mul", disc, comp))
        targets = O.clamp_fwd(targets, -qc, qc)
        # policy forward, clamp in place (outside the graph, :196-198), gather by action (:204)
        q_all = self.policy.forward(states)
        q_all[...] = O.clamp_fwd(q_all.ravel().copy(), -qc, qc).reshape(q_all.shape)
        offs = (np.arange(B, dtype=np.uint64) * np.uint64(Cn) + actions.astype(np.uint64)).astype(np.uint64)
        q = O.take(q_all.ravel(), offs)
        loss = O.smooth_l1_fwd(q, targets, 1.0)
        dq = O.smooth_l1_bwd(q, targets, np.zeros(B, np.float32), 1.0)
        d_all = O.scatter_add(dq, offs, np.zeros(B * Cn, np.float32))  # gather backward (src/ndtensor.zig:1354-1397)
        self.policy.backward(states, d_all)
        self.adam.step(self.policy.tensors(), self.policy.grads())
        for p, t in zip(self.policy.tensors(), self.target.tensors()):  # soft update (:111-123)
            t[...] = (np.float32(1) - np.float32(self.tau)) * t + np.float32(self.tau) * p
        self.q, self.targets, self.d_all = q, targets, d_all
        return float(np.float32(loss))


def _mm(A, B, ta, tb, beta=0.0, Cin=None):
    A, B = f32(A), f32(B)
    m = A.shape[1] if ta else A.shape[0]
    k = A.shape[0] if ta else A.shape[1]
    n = B.shape[0] if tb else B.shape[1]
    Cm = np.zeros((m, n), np.float32) if Cin is None else Cin
    return O.matmul(A, B, Cm, m, n, k, ta, tb, A.shape[1], B.shape[1], n, 1.0, beta)


class GcnOracle:
    """Two-layer GCN with a DENSE normalised adjacency: every layer is
    h = x.W^T (bmm_acc trans_b), p = A_hat.h, y = p + bias
    (examples/gcn/src/model.zig:100-112 with the edge scatter of :116-224 replaced
    by the dense product it equals), ReLU between the layers (:36), row mask
    (MaskLayer :296-353), softmax cross-entropy over the masked rows, Adam with
    the library's default clipping (examples/gcn/src/main.zig:40-46)."""

    def __init__(self, A_hat, W1, b1, W2, b2, lr=0.01):
        self.A = f32(A_hat)
        self.W = [f32(W1).copy(), f32(W2).copy()]
        self.b = [f32(b1).copy(), f32(b2).copy()]
        self.adam = AdamState(self.tensors(), lr, clip=True)

    def tensors(self):
        return [self.W[0], self.b[0], self.W[1], self.b[1]]

    def step(self, X, T_masked, mask_idx, update=True):
        X, A = f32(X), self.A
        N = X.shape[0]
        H, C = self.W[0].shape[0], self.W[1].shape[0]
        # forward
        h1 = _mm(X, self.W[0], False, True)
        a1 = O.elwise("add", self.b[0], _mm(A, h1, False, False).ravel()).reshape(N, H)
        a1 = O.unary("relu_fwd", a1.ravel()).reshape(N, H)
        h2 = _mm(a1, self.W[1], False, True)
        logits = O.elwise("add", self.b[1], _mm(A, h2, False, False).ravel()).reshape(N, C)
        masked = logits[mask_idx]
        loss, sm = O.softmax_ce_fwd(masked, T_masked, len(mask_idx))
        # backward
        dm = O.softmax_ce_bwd(sm.ravel(), f32(T_masked).ravel(), np.zeros(masked.size, np.float32), len(mask_idx)).reshape(masked.shape)
        dlog = np.zeros((N, C), np.float32)
        dlog[mask_idx] = dm
        db2 = O.fold_rows(dlog.ravel(), np.zeros(C, np.float32), N, C, 1.0, 1.0)
        dh2 = _mm(A, dlog, True, False)           # d(A.h)/dh = A^T . dy
        dW2 = _mm(dh2, a1, True, False)
        da1 = _mm(dh2, self.W[1], False, False)
        da1 = O.relu_inplace_bwd(a1.ravel(), da1.ravel()).reshape(N, H)
        db1 = O.fold_rows(da1.ravel(), np.zeros(H, np.float32), N, H, 1.0, 1.0)
        dh1 = _mm(A, da1, True, False)
        dW1 = _mm(dh1, X, True, False)
        self.logits, self.a1, self.dlog, self.da1 = logits, a1, dlog, da1
        self.grads = [dW1, db1, dW2, db2]
        if update:
            self.adam.step(self.tensors(), self.grads)
        return float(np.float32(loss))


class GcnSparseOracle:
    """The reference's own GCN algorithm: every GraphConvLayer is h = x.W^T,
    y = scatter_gcn_deg_scaled(h) over the edge list + bias
    (examples/gcn/src/model.zig:100-112, :116-248; host_device.zig:1356-1403 for
    the scatter and its backward), ReLU between the layers, row mask, softmax
    cross-entropy over the masked rows, Adam with default clipping."""

    def __init__(self, src, tgt, deg, W1, b1, W2, b2, lr=0.01):
        self.src, self.tgt, self.deg = np.ascontiguousarray(src, np.uint64), np.ascontiguousarray(tgt, np.uint64), f32(deg)
        self.W = [f32(W1).copy(), f32(W2).copy()]
        self.b = [f32(b1).copy(), f32(b2).copy()]
        self.adam = AdamState(self.tensors(), lr, clip=True)

    def tensors(self):
        return [self.W[0], self.b[0], self.W[1], self.b[1]]

    def _prop(self, h):
        N, F = h.shape
        return O.scatter_gcn_deg_scaled(np.zeros(N * F, np.float32), f32(h).ravel(), self.deg, self.src, self.tgt, F).reshape(N, F)

    def _prop_bwd(self, go, h):
        N, F = go.shape
        gh, _ = O.scatter_gcn_deg_scaled_bwd(f32(go).ravel(), f32(h).ravel(), self.deg, self.src, self.tgt, np.zeros(N * F, np.float32),
                                             np.zeros(N, np.float32), F)
        return gh.reshape(N, F)

    def step(self, X, T_masked, mask_idx, update=True):
        X = f32(X)
        N = X.shape[0]
        H, C = self.W[0].shape[0], self.W[1].shape[0]
        h1 = _mm(X, self.W[0], False, True)
        a1 = O.elwise("add", self.b[0], self._prop(h1).ravel()).reshape(N, H)
        a1 = O.unary("relu_fwd", a1.ravel()).reshape(N, H)
        h2 = _mm(a1, self.W[1], False, True)
        logits = O.elwise("add", self.b[1], self._prop(h2).ravel()).reshape(N, C)
        masked = logits[mask_idx]
        loss, sm = O.softmax_ce_fwd(masked, T_masked, len(mask_idx))
        dm = O.softmax_ce_bwd(sm.ravel(), f32(T_masked).ravel(), np.zeros(masked.size, np.float32), len(mask_idx)).reshape(masked.shape)
        dlog = np.zeros((N, C), np.float32)
        dlog[mask_idx] = dm
        db2 = O.fold_rows(dlog.ravel(), np.zeros(C, np.float32), N, C, 1.0, 1.0)
        dh2 = self._prop_bwd(dlog, h2)
        dW2 = _mm(dh2, a1, True, False)
        da1 = _mm(dh2, self.W[1], False, False)
        da1 = O.relu_inplace_bwd(a1.ravel(), da1.ravel()).reshape(N, H)
        db1 = O.fold_rows(da1.ravel(), np.zeros(H, np.float32), N, H, 1.0, 1.0)
        dh1 = self._prop_bwd(da1, h1)
        dW1 = _mm(dh1, X, True, False)
        self.logits, self.a1, self.dlog, self.da1 = logits, a1, dlog, da1
        self.grads = [dW1, db1, dW2, db2]
        if update:
            self.adam.step(self.tensors(), self.grads)
        return float(np.float32(loss))
