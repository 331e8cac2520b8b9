"""Two numpy-in / numpy-out views of the device interface for the tests:

* ``OracleBackend`` -- the CPU oracle (reference HostDevice restated);
* ``GpuBackend``    -- the CUDA library through ``CudaDevice.dispatch`` (C ABI).

Both expose the same methods, so every golden-vector and parity test is
written once (``tests/callers.py`` holds the NDArray/NDTensor-level caller
logic) and runs against either.
"""
from __future__ import annotations

import numpy as np

import oracle
from zigrad_b200 import opspec
from zigrad_b200.abi import SINGLE
from zigrad_b200.device import USIZE, DeviceSlice

# Every buffer a GPU test uploads sits between two guard regions filled with this byte; they are
# checked when the test's buffers are released, so a store that strays outside its operand -- which
# the caching allocator would otherwise let land silently in a neighbouring block -- fails the test.
GUARD_BYTES = 256
GUARD_FILL = 0xA5


def f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


class OracleBackend:
    name = "oracle"

    def elwise(self, op, x, y):
        return oracle.elwise(op, f32(x), f32(y))

    def bmm_acc(self, A, B, C, As, Bs, Cs, ta, tb, lda, ldb, ldc, alpha, beta):
        C = f32(C).copy()
        return oracle.bmm_acc(f32(A), f32(B), C, As, Bs, Cs, ta, tb, lda, ldb, ldc, alpha, beta)

    def matvec(self, A, x, m, n, ta, alpha=1.0, beta=0.0, y=None):
        y = np.zeros(n if ta else m, np.float32) if y is None else f32(y).copy()
        return oracle.matvec(f32(A), f32(x), y, m, n, ta, alpha, beta)

    def dot(self, x, y):
        return oracle.dot(f32(x), f32(y))

    def unbroadcast(self, x, x_shape, y, y_shape, alpha=1.0, beta=0.0):
        return oracle.unbroadcast(f32(x).ravel(), x_shape, f32(y).ravel().copy(), y_shape, alpha, beta)

    def sum_along(self, x, shape, dim, alpha=1.0, beta=0.0, y=None):
        return oracle.sum_along(f32(x).ravel(), shape, dim, None if y is None else f32(y).copy(), alpha, beta)

    def max_along(self, x, shape, dim):
        return oracle.max_along(f32(x).ravel(), shape, dim)

    def fold_rows(self, x, row, col, alpha=1.0, beta=0.0, y=None):
        y = np.zeros(col, np.float32) if y is None else f32(y).copy()
        return oracle.fold_rows(f32(x).ravel(), y, row, col, alpha, beta)

    def fold_cols(self, x, row, col, alpha=1.0, beta=0.0, y=None):
        y = np.zeros(row, np.float32) if y is None else f32(y).copy()
        return oracle.fold_cols(f32(x).ravel(), y, row, col, alpha, beta)

    def relu_fwd(self, x):
        return oracle.unary("relu_fwd", f32(x).ravel())

    def relu_bwd(self, x, x_g, y_g):
        return oracle.relu_bwd(f32(x), f32(x_g).copy(), f32(y_g))

    def relu_inplace_bwd(self, x, x_g):
        return oracle.relu_inplace_bwd(f32(x), f32(x_g).copy())

    def clamp_fwd(self, x, lo, hi):
        return oracle.clamp_fwd(f32(x), lo, hi)

    def clamp_bwd(self, x, x_g, y_g, lo, hi):
        return oracle.clamp_bwd(f32(x), f32(x_g).copy(), f32(y_g), lo, hi)

    def unary(self, name, x, p=0.0):
        x = f32(x).ravel()
        if name == "rsqrt":
            return oracle.rsqrt_fwd(x, p)
        return oracle.unary(name + "_fwd", x)

    def unary_bwd(self, name, v, y_g, x_g, p=0.0):
        v, y_g, x_g = f32(v), f32(y_g), f32(x_g).copy()
        if name == "rsqrt":
            return oracle.rsqrt_bwd(v, x_g, y_g, p)
        if name == "sqrt":
            return oracle.sqrt_bwd(v, x_g, y_g, p)
        return oracle.bwd3(name + "_bwd", x_g, v, y_g)

    def pow_fwd(self, x, e):
        return oracle.pow_fwd(f32(x).ravel(), e)

    def pow_bwd(self, x, x_g, y_g, e, eps):
        return oracle.pow_bwd(f32(x), f32(x_g).copy(), f32(y_g), e, eps)

    def inplace_bwd(self, name, x, x_g):
        return oracle.inplace_bwd(name + "_inplace_bwd", f32(x), f32(x_g).copy())

    def relu_mask_fwd(self, x):
        x = f32(x).copy()
        mask = oracle.relu_mask_fwd(x)
        return x, mask

    def relu_mask_bwd(self, x_g, mask):
        return oracle.relu_mask_bwd(f32(x_g).copy(), np.ascontiguousarray(mask, np.uint8))

    def clamp_mask_fwd(self, x, lo, hi):
        return oracle.clamp_mask_fwd(f32(x), lo, hi)

    def clamp_mask_bwd(self, x_g, y_g, mask):
        return oracle.clamp_mask_bwd(f32(x_g).copy(), f32(y_g), np.ascontiguousarray(mask, np.uint8))

    def scatter_add_2d(self, src, indices, dst, stride):
        return oracle.scatter_add_2d(f32(src).ravel(), np.ascontiguousarray(indices, np.uint64), f32(dst).ravel().copy(), stride)

    def scatter_add_csr(self, src, row_ptr, dst):
        return oracle.scatter_add_csr(f32(src), np.ascontiguousarray(row_ptr, np.uint64), f32(dst).copy())

    def segment_sum_csr(self, src, row_offsets):
        return oracle.segment_sum_csr(f32(src), np.ascontiguousarray(row_offsets, np.uint64))

    def nrm2(self, x):
        return oracle.nrm2(f32(x))

    def asum(self, x):
        return oracle.asum(f32(x))

    def clip_nrm2(self, x, max_norm, delta):
        return oracle.clip_nrm2(f32(x).copy(), max_norm, delta)

    def scale(self, x, alpha):
        return oracle.scale(f32(x).copy(), alpha)

    def axpy(self, x, y, alpha):
        return oracle.axpy(f32(x), f32(y).copy(), alpha)

    def max_fwd(self, x):
        return oracle.max_fwd(f32(x))

    def max_bwd(self, x, x_g, y, y_g):
        return oracle.max_bwd(f32(x), f32(x_g).copy(), f32(y), f32(y_g))

    def transpose(self, A, B, m, n, alpha):
        return oracle.transpose(f32(A), f32(B).copy(), m, n, alpha)

    def take(self, src, idx):
        return oracle.take(f32(src), np.ascontiguousarray(idx, dtype=np.uint64))

    def scatter_add(self, src, offs, dst):
        return oracle.scatter_add(f32(src), np.ascontiguousarray(offs, dtype=np.uint64), f32(dst).copy())

    def scatter_gcn(self, dst, h, deg, s, t, stride):
        return oracle.scatter_gcn_deg_scaled(f32(dst).copy(), f32(h), f32(deg), s, t, stride)

    def scatter_gcn_bwd(self, go, h, deg, s, t, grad_h, grad_deg, stride):
        return oracle.scatter_gcn_deg_scaled_bwd(f32(go), f32(h), f32(deg), s, t, f32(grad_h).copy(), f32(grad_deg).copy(), stride)

    def softmax_ce(self, logits, target, loss_div=None, grad0=None):
        logits, target = f32(logits), f32(target)
        rows = 1 if logits.ndim == 1 else logits.shape[0]
        div = rows if loss_div is None else loss_div
        loss, sm = oracle.softmax_ce_fwd(logits, target, div)
        grad = np.zeros(logits.size, np.float32) if grad0 is None else f32(grad0).ravel().copy()
        oracle.softmax_ce_bwd(sm.ravel(), target.ravel(), grad, div)
        return loss, grad.reshape(logits.shape), sm.reshape(logits.shape)

    def smooth_l1(self, pred, target, beta):
        pred, target = f32(pred).ravel(), f32(target).ravel()
        grad = np.zeros_like(pred)
        loss = oracle.smooth_l1_fwd(pred, target, beta)
        oracle.smooth_l1_bwd(pred, target, grad, beta)
        return loss, grad

    def sgd(self, params, grads, segments, lr, clip=False, max_norm=10.0, delta=1e-6):
        p, g = f32(params).copy(), f32(grads).copy()
        for off, n in segments:
            oracle.sgd_update(p[off:off + n], g[off:off + n], lr, clip, max_norm, delta)
        return p, g

    def adam(self, params, grads, m, v, segments, t_first, lr, b1=0.9, b2=0.999, eps=1e-8, clip=False, max_norm=10.0,
             delta=1e-6):
        p, g, m, v = f32(params).copy(), f32(grads).copy(), f32(m).copy(), f32(v).copy()
        for j, (off, n) in enumerate(segments):
            oracle.adam_update(p[off:off + n], g[off:off + n], m[off:off + n], v[off:off + n], lr, b1, b2, eps,
                               t_first + j, clip, max_norm, delta)
        return p, g, m, v


class GpuBackend:
    """Uploads the operands, dispatches ONE op through CudaDevice (C ABI),
    downloads the result.  Buffers come from the stream-ordered cache."""
    name = "gpu"

    def __init__(self, dev):
        self.d = dev
        self._live = []

    def up(self, a, dtype=np.float32):
        a = np.ascontiguousarray(np.asarray(a, dtype=dtype)).ravel()
        g = GUARD_BYTES // a.itemsize
        padded = np.empty(a.size + 2 * g, a.dtype)
        padded.view(np.uint8)[:] = GUARD_FILL
        padded[g:g + a.size] = a
        base = self.d.from_numpy(padded)
        self._live.append((base, g, a.size))
        return DeviceSlice(base.ptr + GUARD_BYTES, a.size, base.dtype, 0)

    def check_guards(self):
        for base, g, n in self._live:
            lo = self.d.to_numpy(base.view(0, g)).view(np.uint8)
            hi = self.d.to_numpy(base.view(g + n, g)).view(np.uint8)
            assert (lo == GUARD_FILL).all(), "a kernel wrote BEFORE a %d-element operand" % n
            assert (hi == GUARD_FILL).all(), "a kernel wrote PAST a %d-element operand" % n

    def down(self, s, shape=None):
        out = self.d.to_numpy(s, shape)
        self.check_guards()
        for base, _, _ in self._live:
            self.d.mem_cache_free(base)
        self._live = []
        return out

    def scalar(self):
        return self.up(np.zeros(1, np.float32))

    def elwise(self, op, x, y):
        x, y = f32(x).ravel(), f32(y).ravel()
        X, Y, Z = self.up(x), self.up(y), self.up(np.zeros(max(x.size, y.size), np.float32))
        self.d.dispatch(getattr(opspec, op)(X, Y, Z))
        return self.down(Z)

    def bmm_acc(self, A, B, C, As, Bs, Cs, ta, tb, lda, ldb, ldc, alpha, beta):
        a, b, c = self.up(A), self.up(B), self.up(C)
        self.d.dispatch(opspec.bmm_acc(a, b, c, As, Bs, Cs, ta, tb, lda, ldb, ldc, alpha, beta))
        return self.down(c, np.asarray(C).shape)

    def linear(self, A, B, C, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bias=None, mask=None, colsum=None, sm_budget=0):
        a, b, c = self.up(A), self.up(B), self.up(C)
        bs = self.up(bias) if bias is not None else None
        mk = self.up(mask) if mask is not None else None
        cs = self.up(colsum) if colsum is not None else None
        self.d.dispatch(opspec.linear(a, b, c, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bs, mk, colsum=cs, sm_budget=sm_budget))
        sums = self.d.to_numpy(cs) if cs is not None else None
        out = self.down(c, np.asarray(C).shape)
        return (out, sums) if colsum is not None else out

    def matvec(self, A, x, m, n, ta, alpha=1.0, beta=0.0, y=None):
        y0 = np.zeros(n if ta else m, np.float32) if y is None else f32(y)
        a, xv, yv = self.up(A), self.up(x), self.up(y0)
        self.d.dispatch(opspec.matvec(a, xv, yv, m, n, ta, alpha, beta))
        return self.down(yv)

    def dot(self, x, y):
        a, b, z = self.up(x), self.up(y), self.scalar()
        self.d.dispatch(opspec.dot(a, b, z))
        return float(self.down(z)[0])

    def unbroadcast(self, x, x_shape, y, y_shape, alpha=1.0, beta=0.0):
        X, Y = self.up(x), self.up(y)
        n = oracle.unbroadcast_scratch_len(x_shape, y_shape)  # NDArray.unbroadcast_'s sizing rule
        scratch = self.d.mem_scratch(SINGLE, n) if n else None
        self.d.dispatch(opspec.unbroadcast(X, list(x_shape), Y, list(y_shape), scratch, alpha, beta))
        return self.down(Y)

    def sum_along(self, x, shape, dim, alpha=1.0, beta=0.0, y=None):
        ys = list(shape)
        ys[dim] = 1
        y0 = np.zeros(int(np.prod(ys)), np.float32) if y is None else f32(y)
        X, Y = self.up(x), self.up(y0)
        self.d.dispatch(opspec.sum_along(X, list(shape), Y, ys, dim, alpha, beta))
        return self.down(Y)

    def max_along(self, x, shape, dim):
        ys = list(shape)
        ys[dim] = 1
        X, Y = self.up(x), self.up(np.zeros(int(np.prod(ys)), np.float32))
        self.d.dispatch(opspec.max_along(X, list(shape), Y, ys, dim))
        return self.down(Y)

    def fold_rows(self, x, row, col, alpha=1.0, beta=0.0, y=None):
        y0 = np.zeros(col, np.float32) if y is None else f32(y)
        X, Y = self.up(x), self.up(y0)
        self.d.L.zg_fold_rows(SINGLE, self.d.stream, X.ptr, Y.ptr, row, col, alpha, beta)
        return self.down(Y)

    def fold_cols(self, x, row, col, alpha=1.0, beta=0.0, y=None):
        y0 = np.zeros(row, np.float32) if y is None else f32(y)
        X, Y = self.up(x), self.up(y0)
        self.d.L.zg_fold_cols(SINGLE, self.d.stream, X.ptr, Y.ptr, row, col, alpha, beta)
        return self.down(Y)

    def relu_fwd(self, x):
        X = self.up(x)
        self.d.dispatch(opspec.relu_fwd(X, X))  # in place, as nn.relu_ calls it
        return self.down(X)

    def relu_bwd(self, x, x_g, y_g):
        X, XG, YG = self.up(x), self.up(x_g), self.up(y_g)
        self.d.dispatch(opspec.relu_bwd(X, XG, YG))
        return self.down(XG)

    def relu_inplace_bwd(self, x, x_g):
        X, XG = self.up(x), self.up(x_g)
        self.d.dispatch(opspec.relu_inplace_bwd(X, XG))
        return self.down(XG)

    def clamp_fwd(self, x, lo, hi):
        X, Y = self.up(x), self.up(np.zeros(np.asarray(x).size, np.float32))
        self.d.dispatch(opspec.clamp_fwd(X, Y, lo, hi))
        return self.down(Y)

    def clamp_bwd(self, x, x_g, y_g, lo, hi):
        X, XG, YG = self.up(x), self.up(x_g), self.up(y_g)
        self.d.dispatch(opspec.clamp_bwd(X, XG, YG, lo, hi))
        return self.down(XG)

    def unary(self, name, x, p=0.0):
        X, Y = self.up(x), self.up(np.zeros(np.asarray(x).size, np.float32))
        cls = getattr(opspec, name + "_fwd")
        self.d.dispatch(cls(X, Y, p) if name == "rsqrt" else cls(X, Y))
        return self.down(Y)

    def unary_bwd(self, name, v, y_g, x_g, p=0.0):
        V, YG, XG = self.up(v), self.up(y_g), self.up(x_g)
        cls = getattr(opspec, name + "_bwd")
        if name in ("sqrt", "rsqrt"):
            self.d.dispatch(cls(V, XG, YG, p))
        else:
            self.d.dispatch(cls(XG, V, YG))
        return self.down(XG)

    def pow_fwd(self, x, e, inplace=False):
        X = self.up(x)
        if inplace:
            self.d.dispatch(opspec.pow_fwd_(X, e))
            return self.down(X)
        Y = self.up(np.zeros(np.asarray(x).size, np.float32))
        self.d.dispatch(opspec.pow_fwd(X, e, Y))
        return self.down(Y)

    def sqrt_inplace(self, x):
        X = self.up(x)
        self.d.dispatch(opspec.sqrt_fwd_(X))
        return self.down(X)

    def pow_bwd(self, x, x_g, y_g, e, eps):
        X, XG, YG = self.up(x), self.up(x_g), self.up(y_g)
        self.d.dispatch(opspec.pow_bwd(X, XG, e, YG, eps))
        return self.down(XG)

    def inplace_bwd(self, name, x, x_g):
        X, XG = self.up(x), self.up(x_g)
        self.d.dispatch(getattr(opspec, name + "_inplace_bwd")(X, XG))
        return self.down(XG)

    def relu_mask_fwd(self, x):
        X = self.up(x)
        M = self.up(np.full((np.asarray(x).size + 7) // 8, 0xFF, np.uint8), np.uint8)  # stale contents must not survive
        self.d.dispatch(opspec.relu_mask_fwd(X, M))
        m = self.d.to_numpy(M)
        return self.down(X), m

    def relu_mask_bwd(self, x_g, mask):
        XG, M = self.up(x_g), self.up(mask, np.uint8)
        self.d.dispatch(opspec.relu_mask_bwd(XG, M))
        return self.down(XG)

    def clamp_mask_fwd(self, x, lo, hi):
        n = np.asarray(x).size
        X, Y = self.up(x), self.up(np.zeros(n, np.float32))
        M = self.up(np.full((n + 7) // 8, 0xFF, np.uint8), np.uint8)
        self.d.dispatch(opspec.clamp_mask_fwd(X, Y, lo, hi, M))
        m = self.d.to_numpy(M)
        return self.down(Y), m

    def clamp_mask_bwd(self, x_g, y_g, mask):
        XG, YG, M = self.up(x_g), self.up(y_g), self.up(mask, np.uint8)
        self.d.dispatch(opspec.clamp_mask_bwd(XG, YG, M))
        return self.down(XG)

    def scatter_add_2d(self, src, indices, dst, stride):
        S, I, D = self.up(src), self.up(indices, np.uint64), self.up(dst)
        self.d.dispatch(opspec.scatter_add_2d(S, I, D, stride))
        return self.down(D)

    def scatter_add_csr(self, src, row_ptr, dst):
        S, R, D = self.up(src), self.up(row_ptr, np.uint64), self.up(dst)
        self.d.dispatch(opspec.scatter_add_csr(S, R, D))
        return self.down(D)

    def segment_sum_csr(self, src, row_offsets):
        S, R = self.up(src), self.up(row_offsets, np.uint64)
        D = self.up(np.full(np.asarray(row_offsets).size - 1, 7.0, np.float32))  # dst is overwritten
        self.d.dispatch(opspec.segment_sum_csr(S, R, D))
        return self.down(D)

    def nrm2(self, x):
        X, Y = self.up(x), self.scalar()
        self.d.dispatch(opspec.nrm2(X, Y))
        return float(self.down(Y)[0])

    def asum(self, x):
        X, Y = self.up(x), self.scalar()
        self.d.dispatch(opspec.sum(X, Y))
        return float(self.down(Y)[0])

    def clip_nrm2(self, x, max_norm, delta):
        X = self.up(x)
        self.d.dispatch(opspec.clip_nrm2(X, max_norm, delta))
        return self.down(X)

    def scale(self, x, alpha):
        X = self.up(x)
        self.d.dispatch(opspec.scale(X, alpha))
        return self.down(X)

    def axpy(self, x, y, alpha, device_alpha=False):
        X, Y = self.up(x), self.up(y)
        a = self.up(np.array([alpha], np.float32)) if device_alpha else alpha
        self.d.dispatch(opspec.axpy(X, Y, a))
        return self.down(Y)

    def max_fwd(self, x):
        X, Y = self.up(x), self.scalar()
        self.d.dispatch(opspec.max_fwd(X, Y))
        return self.down(Y)

    def max_bwd(self, x, x_g, y, y_g):
        X, XG, Y, YG = self.up(x), self.up(x_g), self.up(y), self.up(y_g)
        self.d.dispatch(opspec.max_bwd(X, XG, Y, YG))
        return self.down(XG)

    def transpose(self, A, B, m, n, alpha):
        a, b = self.up(A), self.up(B)
        self.d.dispatch(opspec.transpose(a, b, m, n, alpha))
        return self.down(b)

    def take(self, src, idx):
        S, I = self.up(src), self.up(idx, np.uint64)
        D = self.up(np.zeros(np.asarray(idx).size, np.float32))
        self.d.mem_take(S, I, D)
        return self.down(D)

    def scatter_add(self, src, offs, dst):
        S, O, D = self.up(src), self.up(offs, np.uint64), self.up(dst)
        self.d.dispatch(opspec.scatter_add(S, O, D))
        return self.down(D)

    def scatter_gcn(self, dst, h, deg, s, t, stride):
        D, H, G = self.up(dst), self.up(h), self.up(deg)
        Si, Ti = self.up(s, np.uint64), self.up(t, np.uint64)
        self.d.dispatch(opspec.scatter_gcn_deg_scaled(D, H, G, Si, Ti, stride, len(s)))
        return self.down(D)

    def scatter_gcn_bwd(self, go, h, deg, s, t, grad_h, grad_deg, stride):
        GO, H, G = self.up(go), self.up(h), self.up(deg)
        Si, Ti = self.up(s, np.uint64), self.up(t, np.uint64)
        GH, GD = self.up(grad_h), self.up(grad_deg)
        self.d.dispatch(opspec.scatter_gcn_deg_scaled_bwd(GO, H, G, Si, Ti, GH, GD, stride, len(s)))
        gh = self.d.to_numpy(GH)
        return gh, self.down(GD)

    def softmax_ce(self, logits, target, loss_div=None, grad0=None, index_labels=None, ld=0, want_bias=False):
        logits = f32(logits)
        rows, Cc = (1, logits.shape[0]) if logits.ndim == 1 else logits.shape
        ldv = ld if ld else Cc
        padded = np.zeros((rows, ldv), np.float32)
        padded[:, :Cc] = logits.reshape(rows, Cc)
        g0 = np.zeros((rows, ldv), np.float32)
        if grad0 is not None:
            g0[:, :Cc] = f32(grad0).reshape(rows, Cc)
        X = self.up(padded)
        T = self.up(index_labels, np.uint64) if index_labels is not None else self.up(target)
        G, P, Ls = self.up(g0), self.up(np.zeros((rows, ldv), np.float32)), self.scalar()
        Bg = self.up(np.zeros(Cc, np.float32)) if want_bias else None
        self.d.dispatch(opspec.softmax_ce(X, T, rows, Cc, Ls, G, loss_div, True, P, ld, Bg))
        g = self.d.to_numpy(G, (rows, ldv))[:, :Cc].reshape(logits.shape)
        pr = self.d.to_numpy(P, (rows, ldv))[:, :Cc].reshape(logits.shape)
        bias = self.d.to_numpy(Bg) if want_bias else None
        loss = float(self.down(Ls)[0])
        return (loss, g, pr, bias) if want_bias else (loss, g, pr)

    def smooth_l1(self, pred, target, beta):
        Pd, T = self.up(pred), self.up(target)
        G, Ls = self.up(np.zeros(np.asarray(pred).size, np.float32)), self.scalar()
        self.d.dispatch(opspec.smooth_l1(Pd, T, beta, Ls, G))
        g = self.d.to_numpy(G)
        return float(self.down(Ls)[0]), g

    def sgd(self, params, grads, segments, lr, clip=False, max_norm=10.0, delta=1e-6):
        P, G = self.up(params), self.up(grads)
        N = self.up(np.zeros(len(segments), np.float32))
        self.d.dispatch(opspec.sgd(P, G, segments, lr, clip, max_norm, delta, N))
        p = self.d.to_numpy(P)
        return p, self.down(G)

    def adam(self, params, grads, m, v, segments, t_first, lr, b1=0.9, b2=0.999, eps=1e-8, clip=False, max_norm=10.0,
             delta=1e-6):
        P, G, M, V = self.up(params), self.up(grads), self.up(m), self.up(v)
        N = self.up(np.zeros(len(segments), np.float32))
        self.d.dispatch(opspec.adam(P, G, M, V, segments, t_first, lr, b1, b2, eps, clip, max_norm, delta, N))
        p, g, mm = self.d.to_numpy(P), self.d.to_numpy(G), self.d.to_numpy(M)
        return p, g, mm, self.down(V)
