"""Caller-side logic of the reference restated for the tests: what NDArray /
NDTensor do ABOVE the device interface (shape algebra, which device ops a
backward pass issues).  Works over either backend of tests/backends.py."""
from __future__ import annotations

import numpy as np


def f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def bmm(be, A, B, ta=False, tb=False, alpha=1.0, beta=0.0, C=None):
    """NDArray.bmm_acc_impl (src/ndarray.zig:817-899): batch dims, M/N/K and
    leading dimensions, then ONE bmm_acc device call."""
    A, B = f32(A), f32(B)
    a_shape = A.shape if A.ndim >= 2 else (1,) + A.shape
    b_shape = B.shape if B.ndim >= 2 else (1,) + B.shape
    a_batch = a_shape[:-2] if len(a_shape) > 2 else (1,)
    b_batch = b_shape[:-2] if len(b_shape) > 2 else (1,)
    bb = () if (len(a_shape) == 2 and len(b_shape) == 2) else tuple(np.broadcast_shapes(a_batch, b_batch))
    a_rows, a_cols = a_shape[-2:]
    b_rows, b_cols = b_shape[-2:]
    M = a_cols if ta else a_rows
    K = a_rows if ta else a_cols
    N = b_rows if tb else b_cols
    c_shape = bb + (M, N)
    if C is None:
        C = np.zeros(c_shape, np.float32)
    nA, nB = int(np.prod(a_batch)), int(np.prod(b_batch))
    nC = int(np.prod(bb)) if bb else 1
    out = be.bmm_acc(A, B, f32(C), (nA, M, K), (nB, K, N), (nC, M, N), ta, tb, a_cols, b_cols, N, alpha, beta)
    return np.asarray(out).reshape(c_shape)


def bmm_backward(be, A, B, ta, tb, dC):
    """BmmAccBwd (src/ndtensor.zig:1092-1136): the eight beta=1 GEMMs into
    zero-filled gradients, keyed on the forward transposes."""
    A, B, dC = f32(A), f32(B), f32(dC)
    gA, gB = np.zeros_like(A), np.zeros_like(B)
    if not ta and not tb:      # MATMUL_AB
        gA = bmm(be, dC, B, False, True, 1.0, 1.0, gA)
        gB = bmm(be, A, dC, True, False, 1.0, 1.0, gB)
    elif ta and not tb:        # MATMUL_AtB
        gA = bmm(be, B, dC, False, True, 1.0, 1.0, gA)
        gB = bmm(be, A, dC, False, False, 1.0, 1.0, gB)
    elif not ta and tb:        # MATMUL_ABt
        gA = bmm(be, dC, B, False, False, 1.0, 1.0, gA)
        gB = bmm(be, dC, A, True, False, 1.0, 1.0, gB)
    else:                      # MATMUL_AtBt
        gA = bmm(be, B, dC, True, True, 1.0, 1.0, gA)
        gB = bmm(be, dC, A, True, True, 1.0, 1.0, gB)
    return gA, gB


def add_forward_backward(be, x, x_shape, y, y_shape):
    """NDTensor.add + AddBwd (src/ndtensor.zig:745-778): z = x + y through the
    wrapping-broadcast add; grads = unbroadcast(ones, alpha=1, beta=1)."""
    z = be.elwise("add", x, y)
    gz = np.ones(z.size, np.float32)
    gx = be.unbroadcast(gz, list(x_shape), np.zeros(int(np.prod(x_shape)), np.float32), list(x_shape), 1.0, 1.0)
    gy = be.unbroadcast(gz, list(x_shape), np.zeros(int(np.prod(y_shape)), np.float32), list(y_shape), 1.0, 1.0)
    return z, gx, gy


def div_backward(be, a, b, gc):
    """DivBwd (src/ndtensor.zig:862-893)."""
    n = np.asarray(a).size
    ga = be.unbroadcast(be.elwise("div", gc, b), [n], np.zeros(n, np.float32), [n], 1.0, 1.0)
    t = be.elwise("div", be.elwise("mul", gc, a), be.elwise("mul", b, b))
    gb = be.unbroadcast(t, [n], np.zeros(n, np.float32), [n], -1.0, 1.0)
    return ga, gb


def mul_backward(be, a, b, gc):
    """MulBwd (src/ndtensor.zig:826-847)."""
    n = np.asarray(a).size
    ga = be.unbroadcast(be.elwise("mul", b, gc), [n], np.zeros(n, np.float32), [n], 1.0, 1.0)
    gb = be.unbroadcast(be.elwise("mul", a, gc), [n], np.zeros(n, np.float32), [n], 1.0, 1.0)
    return ga, gb


def gather_dim(be, x, shape, index, index_shape, dim):
    """NDArray.gather (src/ndarray.zig:593-633): offsets on the host, then mem_take."""
    x_str = np.cumprod([1] + list(shape[::-1]))[:-1][::-1]
    offs = []
    for i in range(int(np.prod(index_shape))):
        coord = list(np.unravel_index(i, index_shape))
        coord[dim] = int(index[i])
        assert coord[dim] < shape[dim]
        offs.append(int(np.dot(coord, x_str)))
    return be.take(x, np.asarray(offs, np.uint64))
