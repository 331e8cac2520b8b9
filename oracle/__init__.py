"""ctypes front-end of the CPU oracle (``oracle/host_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke``
and by the CPU-baseline leg of ``bench.py``; never by the product package.

The oracle restates zigrad's HostDevice (BLAS) backend for the training hot
path; its BLAS is the OpenBLAS bundled with SciPy, loaded at run time.
Parity status: pinned against the reference's literal golden vectors
(``tests/golden/``) for GEMM forward/backward, broadcast add/unbroadcast,
sum_along/max_along, gather, clamp, clip-norm, softmax-CE and smooth-L1;
*unpinned* (no test exists in the reference) for SGD/Adam updates,
relu_inplace_bwd, scatter_gcn_deg_scaled and the whole-step drivers.
"""
from __future__ import annotations

import ctypes as C
import glob
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")

f32p = C.POINTER(C.c_float)
u64p = C.POINTER(C.c_ulong)
len_t = C.c_ulong


def build(force: bool = False) -> str:
    """Compile the oracle with g++ (via its Makefile) if it is not built yet."""
    src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("host_oracle.cpp", "steps.inc"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_m:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def _find_openblas() -> str | None:
    try:
        import scipy  # noqa: F401
    except Exception:
        return None
    base = os.path.join(os.path.dirname(os.path.dirname(scipy.__file__)), "scipy.libs")
    hits = sorted(glob.glob(os.path.join(base, "libscipy_openblas*.so")))
    return hits[0] if hits else None


_lib = None
blas_name = "naive-loops"


def lib():
    """Load (building on first use) the oracle library and bind OpenBLAS."""
    global _lib, blas_name
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(_LIB_PATH)
    L.orc_dot.restype = C.c_float
    L.orc_sum.restype = C.c_float
    L.orc_nrm2.restype = C.c_float
    L.orc_softmax_ce_fwd.restype = C.c_float
    L.orc_smooth_l1_fwd.restype = C.c_float
    L.orc_mlp_step.restype = C.c_float
    path = _find_openblas()
    if path is not None and L.orc_blas_init(path.encode()) == 0:
        blas_name = "OpenBLAS (scipy bundled: %s)" % os.path.basename(path)
    _lib = L
    return L


def set_threads(n: int) -> None:
    lib().orc_blas_set_threads(int(n))


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------
def _f(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(f32p)


def _u(a: np.ndarray):
    assert a.dtype == np.uint64 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(u64p)


def _shape(s):
    return (len_t * len(s))(*[int(v) for v in s])


def f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3}


# --------------------------------------------------------------------------
# op wrappers (numpy in, numpy out / in-place)
# --------------------------------------------------------------------------
def elwise(op: str, x, y, z=None) -> np.ndarray:
    x, y = f32(x).ravel(), f32(y).ravel()
    n = max(x.size, y.size)
    if z is None:
        z = np.empty(n, np.float32)
    lib().orc_elwise(OPS[op], _f(x), len_t(x.size), _f(y), len_t(y.size), _f(z), len_t(z.size))
    return z


def matmul(A, B, C_, m, n, k, ta, tb, lda, ldb, ldc, alpha=1.0, beta=0.0) -> np.ndarray:
    lib().orc_matmul(_f(A), _f(B), _f(C_), len_t(m), len_t(n), len_t(k), int(ta), int(tb),
                     len_t(lda), len_t(ldb), len_t(ldc), C.c_float(alpha), C.c_float(beta))
    return C_


def bmm_acc(A, B, C_, A_shape, B_shape, C_shape, ta, tb, lda, ldb, ldc, alpha=1.0, beta=0.0):
    lib().orc_bmm_acc(_f(A), _f(B), _f(C_), _shape(A_shape), _shape(B_shape), _shape(C_shape),
                      int(ta), int(tb), len_t(lda), len_t(ldb), len_t(ldc),
                      C.c_float(alpha), C.c_float(beta))
    return C_


def bmm(A: np.ndarray, B: np.ndarray, ta=False, tb=False, alpha=1.0, beta=0.0, C_=None):
    """NDArray.bmm_acc_impl's shape logic (ndarray.zig:817-899) over numpy
    arrays: derives batch dims, M/N/K and leading dimensions, then calls the
    device op."""
    A, B = f32(A), f32(B)
    a_shape = A.shape if A.ndim >= 2 else (1,) + A.shape
    b_shape = B.shape if B.ndim >= 2 else (1,) + B.shape
    a_batch = a_shape[:-2] if len(a_shape) > 2 else (1,)
    b_batch = b_shape[:-2] if len(b_shape) > 2 else (1,)
    if len(a_shape) == 2 and len(b_shape) == 2:
        bb = ()
    else:
        bb = np.broadcast_shapes(a_batch, b_batch)
    a_rows, a_cols = a_shape[-2:]
    b_rows, b_cols = b_shape[-2:]
    M = a_cols if ta else a_rows
    K = a_rows if ta else a_cols
    N = b_rows if tb else b_cols
    c_shape = tuple(bb) + (M, N)
    if C_ is None:
        C_ = np.zeros(c_shape, np.float32)
    nA, nB, nC = int(np.prod(a_batch)), int(np.prod(b_batch)), int(np.prod(bb)) if bb else 1
    bmm_acc(A, B, C_, (nA, M, K), (nB, K, N), (nC, M, N), ta, tb, a_cols, b_cols, N, alpha, beta)
    return C_


def axpy(x, y, alpha):
    lib().orc_axpy(_f(x), _f(y), len_t(x.size), C.c_float(alpha))
    return y


def dot(x, y) -> float:
    return float(lib().orc_dot(_f(x), _f(y), len_t(x.size)))


def asum(x) -> float:
    return float(lib().orc_sum(_f(x), len_t(x.size)))


def nrm2(x) -> float:
    return float(lib().orc_nrm2(_f(x), len_t(x.size)))


def scale(x, alpha):
    lib().orc_scale(_f(x), len_t(x.size), C.c_float(alpha))
    return x


def clip_nrm2(x, max_norm, delta):
    lib().orc_clip_nrm2(_f(x), len_t(x.size), C.c_float(max_norm), C.c_float(delta))
    return x


def transpose(A, B, m, n, alpha):
    lib().orc_transpose(_f(A), _f(B), len_t(m), len_t(n), C.c_float(alpha))
    return B


def matvec(A, x, y, m, n, ta, alpha, beta):
    lib().orc_matvec(_f(A), _f(x), _f(y), len_t(m), len_t(n), int(ta), C.c_float(alpha), C.c_float(beta))
    return y


def unary(name: str, x, y=None):
    """relu_fwd / exp_fwd / sqrt_fwd / tanh_fwd / sigm_fwd: y = f(x)."""
    if y is None:
        y = np.empty_like(x)
    getattr(lib(), "orc_" + name)(_f(x), _f(y), len_t(x.size))
    return y


def relu_bwd(x, x_g, y_g):
    lib().orc_relu_bwd(_f(x), _f(x_g), _f(y_g), len_t(x.size))
    return x_g


def relu_inplace_bwd(x, x_g):
    lib().orc_relu_inplace_bwd(_f(x), _f(x_g), len_t(x.size))
    return x_g


def clamp_fwd(x, lo, hi, y=None):
    if y is None:
        y = np.empty_like(x)
    lib().orc_clamp_fwd(_f(x), _f(y), len_t(x.size), C.c_float(lo), C.c_float(hi))
    return y


def clamp_bwd(x, x_g, y_g, lo, hi):
    lib().orc_clamp_bwd(_f(x), _f(x_g), _f(y_g), len_t(x.size), C.c_float(lo), C.c_float(hi))
    return x_g


def bwd3(name: str, x_g, y, y_g):
    """exp_bwd / tanh_bwd / sigm_bwd: x_g += f'(y) * y_g."""
    getattr(lib(), "orc_" + name)(_f(x_g), _f(y), _f(y_g), len_t(y.size))
    return x_g


def inplace_bwd(name: str, x, x_g):
    """tanh_inplace_bwd / sigm_inplace_bwd: x_g *= f'(x), x the activation's output."""
    getattr(lib(), "orc_" + name)(_f(x), _f(x_g), len_t(x.size))
    return x_g


def pow_fwd(x, e, y=None):
    if y is None:
        y = np.empty_like(x)
    lib().orc_pow_fwd(_f(x), _f(y), len_t(x.size), C.c_float(e))
    return y


def pow_bwd(x, x_g, y_g, e, eps):
    lib().orc_pow_bwd(_f(x), _f(x_g), _f(y_g), len_t(x.size), C.c_float(e), C.c_float(eps))
    return x_g


def _m(a: np.ndarray):
    assert a.dtype == np.uint8 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.POINTER(C.c_ubyte))


def relu_mask_fwd(x):
    """In place on x; returns the byte mask (ceil(n/8) bytes)."""
    mask = np.zeros((x.size + 7) // 8, np.uint8)
    lib().orc_relu_mask_fwd(_f(x), _m(mask), len_t(x.size))
    return mask


def relu_mask_bwd(x_g, mask):
    lib().orc_relu_mask_bwd(_f(x_g), _m(mask), len_t(x_g.size))
    return x_g


def clamp_mask_fwd(x, lo, hi):
    y = np.empty_like(x)
    mask = np.zeros((x.size + 7) // 8, np.uint8)
    lib().orc_clamp_mask_fwd(_f(x), _f(y), _m(mask), len_t(x.size), C.c_float(lo), C.c_float(hi))
    return y, mask


def clamp_mask_bwd(x_g, y_g, mask):
    lib().orc_clamp_mask_bwd(_f(x_g), _f(y_g), _m(mask), len_t(x_g.size))
    return x_g


def scatter_add_2d(src, indices, dst, stride):
    lib().orc_scatter_add_2d(_f(src), _u(indices), len_t(indices.size), len_t(stride), _f(dst))
    return dst


def scatter_add_csr(src, row_ptr, dst):
    lib().orc_scatter_add_csr(_f(src), _u(row_ptr), len_t(src.size), _f(dst))
    return dst


def segment_sum_csr(src, row_offsets):
    dst = np.zeros(row_offsets.size - 1, np.float32)
    lib().orc_segment_sum_csr(_f(src), _u(row_offsets), len_t(dst.size), _f(dst))
    return dst


def rsqrt_fwd(x, eps, y=None):
    if y is None:
        y = np.empty_like(x)
    lib().orc_rsqrt_fwd(_f(x), _f(y), len_t(x.size), C.c_float(eps))
    return y


def rsqrt_bwd(x, x_g, y_g, eps):
    lib().orc_rsqrt_bwd(_f(x), _f(x_g), _f(y_g), len_t(x.size), C.c_float(eps))
    return x_g


def sqrt_bwd(x, x_g, y_g, eps):
    lib().orc_sqrt_bwd(_f(x), _f(x_g), _f(y_g), len_t(x.size), C.c_float(eps))
    return x_g


def max_fwd(x):
    y = np.zeros(1, np.float32)
    lib().orc_max_fwd(_f(x), _f(y), len_t(x.size))
    return y


def max_bwd(x, x_g, y, y_g):
    lib().orc_max_bwd(_f(x), _f(x_g), _f(y), _f(y_g), len_t(x.size))
    return x_g


def fold_rows(x, y, row, col, alpha=1.0, beta=0.0):
    lib().orc_fold_rows(_f(x), _f(y), len_t(row), len_t(col), C.c_float(alpha), C.c_float(beta))
    return y


def fold_cols(x, y, row, col, alpha=1.0, beta=0.0):
    lib().orc_fold_cols(_f(x), _f(y), len_t(row), len_t(col), C.c_float(alpha), C.c_float(beta))
    return y


def sum_along(x, x_shape, dim, y=None, alpha=1.0, beta=0.0):
    ys = list(x_shape)
    ys[dim] = 1
    if y is None:
        y = np.zeros(int(np.prod(ys)), np.float32)
    lib().orc_sum_along(_f(x), _shape(x_shape), len_t(len(x_shape)), _f(y), len_t(y.size),
                        len_t(dim), C.c_float(alpha), C.c_float(beta))
    return y


def max_along(x, x_shape, dim, y=None):
    ys = list(x_shape)
    ys[dim] = 1
    if y is None:
        y = np.zeros(int(np.prod(ys)), np.float32)
    lib().orc_max_along(_f(x), _shape(x_shape), len_t(len(x_shape)), _f(y), len_t(y.size), len_t(dim))
    return y


def unbroadcast_scratch_len(x_shape, y_shape) -> int:
    """Scratch sizing rule of NDArray.unbroadcast_ (ndarray.zig:697-715)."""
    x_shape, y_shape = list(x_shape), list(y_shape)
    xsz, ysz = int(np.prod(x_shape)), int(np.prod(y_shape))
    delta = len(x_shape) - len(y_shape)
    if delta > 0:
        coef = int(np.prod(x_shape[:delta]))
    else:
        mm = [i for i, (a, b) in enumerate(zip(x_shape, y_shape)) if a != b]
        if not mm:
            return 0
        coef = x_shape[mm[0]]
    n = ysz * coef
    return 0 if n == xsz else n


class ReferenceOutOfBounds(RuntimeError):
    """The reference's algorithm would write past an output for these shapes."""


def unbroadcast(x, x_shape, y, y_shape, alpha=1.0, beta=0.0):
    # the reference's own sizing rule (unbroadcast_scratch_len) under-allocates
    # when a leading fold is followed by an interior reduction; give the C
    # restatement room for the largest intermediate instead of overflowing
    n = max(unbroadcast_scratch_len(x_shape, y_shape), int(np.prod(x_shape)))
    scratch = np.zeros(max(n, 1), np.float32)
    rc = lib().orc_unbroadcast(_f(x), _shape(x_shape), len_t(len(x_shape)), _f(y), _shape(y_shape),
                               len_t(len(y_shape)), _f(scratch), C.c_float(alpha), C.c_float(beta))
    if rc == 2:
        raise ReferenceOutOfBounds("unbroadcast %s -> %s: the host code drops y's trailing ones and mis-aligns (or overruns) y" % (list(x_shape), list(y_shape)))
    assert rc == 0
    return y


def broadcast(x, y, alpha=1.0, beta=0.0):
    lib().orc_broadcast(_f(x), len_t(x.size), _f(y), len_t(y.size), C.c_float(alpha), C.c_float(beta))
    return y


def take(src, idx, dst=None):
    if dst is None:
        dst = np.empty(idx.size, np.float32)
    lib().orc_take(_f(src), _u(idx), len_t(idx.size), _f(dst))
    return dst


def scatter_add(src, offs, dst):
    lib().orc_scatter_add(_f(src), _u(offs), len_t(src.size), _f(dst))
    return dst


def scatter_gcn_deg_scaled(dst, h, deg, src_idx, tgt_idx, stride):
    lib().orc_scatter_gcn_deg_scaled(_f(dst), _f(h), _f(deg), _u(src_idx), _u(tgt_idx),
                                     len_t(stride), len_t(src_idx.size))
    return dst


def scatter_gcn_deg_scaled_bwd(grad_out, h, deg, src_idx, tgt_idx, grad_h, grad_deg, stride):
    lib().orc_scatter_gcn_deg_scaled_bwd(_f(grad_out), _f(h), _f(deg), _u(src_idx), _u(tgt_idx),
                                         _f(grad_h), _f(grad_deg), len_t(stride), len_t(src_idx.size))
    return grad_h, grad_deg


def softmax_ce_fwd(logits, target, batch=None):
    logits, target = f32(logits), f32(target)
    if logits.ndim == 1:
        rows, Cc = 1, logits.shape[0]
    else:
        rows, Cc = logits.shape
    if batch is None:
        batch = rows
    sm = np.empty((rows, Cc), np.float32)
    loss = lib().orc_softmax_ce_fwd(_f(logits), _f(target), _f(sm), len_t(rows), len_t(Cc), len_t(batch))
    return float(np.float32(loss)), sm


def softmax_ce_bwd(sm, target, grad, batch):
    lib().orc_softmax_ce_bwd(_f(sm), _f(f32(target)), _f(grad), len_t(sm.size), len_t(batch))
    return grad


def smooth_l1_fwd(pred, target, beta) -> float:
    return float(lib().orc_smooth_l1_fwd(_f(pred), _f(target), len_t(pred.size), C.c_float(beta)))


def smooth_l1_bwd(pred, target, grad, beta):
    lib().orc_smooth_l1_bwd(_f(pred), _f(target), _f(grad), len_t(pred.size), C.c_float(beta))
    return grad


def sgd_update(p, g, lr, clip=False, max_norm=10.0, delta=1e-6):
    lib().orc_sgd_update(_f(p), _f(g), len_t(p.size), C.c_double(lr), int(clip),
                         C.c_float(max_norm), C.c_float(delta))
    return p


def adam_update(p, g, m, v, lr, beta1, beta2, eps, t, clip=False, max_norm=10.0, delta=1e-6):
    lib().orc_adam_update(_f(p), _f(g), _f(m), _f(v), len_t(p.size), C.c_double(lr), C.c_double(beta1),
                          C.c_double(beta2), C.c_double(eps), len_t(t), int(clip),
                          C.c_float(max_norm), C.c_float(delta))
    return p


def round_bf16(x):
    y = np.empty_like(x)
    lib().orc_round_bf16(_f(x), _f(y), len_t(x.size))
    return y


# --------------------------------------------------------------------------
# step drivers
# --------------------------------------------------------------------------
def _pp(arrs):
    return (f32p * len(arrs))(*[_f(a) for a in arrs])


class MlpOracle:
    """State + one-step driver for an MLP (Linear+ReLU ... Linear) trained with
    softmax cross-entropy, as examples/mnist/src/model.zig builds it."""

    def __init__(self, dims, weights, biases, opt="sgd", lr=0.01, beta1=0.9, beta2=0.999,
                 eps=1e-8, clip=False, max_norm=10.0, delta=1e-6):
        self.dims = [int(d) for d in dims]
        self.L = len(dims) - 1
        self.W = [f32(w).copy() for w in weights]
        self.b = [f32(x).copy() for x in biases]
        self.dW = [np.zeros_like(w) for w in self.W]
        self.db = [np.zeros_like(x) for x in self.b]
        self.opt = {"none": -1, "sgd": 0, "adam": 1}[opt]
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.clip, self.max_norm, self.delta = clip, max_norm, delta
        self.m = [np.zeros(a.size, np.float32) for pair in zip(self.W, self.b) for a in pair]
        self.v = [np.zeros(a.size, np.float32) for pair in zip(self.W, self.b) for a in pair]
        self.t = len_t(0)
        self.act = self.dact = self.sm = None

    def step(self, X, T, loss_div=None, update=True) -> float:
        X, T = f32(X), f32(T)
        B = X.shape[0]
        if self.act is None or self.act[0].shape[0] != B:
            self.act = [np.zeros((B, self.dims[l + 1]), np.float32) for l in range(self.L)]
            self.dact = [np.zeros((B, self.dims[l + 1]), np.float32) for l in range(self.L)]
            self.sm = np.zeros((B, self.dims[-1]), np.float32)
        loss = lib().orc_mlp_step(
            self.L, _shape(self.dims), _pp(self.W), _pp(self.b), _pp(self.dW), _pp(self.db),
            _f(X), _f(T), len_t(B), _pp(self.act), _pp(self.dact), _f(self.sm),
            len_t(loss_div if loss_div is not None else B), self.opt if update else -1,
            C.c_double(self.lr), C.c_double(self.beta1), C.c_double(self.beta2), C.c_double(self.eps),
            _pp(self.m), _pp(self.v), C.byref(self.t), int(self.clip),
            C.c_float(self.max_norm), C.c_float(self.delta), 0, None)
        return float(np.float32(loss))
