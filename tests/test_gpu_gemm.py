"""GEMM parity through zg_bmm / the bmm_acc op: the tcgen05 kernel in its
three math modes and the FFMA kernel, all four transpose combinations, the
training shapes of the benchmark configurations, ragged shapes, alpha/beta,
batch broadcast, fused epilogues and split-K.

Tolerances (max |got-want| / max |want| per tensor, oracle = OpenBLAS sgemm):
  FFMA                       1e-5
  FP32X3 (3xTF32)            3e-5   (both inside the 1e-4 the hot path is held to)
  TF32 single pass           2e-3   (stated separately, as the spec allows)
  BF16 inputs, fp32 output   1e-5 against the oracle on bf16-rounded inputs
  BF16 output                4e-3   (one bf16 rounding of the result)
"""
import numpy as np
import pytest

import oracle
from zigrad_b200 import abi, opspec
from zigrad_b200.abi import BF16, SINGLE

from .backends import GpuBackend, OracleBackend
from .test_gpu_ops import rel_err, rng

pytestmark = pytest.mark.gpu
ORC = OracleBackend()

# FP32X3: the split itself is good to ~1e-6; what remains is the tensor core's
# fp32 accumulator, which truncates instead of rounding to nearest, a bias that
# grows with the number of accumulation steps (observed 1.3e-5 at k = 1433).
MODES = {"ffma": (abi.MATH_FFMA, 1e-5), "fp32x3": (abi.MATH_FP32X3, 3e-5), "tf32": (abi.MATH_TF32, 2e-3)}
TRANS = {"NN": (False, False), "NT": (False, True), "TN": (True, False), "TT": (True, True)}

# (m, n, k): the MLP / GCN / DQN GEMMs plus ragged cases
SHAPES = [
    (64, 128, 784), (64, 64, 128), (64, 10, 64),          # config 1 forward
    (128, 784, 64), (64, 128, 128),                        # config 1 dW / dX
    (1024, 128, 784), (128, 784, 1024), (1024, 64, 10),    # config 2 per-GPU shard sizes
    (2708, 16, 1433), (2708, 16, 2708), (16, 1433, 2708),  # GCN
    (256, 128, 4), (256, 2, 128),                          # DQN
    (1, 1, 1), (5, 3, 2), (129, 65, 33), (255, 130, 257), (128, 128, 32), (300, 200, 100),
]


def run_gemm(gpu, mode, m, n, k, ta, tb, alpha=1.0, beta=0.0, seed=0, lda_pad=0):
    g = rng(seed + m * 3 + n * 5 + k * 7)
    a_shape = (k, m) if ta else (m, k)
    b_shape = (n, k) if tb else (k, n)
    A = g.standard_normal(a_shape).astype(np.float32)
    B = g.standard_normal(b_shape).astype(np.float32)
    C0 = g.standard_normal((m, n)).astype(np.float32)
    lda, ldb = a_shape[1], b_shape[1]
    gpu.L.zg_set_math_mode(mode)
    try:
        got = GpuBackend(gpu).bmm_acc(A, B, C0, (1, m, k), (1, k, n), (1, m, n), ta, tb, lda, ldb, n, alpha, beta)
    finally:
        gpu.L.zg_set_math_mode(abi.MATH_FP32X3)
    want = ORC.bmm_acc(A, B, C0, (1, m, k), (1, k, n), (1, m, n), ta, tb, lda, ldb, n, alpha, beta)
    return got, want


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("trans", list(TRANS))
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_modes_transposes_shapes(gpu, mode, trans, shape):
    m, n, k = shape
    ta, tb = TRANS[trans]
    got, want = run_gemm(gpu, MODES[mode][0], m, n, k, ta, tb)
    assert rel_err(got, want) <= MODES[mode][1], (mode, trans, shape, rel_err(got, want))


@pytest.mark.parametrize("mode", ["ffma", "fp32x3"])
@pytest.mark.parametrize("alpha,beta", [(1.0, 1.0), (2.0, 3.0), (-0.5, 0.0), (0.0, 1.0)])
def test_gemm_alpha_beta(gpu, mode, alpha, beta):
    for (m, n, k, ta, tb) in [(128, 784, 1024, True, False), (256, 128, 128, False, True), (77, 33, 65, False, False)]:
        got, want = run_gemm(gpu, MODES[mode][0], m, n, k, ta, tb, alpha, beta, seed=3)
        assert rel_err(got, want) <= MODES[mode][1], (m, n, k, rel_err(got, want))


@pytest.mark.parametrize("mode", ["ffma", "fp32x3", "tf32"])
def test_gemm_split_k_weight_gradient_shapes(gpu, mode):
    # dW = dY^T . X with k = batch: few output tiles, very deep k -> split-K path
    for (m, n, k) in [(128, 784, 8192), (64, 128, 8192), (10, 64, 8192), (16, 1433, 2708)]:
        got, want = run_gemm(gpu, MODES[mode][0], m, n, k, True, False, 1.0, 1.0, seed=5)
        assert rel_err(got, want) <= MODES[mode][1], (mode, m, n, k, rel_err(got, want))


@pytest.mark.parametrize("budget", [1, 15, 22, 126, 133, 1000])
def test_weight_gradient_with_a_share_of_the_sms(gpu, budget):
    """zg_bmm_sm_budget only changes how many K ranges the split-K grid has: the result stays the
    product (the guard regions around the operands catch a range that runs past k)."""
    g = rng(budget)
    for (m, n, k) in [(128, 784, 8192), (64, 128, 8192), (128, 784, 1000)]:
        A = g.standard_normal((k, m)).astype(np.float32)
        B = g.standard_normal((k, n)).astype(np.float32)
        C0 = g.standard_normal((m, n)).astype(np.float32)
        got = GpuBackend(gpu).linear(A, B, C0, m, n, k, True, False, m, n, n, 1.0, 1.0, "none", sm_budget=budget)
        want = ORC.bmm_acc(A, B, C0, (1, m, k), (1, k, n), (1, m, n), True, False, m, n, n, 1.0, 1.0)
        # 1e-4, the bound of the hot path: with a budget of one SM the 8192 products of an element are
        # accumulated in ONE tensor-memory accumulator, whose truncation bias grows with the number of steps
        assert rel_err(got, want) <= 1e-4, (budget, m, n, k, rel_err(got, want))
    # the budget is consumed by one call: the next product is sized for the whole GPU again
    assert gpu.sm_count() >= 1


@pytest.mark.parametrize("m,n,k,ldc", [(128, 64, 96, 64), (130, 68, 100, 68), (1, 36, 64, 36), (257, 100, 784, 104), (8192, 128, 784, 128),
                                       (97, 32, 33, 40)])
@pytest.mark.parametrize("epilogue", ["none", "bias", "bias_relu"])
def test_output_through_the_tensor_map_on_ragged_edges(gpu, m, n, k, ldc, epilogue):
    """Forward products whose output leaves through the C tensor map (beta = 0, fp32, 16-byte-aligned
    rows): tiles that hang over the last rows / columns are clipped by the TMA unit, the padding
    columns of a wider row stride keep their contents."""
    g = rng(m + n + k)
    A = g.standard_normal((m, k)).astype(np.float32)
    B = g.standard_normal((n, k)).astype(np.float32)
    bias = g.standard_normal(n).astype(np.float32)
    C0 = np.full((m, ldc), 7.0, np.float32)
    lda = ldb = k if k % 4 == 0 else None
    if lda is None:  # rows of A / B must be 16-byte aligned for the tensor maps: pad k's stride
        kp = (k + 3) // 4 * 4
        Ap, Bp = np.zeros((m, kp), np.float32), np.zeros((n, kp), np.float32)
        Ap[:, :k], Bp[:, :k] = A, B
        A_, B_, lda, ldb = Ap, Bp, kp, kp
    else:
        A_, B_ = A, B
    got = GpuBackend(gpu).linear(A_, B_, C0, m, n, k, False, True, lda, ldb, ldc, 1.0, 0.0, epilogue, bias if epilogue != "none" else None)
    want = A.astype(np.float64) @ B.T.astype(np.float64)
    if epilogue != "none":
        want = want + bias[None, :]
    if epilogue == "bias_relu":
        want = np.maximum(want, 0)
    assert rel_err(got[:, :n], want) <= 3e-5, rel_err(got[:, :n], want)
    assert (got[:, n:] == 7.0).all()  # nothing written beyond column n


@pytest.mark.parametrize("mode", ["ffma", "fp32x3"])
def test_bmm_batch_broadcast(gpu, mode):
    g = rng(17)
    gpu.L.zg_set_math_mode(MODES[mode][0])
    try:
        for (nA, nB, nC, m, n, k) in [(4, 2, 4, 130, 66, 40), (1, 3, 3, 64, 64, 64), (3, 1, 3, 200, 36, 72)]:
            A = g.standard_normal((nA, m, k)).astype(np.float32)
            B = g.standard_normal((nB, k, n)).astype(np.float32)
            C0 = np.zeros((nC, m, n), np.float32)
            got = GpuBackend(gpu).bmm_acc(A, B, C0, (nA, m, k), (nB, k, n), (nC, m, n), False, False, k, n, n, 1.0, 0.0)
            want = ORC.bmm_acc(A, B, C0, (nA, m, k), (nB, k, n), (nC, m, n), False, False, k, n, n, 1.0, 0.0)
            assert rel_err(got, want) <= 1e-5
    finally:
        gpu.L.zg_set_math_mode(abi.MATH_FP32X3)


@pytest.mark.parametrize("mode", ["ffma", "fp32x3"])
@pytest.mark.parametrize("m,n,k", [(64, 128, 784), (1024, 64, 128), (1024, 10, 64), (33, 17, 9), (2708, 16, 2708), (200, 100, 3000)])
def test_linear_fused_epilogues_equal_separate_ops(gpu, mode, m, n, k):
    """bias / bias+ReLU / ReLU-mask epilogues against the reference's separate
    device calls (bmm_acc, add, relu_fwd; relu_inplace_bwd) run by the oracle."""
    g = rng(m + n + k)
    X, W, b = g.standard_normal((m, k)).astype(np.float32), g.standard_normal((n, k)).astype(np.float32), g.standard_normal(n).astype(np.float32)
    gpu.L.zg_set_math_mode(MODES[mode][0])
    try:
        be = GpuBackend(gpu)
        z = ORC.bmm_acc(X, W, np.zeros((m, n), np.float32), (1, m, k), (1, k, n), (1, m, n), False, True, k, k, n, 1.0, 0.0)
        zb = ORC.elwise("add", b, z.ravel()).reshape(m, n)
        got = be.linear(X, W, np.zeros((m, n), np.float32), m, n, k, False, True, k, k, n, 1.0, 0.0, "bias", bias=b)
        assert rel_err(got, zb) <= 1e-5
        act = ORC.relu_fwd(zb.ravel()).reshape(m, n)
        got = be.linear(X, W, np.zeros((m, n), np.float32), m, n, k, False, True, k, k, n, 1.0, 0.0, "bias_relu", bias=b)
        assert rel_err(got, act) <= 1e-5
        assert np.array_equal(got > 0, act > 0) or rel_err(got, act) <= 1e-6
        # dX = dY . W masked by the previous activation (mask has dX's shape [m, k])
        dY, prev = g.standard_normal((m, n)).astype(np.float32), g.standard_normal((m, k)).astype(np.float32)
        prev = np.maximum(prev, 0)
        dx = ORC.bmm_acc(dY, W, np.zeros((m, k), np.float32), (1, m, n), (1, n, k), (1, m, k), False, False, n, k, k, 1.0, 1.0)
        dx = ORC.relu_inplace_bwd(prev.ravel(), dx.ravel()).reshape(m, k)
        got = be.linear(dY, W, np.zeros((m, k), np.float32), m, k, n, False, False, n, k, k, 1.0, 0.0, "relu_mask", mask=prev)
        assert rel_err(got, dx) <= 1e-5
        np.testing.assert_array_equal(got == 0, dx == 0)
    finally:
        gpu.L.zg_set_math_mode(abi.MATH_FP32X3)


@pytest.mark.parametrize("mode", ["ffma", "fp32x3"])
@pytest.mark.parametrize("m,n,k", [(8192, 128, 64), (1024, 64, 12), (300, 100, 40), (33, 17, 9), (300, 100, 2048), (2708, 16, 1536)])
def test_gemm_epilogue_column_sums_are_the_bias_gradient(gpu, mode, m, n, k):
    """dX GEMM with the ReLU mask AND the column sums of what it stores, added to
    a pre-existing vector: equals relu_inplace_bwd followed by unbroadcast
    (alpha = beta = 1) on the oracle."""
    g = rng(m * 2 + n + k)
    dY, W = g.standard_normal((m, k)).astype(np.float32), g.standard_normal((k, n)).astype(np.float32)
    prev = np.maximum(g.standard_normal((m, n)).astype(np.float32), 0)
    db0 = g.standard_normal(n).astype(np.float32)
    dx = ORC.bmm_acc(dY, W, np.zeros((m, n), np.float32), (1, m, k), (1, k, n), (1, m, n), False, False, k, n, n, 1.0, 0.0)
    dx = ORC.relu_inplace_bwd(prev.ravel(), dx.ravel()).reshape(m, n)
    want_db = ORC.unbroadcast(dx.ravel(), [m, n], db0, [n], 1.0, 1.0)
    gpu.L.zg_set_math_mode(MODES[mode][0])
    try:
        got, sums = GpuBackend(gpu).linear(dY, W, np.zeros((m, n), np.float32), m, n, k, False, False, k, n, n, 1.0, 0.0,
                                           "relu_mask", mask=prev, colsum=db0)
    finally:
        gpu.L.zg_set_math_mode(abi.MATH_FP32X3)
    assert rel_err(got, dx) <= MODES[mode][1]
    assert rel_err(sums, want_db) <= 3e-5, rel_err(sums, want_db)


@pytest.mark.parametrize("m,n,k,tb", [(8192, 10, 64, True), (5003, 7, 16, False), (1000, 16, 512, True), (3001, 13, 100, True),
                                      (8192, 64, 10, False), (4097, 256, 16, False), (999, 20, 3, True), (2050, 128, 7, False)])
def test_short_dimension_gemms(gpu, m, n, k, tb):
    """The FFMA kernels for n <= 16 or k <= 16 (the classifier layer forward and
    backward): plain product with alpha/beta where the kernel takes it, and the
    bias + ReLU epilogue, against the oracle's sgemm."""
    g = rng(m + 31 * n + 7 * k)
    A = g.standard_normal((m, k)).astype(np.float32)
    B = g.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    C0 = g.standard_normal((m, n)).astype(np.float32)
    b = g.standard_normal(n).astype(np.float32)
    ldb = k if tb else n
    be = GpuBackend(gpu)
    for alpha, beta in ((1.0, 0.0), (-0.5, 2.0)):
        got = be.bmm_acc(A, B, C0, (1, m, k), (1, k, n), (1, m, n), False, tb, k, ldb, n, alpha, beta)
        want = ORC.bmm_acc(A, B, C0, (1, m, k), (1, k, n), (1, m, n), False, tb, k, ldb, n, alpha, beta)
        assert rel_err(got, want) <= 1e-5, (alpha, beta, rel_err(got, want))
    z = ORC.bmm_acc(A, B, np.zeros((m, n), np.float32), (1, m, k), (1, k, n), (1, m, n), False, tb, k, ldb, n, 1.0, 0.0)
    act = ORC.relu_fwd(ORC.elwise("add", b, z.ravel())).reshape(m, n)
    got = be.linear(A, B, np.zeros((m, n), np.float32), m, n, k, False, tb, k, ldb, n, 1.0, 0.0, "bias_relu", bias=b)
    assert rel_err(got, act) <= 1e-5


@pytest.mark.parametrize("m,n,k", [(10, 64, 8192), (16, 128, 4096), (3, 256, 2000), (7, 32, 1024)])
@pytest.mark.parametrize("beta", [1.0, 0.0, 0.5])
def test_narrow_weight_gradient(gpu, m, n, k, beta):
    """dW = dY^T X for a layer with at most 16 outputs (A stored [k, m], B stored
    [k, n], deep k): the FFMA kernel that folds k blocks with atomics."""
    g = rng(m * 5 + n + k)
    A = g.standard_normal((k, m)).astype(np.float32)
    B = g.standard_normal((k, n)).astype(np.float32)
    C0 = g.standard_normal((m, n)).astype(np.float32)
    got = GpuBackend(gpu).bmm_acc(A, B, C0, (1, m, k), (1, k, n), (1, m, n), True, False, m, n, n, 1.0, beta)
    want = ORC.bmm_acc(A, B, C0, (1, m, k), (1, k, n), (1, m, n), True, False, m, n, n, 1.0, beta)
    assert rel_err(got, want) <= 1e-5, rel_err(got, want)


def to_bf16_bits(x):
    return (oracle.round_bf16(np.ascontiguousarray(x, np.float32).ravel()).view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("trans", list(TRANS))
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (1024, 512, 384), (300, 200, 100), (128, 1000, 512), (64, 64, 64)])
@pytest.mark.parametrize("c_bf16", [False, True])
def test_gemm_bf16_inputs(gpu, trans, m, n, k, c_bf16):
    ta, tb = TRANS[trans]
    g = rng(m + 2 * n + 3 * k)
    a_shape, b_shape = ((k, m) if ta else (m, k)), ((n, k) if tb else (k, n))
    A, B = g.standard_normal(a_shape).astype(np.float32), g.standard_normal(b_shape).astype(np.float32)
    Ar, Br = oracle.round_bf16(A.ravel()).reshape(a_shape), oracle.round_bf16(B.ravel()).reshape(b_shape)
    want = ORC.bmm_acc(Ar, Br, np.zeros((m, n), np.float32), (1, m, k), (1, k, n), (1, m, n), ta, tb, a_shape[1], b_shape[1], n, 1.0, 0.0)
    be = GpuBackend(gpu)
    a, b = be.up(to_bf16_bits(A), np.uint16), be.up(to_bf16_bits(B), np.uint16)
    c = be.up(np.zeros(m * n, np.uint16), np.uint16) if c_bf16 else be.up(np.zeros(m * n, np.float32))
    gpu.dispatch(opspec.linear(a, b, c, m, n, k, ta, tb, a_shape[1], b_shape[1], n))
    out = be.down(c)
    if c_bf16:
        out = (out.astype(np.uint32) << 16).view(np.float32)
    assert rel_err(out.reshape(m, n), want) <= (4e-3 if c_bf16 else 1e-5), rel_err(out.reshape(m, n), want)


def test_persistent_gemm_at_the_wide_mlp_shape_against_openblas(gpu):
    """8192 x 4096 x 4096, NT, bf16 operands, fp32 result: the forward GEMM of the wide
    MLP's hidden layers on the persistent 128x256-tile kernel, every element against the
    CPU oracle (OpenBLAS sgemm on the bf16-rounded operands)."""
    m, n, k = 8192, 4096, 4096
    import os
    oracle.set_threads(os.cpu_count() or 1)
    g = rng(8192)
    A, B = g.standard_normal((m, k)).astype(np.float32), g.standard_normal((n, k)).astype(np.float32)
    Ar, Br = oracle.round_bf16(A.ravel()).reshape(m, k), oracle.round_bf16(B.ravel()).reshape(n, k)
    want = ORC.bmm_acc(Ar, Br, np.zeros((m, n), np.float32), (1, m, k), (1, k, n), (1, m, n), False, True, k, k, n, 1.0, 0.0)
    be = GpuBackend(gpu)
    a, b = be.up(to_bf16_bits(A), np.uint16), be.up(to_bf16_bits(B), np.uint16)
    c = be.up(np.zeros(m * n, np.float32))
    gpu.dispatch(opspec.linear(a, b, c, m, n, k, False, True, k, k, n))
    out = be.down(c).reshape(m, n)
    # exact bf16 products, fp32 accumulation in a different order than the host's: k = 4096 terms
    assert rel_err(out, want) <= 2e-5, rel_err(out, want)


def test_gemm_double_precision_ffma(gpu):
    g = rng(99)
    A, B = g.standard_normal((70, 50)), g.standard_normal((50, 30))
    a, b = gpu.from_numpy(A), gpu.from_numpy(B)
    c = gpu.from_numpy(np.zeros(70 * 30))
    gpu.dispatch(opspec.bmm_acc(a, b, c, (1, 70, 50), (1, 50, 30), (1, 70, 30), False, False, 50, 30, 30, 1.0, 0.0))
    np.testing.assert_allclose(gpu.to_numpy(c, (70, 30)), A @ B, rtol=1e-12, atol=1e-12)
    for s in (a, b, c):
        gpu.mem_cache_free(s)


def test_large_gemm_linearity_property(gpu):
    """Size-independent check at a size the CPU oracle would take long on:
    (A1 + A2) B == A1 B + A2 B to fp32x3 accuracy, 4096^3."""
    n = 4096
    be = GpuBackend(gpu)
    d = gpu
    A1, A2, B = (d.mem_cache_alloc(SINGLE, n * n) for _ in range(3))
    for i, s in enumerate((A1, A2, B)):
        d.mem_random(s, "normal", 100 + i)
    S = d.mem_cache_alloc(SINGLE, n * n)
    d.dispatch(opspec.add(A1, A2, S))
    C1, C2 = d.mem_cache_alloc(SINGLE, n * n), d.mem_cache_alloc(SINGLE, n * n)
    mk = lambda a, c, beta: opspec.bmm_acc(a, B, c, (1, n, n), (1, n, n), (1, n, n), False, False, n, n, n, 1.0, beta)
    d.dispatch(mk(S, C1, 0.0))
    d.dispatch(mk(A1, C2, 0.0))
    d.dispatch(mk(A2, C2, 1.0))
    c1, c2 = d.to_numpy(C1), d.to_numpy(C2)
    assert rel_err(c1, c2) <= 2e-5
    for s in (A1, A2, B, S, C1, C2):
        d.mem_cache_free(s)


# ---------------------------------------------------------------- persistent kernel
# Shapes with at least one 128 x 256 tile per SM take the persistent kernel
# (bf16 and single-pass TF32): 40 x 4 = 160 tiles, ragged m / n / k edges.
PERSISTENT_SHAPES = [(5120, 1024, 512), (5000, 1000, 520)]


@pytest.mark.parametrize("trans", list(TRANS))
@pytest.mark.parametrize("shape", PERSISTENT_SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("c_bf16", [False, True])
def test_persistent_gemm_bf16(gpu, trans, shape, c_bf16):
    m, n, k = shape
    ta, tb = TRANS[trans]
    g = rng(m + 2 * n + 3 * k + 1)
    a_shape, b_shape = ((k, m) if ta else (m, k)), ((n, k) if tb else (k, n))
    A, B = g.standard_normal(a_shape).astype(np.float32), g.standard_normal(b_shape).astype(np.float32)
    Ar, Br = oracle.round_bf16(A.ravel()).reshape(a_shape), oracle.round_bf16(B.ravel()).reshape(b_shape)
    want = ORC.bmm_acc(Ar, Br, np.zeros((m, n), np.float32), (1, m, k), (1, k, n), (1, m, n), ta, tb, a_shape[1], b_shape[1], n, 1.0, 0.0)
    be = GpuBackend(gpu)
    a, b = be.up(to_bf16_bits(A), np.uint16), be.up(to_bf16_bits(B), np.uint16)
    c = be.up(np.zeros(m * n, np.uint16), np.uint16) if c_bf16 else be.up(np.zeros(m * n, np.float32))
    gpu.dispatch(opspec.linear(a, b, c, m, n, k, ta, tb, a_shape[1], b_shape[1], n))
    out = be.down(c)
    if c_bf16:
        out = (out.astype(np.uint32) << 16).view(np.float32)
    assert rel_err(out.reshape(m, n), want) <= (4e-3 if c_bf16 else 1e-5), rel_err(out.reshape(m, n), want)


@pytest.mark.parametrize("trans", list(TRANS))
def test_persistent_gemm_tf32_and_accumulate(gpu, trans):
    m, n, k = 5000, 1000, 520
    ta, tb = TRANS[trans]
    got, want = run_gemm(gpu, abi.MATH_TF32, m, n, k, ta, tb, alpha=0.5, beta=1.0, seed=11)
    assert rel_err(got, want) <= 2e-3, rel_err(got, want)


def test_persistent_gemm_bf16_epilogues(gpu):
    """The mixed-precision layer shapes: bias+ReLU with bf16 output, ReLU mask
    with bf16 mask/output plus column sums, fp32 accumulation into dW."""
    m, n, k = 5120, 768, 512
    g = rng(77)
    X, W = g.standard_normal((m, k)).astype(np.float32), g.standard_normal((n, k)).astype(np.float32) * 0.05
    b = g.standard_normal(n).astype(np.float32)
    r16 = lambda a: oracle.round_bf16(np.ascontiguousarray(a, np.float32).ravel()).reshape(a.shape)
    Xr, Wr = r16(X), r16(W)
    be = GpuBackend(gpu)
    x, w = be.up(to_bf16_bits(X), np.uint16), be.up(to_bf16_bits(W), np.uint16)
    bias = be.up(b)
    # forward: relu(X W^T + b) -> bf16
    y = be.up(np.zeros(m * n, np.uint16), np.uint16)
    gpu.dispatch(opspec.linear(x, w, y, m, n, k, False, True, k, k, n, 1.0, 0.0, "bias_relu", bias))
    want = np.maximum(ORC.bmm_acc(Xr, Wr, np.zeros((m, n), np.float32), (1, m, k), (1, k, n), (1, m, n), False, True, k, k, n, 1.0, 0.0) + b, 0)
    got = (gpu.to_numpy(y).astype(np.uint32) << 16).view(np.float32).reshape(m, n)
    assert rel_err(got, want) <= 4e-3
    # dX = dY W masked by the layer input activation (bf16), column sums added to db
    dY = g.standard_normal((m, n)).astype(np.float32)
    prev = np.maximum(g.standard_normal((m, k)).astype(np.float32), 0)
    dy, pv = be.up(to_bf16_bits(dY), np.uint16), be.up(to_bf16_bits(prev), np.uint16)
    dx = be.up(np.zeros(m * k, np.uint16), np.uint16)
    db = be.up(np.zeros(k, np.float32))
    gpu.dispatch(opspec.linear(dy, w, dx, m, k, n, False, False, n, k, k, 1.0, 0.0, "relu_mask", None, pv, colsum=db))
    wdx = ORC.bmm_acc(r16(dY), Wr, np.zeros((m, k), np.float32), (1, m, n), (1, n, k), (1, m, k), False, False, n, k, k, 1.0, 0.0)
    wdx[r16(prev) <= 0] = 0
    gdx = (gpu.to_numpy(dx).astype(np.uint32) << 16).view(np.float32).reshape(m, k)
    assert rel_err(gdx, wdx) <= 4e-3
    assert rel_err(gpu.to_numpy(db), wdx.sum(0)) <= 1e-3
    # dW += dY^T X in fp32 (m = n_out, n = k_in, contraction over the batch)
    dw0 = g.standard_normal((n, k)).astype(np.float32)
    dw = be.up(dw0)
    gpu.dispatch(opspec.linear(dy, x, dw, n, k, m, True, False, n, k, k, 1.0, 1.0))
    wdw = ORC.bmm_acc(r16(dY), Xr, dw0.copy(), (1, n, m), (1, m, k), (1, n, k), True, False, n, k, k, 1.0, 1.0)
    assert rel_err(be.down(dw).reshape(n, k), wdw) <= 1e-5


@pytest.mark.parametrize("beta", [1.0, 0.0, 0.5])
def test_persistent_gemm_split_k_weight_gradient(gpu, beta):
    """160 tiles of 128 x 256 on 148 SMs: the K ranges become work items
    (vector reductions into C, pre-scaled by beta)."""
    m, n, k = 2560, 2048, 4096
    g = rng(5)
    A, B = g.standard_normal((k, m)).astype(np.float32), g.standard_normal((k, n)).astype(np.float32)
    C0 = g.standard_normal((m, n)).astype(np.float32)
    r16 = lambda a: oracle.round_bf16(np.ascontiguousarray(a, np.float32).ravel()).reshape(a.shape)
    want = ORC.bmm_acc(r16(A), r16(B), C0.copy(), (1, m, k), (1, k, n), (1, m, n), True, False, m, n, n, 1.0, beta)
    be = GpuBackend(gpu)
    a, b, c = be.up(to_bf16_bits(A), np.uint16), be.up(to_bf16_bits(B), np.uint16), be.up(C0)
    gpu.dispatch(opspec.linear(a, b, c, m, n, k, True, False, m, n, n, 1.0, beta))
    assert rel_err(be.down(c).reshape(m, n), want) <= 1e-5
