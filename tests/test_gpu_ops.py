"""Op-level parity: every memory-bound kernel against the CPU oracle on the
same seeded inputs, through the C ABI.  Bit-exact where the op is a copy, a
comparison, an index move or a single correctly-rounded arithmetic step;
otherwise max relative error per tensor <= 1e-4 (the bound the hot path is
specified to), usually far tighter and stated per test."""
import numpy as np
import pytest

from zigrad_b200 import opspec

from .backends import GpuBackend, OracleBackend

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 31, 33, 127, 1000, 4099, (1 << 20) + 5]
ORC = OracleBackend()


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    d = np.max(np.abs(a - b)) if a.size else 0.0
    return d / max(np.max(np.abs(b)) if b.size else 0.0, 1e-30)


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("n", SIZES)
def test_binary_equal_length_bit_exact(gpu, op, n):
    g = rng(n)
    x, y = g.standard_normal(n).astype(np.float32), (g.standard_normal(n).astype(np.float32) + 3.0)
    np.testing.assert_array_equal(GpuBackend(gpu).elwise(op, x, y), ORC.elwise(op, x, y))


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("rows,L", [(64, 128), (64, 10), (8192, 64), (7, 33), (5, 1), (1000, 4), (3, 1025)])
def test_binary_broadcast_both_orders_bit_exact(gpu, op, rows, L):
    g = rng(rows * 131 + L)
    long_, short = g.standard_normal(rows * L).astype(np.float32), (g.standard_normal(L).astype(np.float32) + 2.5)
    be = GpuBackend(gpu)
    np.testing.assert_array_equal(be.elwise(op, short, long_), ORC.elwise(op, short, long_))  # bias.add_(y) order
    np.testing.assert_array_equal(be.elwise(op, long_, short), ORC.elwise(op, long_, short))


def test_binary_rejects_non_broadcastable_lengths(dev):
    from zigrad_b200 import abi
    be = GpuBackend(dev)
    abi.lib().zg_clear_error()
    with pytest.raises(abi.DeviceError):
        be.elwise("add", np.ones(6, np.float32), np.ones(4, np.float32))
    abi.lib().zg_clear_error()


@pytest.mark.parametrize("n", SIZES)
def test_relu_family_bit_exact(gpu, n):
    g = rng(n + 7)
    x = g.standard_normal(n).astype(np.float32)
    x[:: 5] = 0.0
    if n > 3:
        x[1], x[2] = -0.0, np.nan
    yg, xg = g.standard_normal(n).astype(np.float32), g.standard_normal(n).astype(np.float32)
    be = GpuBackend(gpu)
    got, want = be.relu_fwd(x), ORC.relu_fwd(x)
    np.testing.assert_array_equal(got, want)  # == treats -0.0 and 0.0 alike, NaN never appears in the output
    np.testing.assert_array_equal(be.relu_bwd(x, xg, yg), ORC.relu_bwd(x, xg, yg))
    act = ORC.relu_fwd(x)
    np.testing.assert_array_equal(be.relu_inplace_bwd(act, xg), ORC.relu_inplace_bwd(act, xg))


@pytest.mark.parametrize("n", [5, 1000, 4099])
def test_clamp_bit_exact(gpu, n):
    g = rng(n)
    x = (g.standard_normal(n) * 2).astype(np.float32)
    x[0], x[-1] = -1.0, 1.0  # exactly on the bounds: open interval in the backward
    xg, yg = g.standard_normal(n).astype(np.float32), g.standard_normal(n).astype(np.float32)
    be = GpuBackend(gpu)
    np.testing.assert_array_equal(be.clamp_fwd(x, -1.0, 1.0), ORC.clamp_fwd(x, -1.0, 1.0))
    np.testing.assert_array_equal(be.clamp_bwd(x, xg, yg, -1.0, 1.0), ORC.clamp_bwd(x, xg, yg, -1.0, 1.0))


@pytest.mark.parametrize("name,tol", [("exp", 1e-6), ("sqrt", 0.0), ("rsqrt", 2e-7), ("tanh", 1e-6), ("sigm", 1e-6)])
def test_unary_maps(gpu, name, tol):
    g = rng(11)
    x = g.uniform(0.0, 4.0, 5001).astype(np.float32)
    x[:3] = [0.0, 1e-13, 1e-12]
    p = 1e-12 if name == "rsqrt" else 0.0
    be = GpuBackend(gpu)
    got, want = be.unary(name, x, p), ORC.unary(name, x, p)
    if tol == 0.0:
        np.testing.assert_array_equal(got, want)
    else:
        np.testing.assert_allclose(got, want, rtol=tol * 4, atol=0)
    v = want if name in ("exp", "tanh", "sigm") else x
    yg, xg = g.standard_normal(x.size).astype(np.float32), g.standard_normal(x.size).astype(np.float32)
    eps = 1e-12 if name in ("sqrt", "rsqrt") else 0.0
    np.testing.assert_allclose(be.unary_bwd(name, v, yg, xg, eps), ORC.unary_bwd(name, v, yg, xg, eps), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("row,col", [(64, 128), (64, 64), (64, 10), (8192, 128), (8192, 10), (1000, 1000), (3, 7), (2, 1),
                                     (4097, 132), (300, 4099)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 1.0), (1.0, 0.0), (-0.5, 2.0)])
def test_fold_rows(gpu, row, col, alpha, beta):
    g = rng(row * 7 + col)
    x, y0 = g.standard_normal(row * col).astype(np.float32), g.standard_normal(col).astype(np.float32)
    got, want = GpuBackend(gpu).fold_rows(x, row, col, alpha, beta, y0), ORC.fold_rows(x, row, col, alpha, beta, y0)
    # different (but fixed) summation tree than the host's sequential row order
    assert rel_err(got, want) <= 2e-6 * max(1.0, np.sqrt(row) / 8), rel_err(got, want)


def test_fold_rows_is_deterministic(gpu):
    x = rng(5).standard_normal(8192 * 128).astype(np.float32)
    be = GpuBackend(gpu)
    a, b = be.fold_rows(x, 8192, 128), be.fold_rows(x, 8192, 128)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("row,col", [(256, 2), (64, 10), (1000, 33), (5, 4099), (8192, 16)])
def test_fold_cols(gpu, row, col):
    g = rng(row + col)
    x, y0 = g.standard_normal(row * col).astype(np.float32), g.standard_normal(row).astype(np.float32)
    got, want = GpuBackend(gpu).fold_cols(x, row, col, 1.0, 1.0, y0), ORC.fold_cols(x, row, col, 1.0, 1.0, y0)
    assert rel_err(got, want) <= 2e-6


@pytest.mark.parametrize("shape,dim", [((2, 3, 4), 0), ((2, 3, 4), 1), ((2, 3, 4), 2), ((17, 33, 5), 1), ((256, 2), 1),
                                       ((6,), 0), ((5, 1, 7), 1), ((3, 4, 5, 6), 2)])
def test_sum_along_and_max_along(gpu, shape, dim):
    g = rng(sum(shape) + dim)
    x = g.standard_normal(int(np.prod(shape))).astype(np.float32)
    be = GpuBackend(gpu)
    assert rel_err(be.sum_along(x, shape, dim, 0.5, 0.0), ORC.sum_along(x, shape, dim, 0.5, 0.0)) <= 2e-6
    np.testing.assert_array_equal(be.max_along(x, shape, dim), ORC.max_along(x, shape, dim))  # selection: bit-exact


@pytest.mark.parametrize("xs,ys", [((2, 3, 3), (3,)), ((2, 3, 3), (2, 1, 3)), ((64, 128), (128,)), ((1, 4, 5), (5,)),
                                   ((4, 5, 6), (1, 5, 6)), ((3, 4), (3, 4)), ((2, 3, 4, 5), (3, 1, 5)), ((8, 7), (1,))])
def test_unbroadcast(gpu, xs, ys):
    g = rng(len(xs) * 100 + len(ys))
    x, y0 = g.standard_normal(int(np.prod(xs))).astype(np.float32), g.standard_normal(int(np.prod(ys))).astype(np.float32)
    got, want = GpuBackend(gpu).unbroadcast(x, xs, y0, ys, 1.0, 1.0), ORC.unbroadcast(x, xs, y0, ys, 1.0, 1.0)
    assert rel_err(got, want) <= 2e-6, (got, want)


@pytest.mark.parametrize("xs,ys", [((4, 5, 6), (5, 1)), ((3, 2, 7, 4), (2, 1, 1)), ((6, 9), (6, 1)), ((4, 5, 1), (5, 1))])
def test_unbroadcast_onto_trailing_ones_stays_inside_y(gpu, xs, ys):
    """y shapes that END in ones: the host code drops them and then lines y up against the wrong
    dimensions of x -- it folds x's last dimension into y, past y's end, or fills y[0] only (the
    oracle reports these shapes instead of restating an out-of-bounds write).  The device keeps
    the alignment: the sums that the broadcasting rule defines, and nothing outside y (the guard
    regions around y are checked)."""
    import oracle
    g = rng(sum(xs) + len(ys))
    x, y0 = g.standard_normal(int(np.prod(xs))).astype(np.float32), g.standard_normal(int(np.prod(ys))).astype(np.float32)
    with pytest.raises(oracle.ReferenceOutOfBounds):
        ORC.unbroadcast(x, xs, y0, ys, 1.0, 1.0)
    lead = len(xs) - len(ys)
    axes = tuple(range(lead)) + tuple(lead + i for i, (a, b) in enumerate(zip(xs[lead:], ys)) if b == 1 and a != 1)
    want = 0.5 * x.reshape(xs).astype(np.float64).sum(axes).ravel() + 2.0 * y0
    got = GpuBackend(gpu).unbroadcast(x, xs, y0, ys, 0.5, 2.0)
    assert rel_err(got, want) <= 2e-6, (got, want)


@pytest.mark.parametrize("n", [1, 4, 1000, 4099, (1 << 20) + 5])
def test_blas1_scalars(gpu, n):
    g = rng(n)
    x, y = g.standard_normal(n).astype(np.float32), g.standard_normal(n).astype(np.float32)
    be = GpuBackend(gpu)
    assert abs(be.nrm2(x) - ORC.nrm2(x)) <= 2e-6 * ORC.nrm2(x) + 1e-30
    assert abs(be.asum(x) - ORC.asum(x)) <= 1e-5 * ORC.asum(x)
    assert abs(be.dot(x, y) - ORC.dot(x, y)) <= 1e-4 * max(1.0, np.sqrt(n))
    np.testing.assert_array_equal(be.scale(x, 0.37), ORC.scale(x, 0.37))
    want = ORC.axpy(x, y, -0.01)
    np.testing.assert_allclose(be.axpy(x, y, -0.01), want, rtol=0, atol=1.2e-7 * np.max(np.abs(want)))
    np.testing.assert_array_equal(be.axpy(x, y, -0.01), be.axpy(x, y, -0.01, device_alpha=True))
    np.testing.assert_array_equal(be.max_fwd(x), ORC.max_fwd(x))
    mx = ORC.max_fwd(x)
    np.testing.assert_array_equal(be.max_bwd(x, y, mx, np.array([2.0], np.float32)), ORC.max_bwd(x, y, mx, np.array([2.0], np.float32)))


def test_clip_nrm2_both_branches(gpu):
    x = rng(3).standard_normal(10007).astype(np.float32)
    be = GpuBackend(gpu)
    np.testing.assert_array_equal(be.clip_nrm2(x, 1e9, 1e-6), x)  # below the bound: untouched
    got, want = be.clip_nrm2(x, 10.0, 1e-6), ORC.clip_nrm2(x, 10.0, 1e-6)
    assert rel_err(got, want) <= 1e-6


def test_transpose_host_semantics(gpu):
    g = rng(9)
    A, B = g.standard_normal(37 * 65).astype(np.float32), g.standard_normal(37 * 65).astype(np.float32)
    np.testing.assert_array_equal(GpuBackend(gpu).transpose(A, B, 37, 65, 0.0), ORC.transpose(A, B, 37, 65, 0.0))
    np.testing.assert_allclose(GpuBackend(gpu).transpose(A, B, 37, 65, 0.5), ORC.transpose(A, B, 37, 65, 0.5), rtol=1e-6)


def test_take_and_scatter_add(gpu):
    g = rng(2)
    src = g.standard_normal(5000).astype(np.float32)
    idx = g.integers(0, 5000, 777).astype(np.uint64)
    be = GpuBackend(gpu)
    np.testing.assert_array_equal(be.take(src, idx), ORC.take(src, idx))  # index path: bit-exact
    # distinct offsets: bit-exact; duplicates: same addends, different order
    offs = g.permutation(5000)[:777].astype(np.uint64)
    vals, dst = g.standard_normal(777).astype(np.float32), g.standard_normal(5000).astype(np.float32)
    np.testing.assert_array_equal(be.scatter_add(vals, offs, dst), ORC.scatter_add(vals, offs, dst))
    np.testing.assert_allclose(be.scatter_add(vals, idx, dst), ORC.scatter_add(vals, idx, dst), rtol=1e-5, atol=1e-5)


def test_gather_rows_dqn_shape(gpu):
    from zigrad_b200.device import USIZE
    g = rng(4)
    q = g.standard_normal((256, 2)).astype(np.float32)
    a = g.integers(0, 2, 256).astype(np.uint64)
    be = GpuBackend(gpu)
    Q, A = be.up(q), be.up(a, np.uint64)
    D, O = be.up(np.zeros(256, np.float32)), be.up(np.zeros(256, np.uint64), np.uint64)
    gpu.gather_rows(Q, A, 256, 2, D, O)
    offs = gpu.to_numpy(O)
    out = be.down(D)
    np.testing.assert_array_equal(out, q[np.arange(256), a.astype(np.int64)])
    np.testing.assert_array_equal(offs, (np.arange(256) * 2 + a.astype(np.int64)).astype(np.uint64))


def test_gcn_edge_scatter(gpu):
    g = rng(6)
    N, E, F = 300, 1200, 16
    s, t = g.integers(0, N, E).astype(np.uint64), g.integers(0, N, E).astype(np.uint64)
    h, deg = g.standard_normal(N * F).astype(np.float32), g.uniform(0.2, 1.0, N).astype(np.float32)
    be = GpuBackend(gpu)
    got, want = be.scatter_gcn(np.zeros(N * F, np.float32), h, deg, s, t, F), ORC.scatter_gcn(np.zeros(N * F, np.float32), h, deg, s, t, F)
    assert rel_err(got, want) <= 1e-5
    go = g.standard_normal(N * F).astype(np.float32)
    gh, gd = be.scatter_gcn_bwd(go, h, deg, s, t, np.zeros(N * F, np.float32), np.zeros(N, np.float32), F)
    wh, wd = ORC.scatter_gcn_bwd(go, h, deg, s, t, np.zeros(N * F, np.float32), np.zeros(N, np.float32), F)
    assert rel_err(gh, wh) <= 1e-5 and rel_err(gd, wd) <= 1e-5


@pytest.mark.parametrize("rows,C", [(64, 10), (8192, 10), (140, 7), (33, 1000), (5, 1), (7, 33), (3, 2500)])
def test_softmax_cross_entropy_fused(gpu, rows, C):
    g = rng(rows + C)
    x = (g.standard_normal((rows, C)) * 3).astype(np.float32)
    lab = g.integers(0, C, rows)
    t = np.zeros((rows, C), np.float32)
    t[np.arange(rows), lab] = 1.0
    be = GpuBackend(gpu)
    loss, grad, probs = be.softmax_ce(x, t)
    wl, wg, wp = ORC.softmax_ce(x, t)
    assert abs(loss - wl) <= 1e-5 * max(1.0, abs(wl))
    assert rel_err(grad, wg) <= 1e-5 and rel_err(probs, wp) <= 1e-5
    # predictions (argmax of the probabilities) are bit-exact
    np.testing.assert_array_equal(np.argmax(probs, axis=1), np.argmax(wp, axis=1))
    # index labels give the same numbers as one-hot labels; a global divisor scales loss and grad
    l2, g2, _ = be.softmax_ce(x, t, loss_div=4 * rows, index_labels=lab.astype(np.uint64))
    wl2, wg2, _ = ORC.softmax_ce(x, t, loss_div=4 * rows)
    assert abs(l2 - wl2) <= 1e-5 * max(1.0, abs(wl2)) and rel_err(g2, wg2) <= 1e-5


@pytest.mark.parametrize("rows,C,ld", [(8192, 10, 12), (64, 10, 16), (33, 1000, 1000), (300, 7, 8)])
def test_softmax_cross_entropy_row_stride_and_fused_bias_gradient(gpu, rows, C, ld):
    g = rng(rows * 3 + C)
    x = (g.standard_normal((rows, C)) * 2).astype(np.float32)
    t = np.eye(C, dtype=np.float32)[g.integers(0, C, rows)]
    loss, grad, probs, bias = GpuBackend(gpu).softmax_ce(x, t, ld=ld, want_bias=True)
    wl, wg, wp = ORC.softmax_ce(x, t)
    assert abs(loss - wl) <= 1e-5 * max(1.0, abs(wl))
    assert rel_err(grad, wg) <= 1e-5 and rel_err(probs, wp) <= 1e-5
    want_bias = ORC.fold_rows(wg.ravel(), rows, C)  # what InplaceAddBwd's unbroadcast would produce
    assert rel_err(bias, want_bias) <= 1e-5


def test_softmax_cross_entropy_accumulates_into_grad(gpu):
    g = rng(1)
    x, g0 = g.standard_normal((16, 10)).astype(np.float32), g.standard_normal((16, 10)).astype(np.float32)
    t = np.eye(10, dtype=np.float32)[g.integers(0, 10, 16)]
    _, got, _ = GpuBackend(gpu).softmax_ce(x, t, grad0=g0)
    _, want, _ = ORC.softmax_ce(x, t, grad0=g0)
    assert rel_err(got, want) <= 1e-5


def test_smooth_l1(gpu):
    g = rng(8)
    p, t = (g.standard_normal(256) * 2).astype(np.float32), g.standard_normal(256).astype(np.float32)
    loss, grad = GpuBackend(gpu).smooth_l1(p, t, 1.0)
    wl, wg = ORC.smooth_l1(p, t, 1.0)
    assert abs(loss - wl) <= 1e-6 * max(1.0, abs(wl))
    np.testing.assert_array_equal(grad, wg)


SEGS = [(0, 100352), (100352, 128), (100480, 8192), (108672, 64), (108736, 640), (109376, 10)]


@pytest.mark.parametrize("clip", [False, True])
def test_sgd_step_flat_buffer(gpu, clip):
    g = rng(12)
    n = 109386
    p, gr = g.standard_normal(n).astype(np.float32), (g.standard_normal(n) * (0.2 if clip else 1.0)).astype(np.float32)
    gp, gg = GpuBackend(gpu).sgd(p, gr, SEGS, 0.01, clip, 10.0, 1e-6)
    wp, wg = ORC.sgd(p, gr, SEGS, 0.01, clip, 10.0, 1e-6)
    assert rel_err(gp, wp) <= 2e-7 and rel_err(gg, wg) <= 1e-6


@pytest.mark.parametrize("clip", [False, True])
def test_sgd_step_that_clears_the_gradients(gpu, clip):
    """zero_grads: the same update, and the applied gradients read back as zeros."""
    g = rng(14)
    n = 109386
    p, gr = g.standard_normal(n).astype(np.float32), (g.standard_normal(n) * (0.2 if clip else 1.0)).astype(np.float32)
    be = GpuBackend(gpu)
    P, G, N = be.up(p), be.up(gr), be.up(np.zeros(len(SEGS), np.float32))
    gpu.dispatch(opspec.sgd(P, G, SEGS, 0.01, clip, 10.0, 1e-6, N, True))
    wp, _ = ORC.sgd(p, gr, SEGS, 0.01, clip, 10.0, 1e-6)
    assert rel_err(gpu.to_numpy(P), wp) <= 2e-7
    assert not gpu.to_numpy(G).any()
    be.down(P), be.down(N)


@pytest.mark.parametrize("clip", [False, True])
def test_adam_step_flat_buffer_per_tensor_counter(gpu, clip):
    g = rng(13)
    n = 109386
    p, gr = g.standard_normal(n).astype(np.float32), g.standard_normal(n).astype(np.float32)
    m, v = (g.standard_normal(n) * 0.1).astype(np.float32), g.uniform(0, 0.1, n).astype(np.float32)
    got = GpuBackend(gpu).adam(p, gr, m, v, SEGS, 7, 1e-3, clip=clip)
    want = ORC.adam(p, gr, m, v, SEGS, 7, 1e-3, clip=clip)
    for a, b in zip(got, want):
        assert rel_err(a, b) <= 2e-6
    if not clip:  # same operation sequence, correctly rounded ops: bit-exact moments
        np.testing.assert_array_equal(got[2], want[2])
        np.testing.assert_array_equal(got[3], want[3])


def test_fill_sequence_random_cast(gpu):
    from zigrad_b200.abi import SINGLE, BF16
    d = gpu
    s = d.mem_cache_alloc(SINGLE, 4099)
    d.mem_fill(s, 1.5)
    np.testing.assert_array_equal(d.to_numpy(s), np.full(4099, 1.5, np.float32))
    d.mem_fill(s.view(1, 4097), 0.0)  # unaligned zero fill
    out = d.to_numpy(s)
    assert out[0] == 1.5 and out[-1] == 1.5 and not out[1:-1].any()
    d.mem_sequence(s, 2.0, 0.5)
    np.testing.assert_array_equal(d.to_numpy(s), (2.0 + 0.5 * np.arange(4099)).astype(np.float32))
    d.mem_random(s, "uniform", 81761)
    u = d.to_numpy(s)
    assert 0.0 <= u.min() and u.max() < 1.0 and 0.45 < u.mean() < 0.55
    d.mem_random(s, "normal", 81761)
    z = d.to_numpy(s)
    assert abs(z.mean()) < 0.1 and 0.9 < z.std() < 1.1
    b = d.mem_cache_alloc(BF16, 4099)
    d.cast(s, b)
    import oracle
    bits = d.to_numpy(b)
    np.testing.assert_array_equal(bits, (oracle.round_bf16(z).view(np.uint32) >> 16).astype(np.uint16))  # RNE, bit-exact
    d.mem_cache_free(s)
    d.mem_cache_free(b)


def test_plan_api_of_the_reference_shim(gpu):
    """get_reduce_plan/reduce, get_contraction_plan/contraction and
    get_permutate_plan/permutate as src/device/cuda_device.zig calls them."""
    import ctypes as C
    from zigrad_b200 import abi
    L, d = gpu.L, gpu
    g = rng(21)
    x = g.standard_normal(2 * 3 * 4).astype(np.float32)
    be = GpuBackend(gpu)
    X, Y = be.up(x), be.up(np.zeros(8, np.float32))
    dims = (abi.len_t * 3)(2, 3, 4)
    ydims = (abi.len_t * 2)(2, 4)
    plan = L.get_reduce_plan(d.cutensor, abi.SINGLE, dims, (C.c_ubyte * 3)(*b"abc"), 3, ydims, (C.c_ubyte * 2)(*b"ac"), 2, abi.ADD)
    one, zero = C.c_float(1.0), C.c_float(0.0)
    L.reduce(d.cutensor, plan.plan, X.ptr, Y.ptr, None, 0, C.byref(one), C.byref(zero))
    got = be.down(Y)
    np.testing.assert_allclose(got, x.reshape(2, 3, 4).sum(1).ravel(), rtol=1e-6)
    # contraction: A [2,3,5] "ijk", B stored [2,4,5] "imk" (transposed), C [2,3,4]
    A, B = g.standard_normal((2, 3, 5)).astype(np.float32), g.standard_normal((2, 4, 5)).astype(np.float32)
    a, b, c = be.up(A), be.up(B), be.up(np.zeros(24, np.float32))
    plan = L.get_contraction_plan(d.cutensor, abi.SINGLE, (abi.len_t * 3)(2, 3, 5), (C.c_ubyte * 3)(*b"ijk"), 3,
                                  (abi.len_t * 3)(2, 5, 4), (C.c_ubyte * 3)(*b"imk"), 3,
                                  (abi.len_t * 3)(2, 3, 4), (C.c_ubyte * 3)(*b"ijm"), 3)
    L.contraction(d.cutensor, plan.plan, a.ptr, b.ptr, c.ptr, None, 0, C.byref(one), C.byref(zero))
    np.testing.assert_allclose(be.down(c).reshape(2, 3, 4), np.einsum("ijk,imk->ijm", A, B), rtol=1e-5, atol=1e-5)
    M = g.standard_normal((5, 7)).astype(np.float32)
    m_, t_ = be.up(M), be.up(np.zeros(35, np.float32))
    plan = L.get_permutate_plan(d.cutensor, abi.SINGLE, (abi.len_t * 2)(5, 7), (C.c_ubyte * 2)(*b"ij"), 2,
                                (abi.len_t * 2)(7, 5), (C.c_ubyte * 2)(*b"ji"), 2)
    L.permutate(d.cutensor, plan.plan, m_.ptr, t_.ptr, None, 0, C.byref(one))
    np.testing.assert_array_equal(be.down(t_).reshape(7, 5), M.T)


@pytest.mark.parametrize("rows,C", [(3000, 1000), (20011, 64), (4100, 256), (2500, 512), (9000, 128),
                                     (120003, 10), (300000, 4), (70001, 16), (50000, 28), (150001, 7),
                                     (30001, 36), (12001, 100), (22003, 48)])
def test_softmax_ce_fast_paths_large_index_labels(gpu, rows, C):
    """The FAST form (index labels, power-of-two divisor, gradient written,
    bias gradient fused) at sizes that take the staged kernel; the last row group
    is ragged.  Oracle: the reference's softmax-CE on one-hot rows."""
    g = rng(rows + C)
    x = (g.standard_normal((rows, C)) * 3).astype(np.float32)
    lab = g.integers(0, C, rows)
    t = np.zeros((rows, C), np.float32)
    t[np.arange(rows), lab] = 1.0
    div = 4096
    wl, wg, _ = ORC.softmax_ce(x, t, loss_div=div)
    d = gpu
    X, T = d.from_numpy(x), d.from_numpy(lab.astype(np.uint64))
    G, Ls, Bg = d.from_numpy(np.full((rows, C), 7.0, np.float32)), d.from_numpy(np.zeros(1, np.float32)), d.from_numpy(np.ones(C, np.float32))
    d.dispatch(opspec.softmax_ce(X, T, rows, C, Ls, G, div, False, None, 0, Bg))
    got_g, got_l, got_b = d.to_numpy(G, (rows, C)), float(d.to_numpy(Ls)[0]), d.to_numpy(Bg)
    # the host loop adds up to 300 000 row losses one after the other in fp32 (rounding ~ sqrt(rows) * 6e-8
    # relative); the device folds per-thread and per-CTA partial sums: 1e-4, the bound of the hot path
    assert abs(got_l - wl) <= 1e-4 * abs(wl), (got_l, wl)
    assert rel_err(got_g, wg) <= 1e-5, rel_err(got_g, wg)
    assert rel_err(got_b, wg.astype(np.float64).sum(0)) <= 1e-4
    for s in (X, T, G, Ls, Bg):
        d.mem_cache_free(s)


# ---------------------------------------------------------------- ops of the interface beyond the training step
@pytest.mark.parametrize("e", [2.0, 0.5, 3.0, -1.5])
def test_pow_forward_in_place_and_backward(gpu, e):
    g = rng(int(e * 10) + 40)
    x = g.uniform(0.05, 4.0, 4099).astype(np.float32)
    x[:3] = [0.0, 1e-13, 1.0]
    be = GpuBackend(gpu)
    want = ORC.pow_fwd(x, e)
    with np.errstate(divide="ignore"):
        np.testing.assert_allclose(be.pow_fwd(x, e), want, rtol=2e-6, atol=0)           # powf vs libm pow: a few ulp
        np.testing.assert_allclose(be.pow_fwd(x, e, inplace=True), want, rtol=2e-6, atol=0)
    xg, yg = g.standard_normal(x.size).astype(np.float32), g.standard_normal(x.size).astype(np.float32)
    # entries below eps (the first two) must come back untouched
    got, wantg = be.pow_bwd(x, xg, yg, e, 1e-12), ORC.pow_bwd(x, xg, yg, e, 1e-12)
    np.testing.assert_array_equal(got[:2], xg[:2])
    np.testing.assert_allclose(got, wantg, rtol=1e-5, atol=1e-6)


def test_sqrt_in_place_bit_exact(gpu):
    x = rng(3).uniform(0.0, 9.0, 1027).astype(np.float32)
    np.testing.assert_array_equal(GpuBackend(gpu).sqrt_inplace(x), ORC.unary("sqrt", x))


@pytest.mark.parametrize("name", ["tanh", "sigm"])
@pytest.mark.parametrize("n", [1, 33, 4099])
def test_inplace_backward_of_tanh_and_sigmoid_bit_exact(gpu, name, n):
    g = rng(n + 77)
    y = ORC.unary(name, g.standard_normal(n).astype(np.float32))   # the op reads the activation's output
    xg = g.standard_normal(n).astype(np.float32)
    # two correctly rounded multiplies and one subtraction, compiled without contraction on both sides
    np.testing.assert_array_equal(GpuBackend(gpu).inplace_bwd(name, y, xg), ORC.inplace_bwd(name, y, xg))


@pytest.mark.parametrize("n", [1, 7, 8, 9, 63, 64, 1000, 4099, (1 << 18) + 3])
def test_byte_mask_relu_bit_exact(gpu, n):
    g = rng(n + 5)
    x = g.standard_normal(n).astype(np.float32)
    x[::7] = 0.0
    if n > 2:
        x[1] = -0.0
    be = GpuBackend(gpu)
    got_x, got_m = be.relu_mask_fwd(x)
    want_x, want_m = ORC.relu_mask_fwd(x)
    np.testing.assert_array_equal(got_m, want_m)   # includes the unused high bits of the last byte: zero
    np.testing.assert_array_equal(got_x, want_x)
    xg = g.standard_normal(n).astype(np.float32)
    np.testing.assert_array_equal(be.relu_mask_bwd(xg, want_m), ORC.relu_mask_bwd(xg, want_m))


@pytest.mark.parametrize("n", [1, 8, 13, 64, 1001, 4099])
def test_byte_mask_clamp_bit_exact(gpu, n):
    g = rng(n + 9)
    x = (g.standard_normal(n) * 2).astype(np.float32)
    x[0] = 1.0  # on the bound: clamping leaves it unchanged, bit clear
    be = GpuBackend(gpu)
    got_y, got_m = be.clamp_mask_fwd(x, -1.0, 1.0)
    want_y, want_m = ORC.clamp_mask_fwd(x, -1.0, 1.0)
    np.testing.assert_array_equal(got_m, want_m)
    np.testing.assert_array_equal(got_y, want_y)
    np.testing.assert_array_equal(got_y, x)        # the reference stores x itself, not the clamped value
    xg, yg = g.standard_normal(n).astype(np.float32), g.standard_normal(n).astype(np.float32)
    np.testing.assert_array_equal(be.clamp_mask_bwd(xg, yg, want_m), ORC.clamp_mask_bwd(xg, yg, want_m))


@pytest.mark.parametrize("n_blocks,stride,n_seg", [(1, 1, 1), (100, 16, 7), (4099, 7, 300), (2708, 33, 2708), (5000, 128, 11)])
def test_scatter_add_2d(gpu, n_blocks, stride, n_seg):
    g = rng(n_blocks + stride)
    src = g.standard_normal((n_blocks, stride)).astype(np.float32)
    idx = g.integers(0, n_seg, n_blocks).astype(np.uint64)
    dst = g.standard_normal((n_seg, stride)).astype(np.float32)
    got, want = GpuBackend(gpu).scatter_add_2d(src, idx, dst, stride), ORC.scatter_add_2d(src, idx, dst, stride)
    # duplicates land in a different order than the host loop: a few ulp of the running sums
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5 * max(1.0, float(np.abs(want).max())))
    uniq = np.arange(min(n_blocks, n_seg), dtype=np.uint64)  # no duplicates: exact
    g2 = GpuBackend(gpu).scatter_add_2d(src[:uniq.size], uniq, dst, stride)
    np.testing.assert_array_equal(g2, ORC.scatter_add_2d(src[:uniq.size], uniq, dst, stride))


def _csr(g, n_seg, max_len):
    lens = g.integers(0, max_len + 1, n_seg)
    lens[::5] = 0                                    # empty segments
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.uint64)


@pytest.mark.parametrize("n_seg,max_len", [(1, 5), (100, 9), (2708, 40), (37, 5000)])
def test_csr_scatter_add_exact_and_segment_sum(gpu, n_seg, max_len):
    g = rng(n_seg + max_len)
    row_ptr = _csr(g, n_seg, max_len)
    total = int(row_ptr[-1])
    be = GpuBackend(gpu)
    src = g.standard_normal(n_seg).astype(np.float32)
    dst = g.standard_normal(max(total, 1)).astype(np.float32)
    np.testing.assert_array_equal(be.scatter_add_csr(src, row_ptr, dst), ORC.scatter_add_csr(src, row_ptr, dst))
    data = g.standard_normal(max(total, 1)).astype(np.float32)
    got, want = be.segment_sum_csr(data, row_ptr), ORC.segment_sum_csr(data, row_ptr)
    short = np.diff(row_ptr.astype(np.int64)) <= 32
    np.testing.assert_array_equal(got[short], want[short])   # left-to-right like the host loop
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-5 * np.sqrt(max_len))
