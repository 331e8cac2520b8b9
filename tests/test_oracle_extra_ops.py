"""The oracle's restatements of the device interface's byte-mask, pow, in-place
backward and CSR ops against an independent numpy formulation (CPU only)."""
import numpy as np

import oracle


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def test_byte_masks_follow_the_little_endian_bit_order(orc):
    for n in (1, 7, 8, 9, 100, 1001):
        x = rng(n).standard_normal(n).astype(np.float32)
        x[::3] = 0.0
        want_mask = np.packbits(x <= 0, bitorder="little")
        y = x.copy()
        mask = oracle.relu_mask_fwd(y)
        np.testing.assert_array_equal(mask, want_mask)
        np.testing.assert_array_equal(y, np.where(x <= 0, np.float32(0), x))
        gx = rng(n + 1).standard_normal(n).astype(np.float32)
        np.testing.assert_array_equal(oracle.relu_mask_bwd(gx.copy(), mask), np.where(x <= 0, np.float32(0), gx))
        yy, cm = oracle.clamp_mask_fwd(x * 2, -1.0, 1.0)
        np.testing.assert_array_equal(yy, x * 2)
        np.testing.assert_array_equal(cm, np.packbits(np.abs(x * 2) > 1, bitorder="little"))
        yg = np.ones(n, np.float32)
        np.testing.assert_array_equal(oracle.clamp_mask_bwd(gx.copy(), yg, cm), gx + (np.abs(x * 2) > 1))


def test_pow_and_inplace_backward(orc):
    x = rng(1).uniform(0.1, 3.0, 257).astype(np.float32)
    np.testing.assert_allclose(oracle.pow_fwd(x, 2.5), x.astype(np.float64) ** 2.5, rtol=1e-6)
    xg = np.zeros_like(x)
    np.testing.assert_allclose(oracle.pow_bwd(x, xg, np.ones_like(x), 3.0, 1e-12), 3.0 * x.astype(np.float64) ** 2, rtol=1e-6)
    y = np.tanh(x)
    np.testing.assert_allclose(oracle.inplace_bwd("tanh_inplace_bwd", y, np.full_like(x, 2.0)), 2 * (1 - y * y), rtol=1e-6)
    s = 1 / (1 + np.exp(-x))
    np.testing.assert_allclose(oracle.inplace_bwd("sigm_inplace_bwd", s, np.full_like(x, 2.0)), 2 * s * (1 - s), rtol=1e-6)


def test_csr_and_blocked_scatter(orc):
    g = rng(2)
    lens = g.integers(0, 9, 50)
    row_ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint64)
    data = g.standard_normal(int(row_ptr[-1])).astype(np.float32)
    want = np.array([data[int(a):int(b)].astype(np.float64).sum() for a, b in zip(row_ptr[:-1], row_ptr[1:])])
    np.testing.assert_allclose(oracle.segment_sum_csr(data, row_ptr), want, atol=1e-5)
    src = g.standard_normal(50).astype(np.float32)
    dst = np.zeros(int(row_ptr[-1]), np.float32)
    np.testing.assert_array_equal(oracle.scatter_add_csr(src, row_ptr, dst), np.repeat(src, lens))
    blocks = g.standard_normal((40, 6)).astype(np.float32)
    idx = g.integers(0, 5, 40).astype(np.uint64)
    out = oracle.scatter_add_2d(blocks.ravel(), idx, np.zeros(30, np.float32), 6).reshape(5, 6)
    want2 = np.zeros((5, 6))
    np.add.at(want2, idx.astype(np.int64), blocks.astype(np.float64))
    np.testing.assert_allclose(out, want2, atol=1e-5)
