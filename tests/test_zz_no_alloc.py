"""zg_fold_rows_noalloc: the fold_rows variant for callers that cannot allocate
device memory (code running under stream capture, real-time agent loops, hosts
with a fixed and audited device-memory budget).  Its scratch is a fixed array
inside the library image instead of a cudaMalloc'ed workspace.

Checked here, through the C ABI: the result equals zg_fold_rows' -- and the CPU
oracle's -- on two calls in a row (the second call must not be disturbed by what
the first left in the shared scratch), for aligned and ragged shapes, in single
and double precision, and inputs that do not fit the fixed array are refused
with a clear error instead of overflowing it.

This file sorts last on purpose, so a run that stops at the first failure has
already executed every other test.
"""
import numpy as np
import pytest

import oracle
from zigrad_b200 import abi
from zigrad_b200.abi import DOUBLE, SINGLE

pytestmark = pytest.mark.gpu


def both(dev, x, row, col, alpha, beta, y0, dt=SINGLE):
    """Runs the allocating and the non-allocating entry point on the same input."""
    X = dev.from_numpy(x)
    Ya, Yb = dev.from_numpy(y0), dev.from_numpy(y0)
    dev.L.zg_fold_rows(dt, dev.stream, X.ptr, Ya.ptr, row, col, alpha, beta)
    dev.L.zg_fold_rows_noalloc(dt, dev.stream, X.ptr, Yb.ptr, row, col, alpha, beta)
    a, b = dev.to_numpy(Ya), dev.to_numpy(Yb)
    for s in (X, Ya, Yb):
        dev.mem_cache_free(s)
    return a, b


@pytest.mark.parametrize("shapes", [((8192, 128), (4097, 132)), ((64, 10), (8192, 64)), ((1000, 1000), (3, 7))])
def test_two_calls_in_a_row_match_the_allocating_entry_point(gpu, shapes):
    g = np.random.Generator(np.random.PCG64(17))
    for k, (row, col) in enumerate(shapes):  # second call reuses the scratch the first one left behind
        x = g.standard_normal(row * col).astype(np.float32)
        y0 = g.standard_normal(col).astype(np.float32)
        want, got = both(gpu, x, row, col, 1.0 if k == 0 else -0.5, 1.0, y0)
        # same kernel, same chunking: the tolerance used for fold_rows elsewhere in this suite
        scale = max(np.max(np.abs(want)), 1e-30)
        assert np.max(np.abs(got - want)) / scale <= 2e-6 * max(1.0, np.sqrt(row) / 8)
        # and against the reference's host loop (reduce.zig:49-128 restated): plain row order per column
        alpha = 1.0 if k == 0 else -0.5
        cpu = oracle.fold_rows(x, y0.copy(), row, col, alpha, 1.0)
        assert np.max(np.abs(got - cpu)) / max(np.max(np.abs(cpu)), 1e-30) <= 2e-6 * max(1.0, np.sqrt(row) / 8)


def test_double_precision_two_calls_in_a_row(gpu):
    g = np.random.Generator(np.random.PCG64(23))
    for k, (row, col) in enumerate([(2048, 96), (513, 1031)]):
        x, y0 = g.standard_normal(row * col), g.standard_normal(col)
        want, got = both(gpu, x, row, col, 2.0, 0.5 if k else 0.0, y0, DOUBLE)
        np.testing.assert_allclose(got, want, rtol=1e-13, atol=1e-13)
        cpu = 2.0 * x.reshape(row, col).sum(0) + (0.5 if k else 0.0) * y0
        np.testing.assert_allclose(got, cpu, rtol=1e-12, atol=1e-12)


def test_refuses_inputs_wider_than_the_fixed_scratch(dev):
    L = abi.lib()
    L.zg_clear_error()
    col = 65536 + 128
    X, Y = dev.mem_cache_alloc(SINGLE, 2 * col), dev.mem_cache_alloc(SINGLE, col)
    dev.mem_fill(Y, 7.0)
    L.zg_fold_rows_noalloc(SINGLE, dev.stream, X.ptr, Y.ptr, 2, col, 1.0, 0.0)
    assert L.zg_last_error() == 2  # kBadArgument
    msg = L.zg_last_error_message().decode()
    assert "zg_fold_rows_noalloc" in msg and "fixed scratch" in msg and "65536" in msg
    L.zg_clear_error()
    out = dev.to_numpy(Y)
    assert np.all(out == 7.0), "a refused call must not touch the output"
    dev.mem_cache_free(X)
    dev.mem_cache_free(Y)
