"""The reference's known-answer vectors (tests/golden/golden.json) replayed
against a backend.  Shared by the CPU (oracle) and GPU (C ABI) test files."""
import json
import os

import numpy as np

from . import callers

G = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))
LIT, TORCH = G["literal"], G["torch"]


def arr(v, shape=None):
    a = np.asarray(v, np.float32)
    return a.reshape(shape) if shape is not None else a


def check_bmm(be):
    for c in LIT["bmm"]:
        out = callers.bmm(be, arr(c["a"], c["a_shape"]), arr(c["b"], c["b_shape"]))
        assert list(out.shape) == c["c_shape"], c
        np.testing.assert_array_equal(out.ravel(), arr(c["c"]))
    c = LIT["bmm_acc"]
    out = callers.bmm(be, arr(c["a"], [2, 2]), arr(c["b"], [2, 2]), alpha=c["alpha"], beta=c["beta"], C=arr(c["c0"], [2, 2]))
    np.testing.assert_array_equal(out.ravel(), arr(c["c"]))


def check_bmm_bwd(be):
    for c in LIT["bmm_bwd"]:
        A, B = arr(c["a"], c["a_shape"]), arr(c["b"], c["b_shape"])
        Cf = callers.bmm(be, A, B, bool(c["ta"]), bool(c["tb"]))
        gA, gB = callers.bmm_backward(be, A, B, bool(c["ta"]), bool(c["tb"]), np.ones_like(Cf))
        np.testing.assert_array_equal(gA.ravel(), arr(c["grad_a"]), err_msg=str(c))
        np.testing.assert_array_equal(gB.ravel(), arr(c["grad_b"]), err_msg=str(c))


def check_matvec_dot(be):
    c = LIT["matvec"]
    np.testing.assert_array_equal(be.matvec(arr(c["a"]), arr(c["x"]), 2, 2, False), arr(c["y"]))
    assert be.dot(arr([1, 2, 3]), arr([1, 1, 1])) == LIT["dot"]["expected_sum"]


def check_reductions(be):
    c = LIT["sum_along"]
    np.testing.assert_array_equal(be.sum_along(arr(c["x"]), c["shape"], c["dim"]), arr(c["y"]))
    c = LIT["max_along"]
    for d in (0, 1, 2):
        np.testing.assert_array_equal(be.max_along(arr(c["x"]), c["shape"], d), arr(c["dim%d" % d]))


def check_gather(be):
    c = LIT["gather"]
    out = callers.gather_dim(be, arr(c["x"]), c["shape"], c["index"], c["index_shape"], c["dim"])
    np.testing.assert_array_equal(out, arr(c["y"]))


def check_clip_clamp(be):
    c = LIT["clip_norm"]
    assert be.nrm2(arr(c["x"])) == c["norm"]
    out = be.clip_nrm2(arr(c["x"]), c["max_norm"], c["delta"])
    np.testing.assert_allclose(out, arr(c["y"]), atol=c["atol"], rtol=0)
    assert be.nrm2(out) <= c["max_norm"]
    c = LIT["clamp"]
    x = arr(c["x"])
    np.testing.assert_array_equal(be.clamp_fwd(x, c["lo"], c["hi"]), arr(c["y"]))
    np.testing.assert_array_equal(be.clamp_bwd(x, np.zeros_like(x), np.ones_like(x), c["lo"], c["hi"]), arr(c["grad"]))


def check_add_broadcast(be):
    for c in LIT["add_bcast"]:
        z, gx, gy = callers.add_forward_backward(be, arr(c["x"]), c["x_shape"], arr(c["y"]), c["y_shape"])
        np.testing.assert_array_equal(z, arr(c["z"]))
        np.testing.assert_array_equal(gy, arr(c["grad_y"]))
        np.testing.assert_array_equal(gx, np.ones_like(gx))


def check_mul_div_bwd(be):
    c = LIT["div_bwd"]
    a, b = arr(c["a"]), arr(c["b"])
    ga, gb = callers.div_backward(be, a, b, np.ones_like(a))
    np.testing.assert_array_equal(ga, arr(c["grad_a"]))
    np.testing.assert_array_equal(gb, arr(c["grad_b"]))
    c = LIT["mul_add_bwd"]
    w, x = arr(c["w"]), arr(c["x"])
    gw, gx = callers.mul_backward(be, w, x, np.ones_like(w))
    np.testing.assert_array_equal(gw, arr(c["grad_w"]))
    np.testing.assert_array_equal(gx, w)
    c = LIT["inplace_add"]
    # x = u*v (ones), then a.add_(x), b.add_(x), c.add_(x): x = 4; every grad = seed grad
    x = be.elwise("mul", np.ones(4, np.float32), np.ones(4, np.float32))
    for _ in range(3):
        x = be.elwise("add", np.ones(4, np.float32), x)
    np.testing.assert_array_equal(x, arr(c["x"]))
    g = np.full(4, c["seed_grad"], np.float32)
    for _ in range(3):  # InplaceAddBwd: unbroadcast(alpha=1, beta=1) into a zero-filled grad
        ga = be.unbroadcast(g, [2, 2], np.zeros(4, np.float32), [2, 2], 1.0, 1.0)
        np.testing.assert_array_equal(ga, arr(c["grads"]))
    gu, gv = callers.mul_backward(be, np.ones(4, np.float32), np.ones(4, np.float32), g)
    np.testing.assert_array_equal(gu, arr(c["grads"]))
    np.testing.assert_array_equal(gv, arr(c["grads"]))


def check_losses(be):
    # tolerances are the reference's own: abs 1e-4 on the loss, rel 1e-4 on the grad
    for key in ("softmax_crossentropy_1d", "softmax_crossentropy_2d"):
        c = TORCH[key]
        loss, grad, _ = be.softmax_ce(arr(c["input"], c["shape"]), arr(c["target"], c["shape"]))
        assert abs(loss - c["loss"]) <= 1e-4, (key, loss, c["loss"])
        np.testing.assert_allclose(grad.ravel(), arr(c["input_grad"]), rtol=1e-4, atol=1e-7)
    c = TORCH["smooth_l1"]
    loss, grad = be.smooth_l1(arr(c["input"]), arr(c["target"]), c["beta"])
    assert abs(loss - c["loss"]) <= 1e-4
    np.testing.assert_array_equal(grad, arr(c["input_grad"]))


def check_pow_sqrt(be):
    c = LIT["pow"]
    x = arr(c["x"])
    np.testing.assert_array_equal(be.pow_fwd(x, c["exp"]), arr(c["y"]))
    np.testing.assert_array_equal(be.pow_bwd(x, np.zeros_like(x), np.ones_like(x), c["exp"], c["eps"]), arr(c["grad"]))
    c = LIT["sqrt"]
    x = arr(c["x"])
    np.testing.assert_array_equal(be.unary("sqrt", x), arr(c["y"]))
    np.testing.assert_array_equal(be.unary_bwd("sqrt", x, np.ones_like(x), np.zeros_like(x), c["eps"]), arr(c["grad"]))


ALL = [check_bmm, check_bmm_bwd, check_matvec_dot, check_reductions, check_gather, check_clip_clamp,
       check_add_broadcast, check_mul_div_bwd, check_losses, check_pow_sqrt]
