"""The fused middle of the MLP step (opspec.mlp_tail / zg_mlp_tail_fwd_bwd) against the CPU
oracle running the same chain as separate ops: Linear + ReLU, Linear, softmax cross-entropy
forward and backward, the two dX products with their ReLU masks and the three bias gradients.
fp32 tensors within 1e-4 of the tensor's largest entry (the bound of the hot path), loss 1e-5
relative, argmax of the logits bit-exact."""
import numpy as np
import pytest

import oracle
from zigrad_b200 import opspec
from zigrad_b200.abi import SINGLE

from .backends import GpuBackend
from .test_gpu_ops import rel_err, rng

pytestmark = pytest.mark.gpu

H1, H2 = 128, 64


def mm(A, B, ta, tb):
    m = A.shape[1] if ta else A.shape[0]
    k = A.shape[0] if ta else A.shape[1]
    n = B.shape[0] if tb else B.shape[1]
    C = np.zeros((m, n), np.float32)
    return oracle.matmul(np.ascontiguousarray(A), np.ascontiguousarray(B), C, m, n, k, ta, tb, A.shape[1], B.shape[1], n, 1.0, 0.0)


def tail_oracle(act0, W1, b1, W2, b2, T, div):
    """The reference's op sequence on the host (model.zig:100-112, loss.zig:130-215, ndtensor.zig:1092-1136)."""
    act1 = np.maximum(mm(act0, W1, False, True) + b1[None, :], 0).astype(np.float32)
    logits = (mm(act1, W2, False, True) + b2[None, :]).astype(np.float32)
    loss, sm = oracle.softmax_ce_fwd(logits, T, div)
    dlog = np.zeros(logits.size, np.float32)
    oracle.softmax_ce_bwd(sm.ravel(), T.ravel(), dlog, div)
    dlog = dlog.reshape(logits.shape)
    dact1 = mm(dlog, W2, False, False)
    dact1[act1 <= 0] = 0
    dact0 = mm(dact1, W1, False, False)
    dact0[act0 <= 0] = 0
    return act1, logits, loss, dlog, dact1, dact0, dlog.sum(0), dact1.sum(0), dact0.sum(0)


@pytest.mark.parametrize("ready", [False, True], ids=["weights-after-the-wait", "weights-before-the-wait"])
@pytest.mark.parametrize("rows,C,ld,index,div", [(128, 10, 12, False, 128), (8192, 10, 12, False, 8192), (300, 10, 10, True, 300),
                                                 (1, 7, 8, False, 64), (1000, 16, 16, True, 65536), (4099, 3, 4, False, 4099),
                                                 (777, 10, 12, "soft", 777)])
def test_tail_matches_the_separate_ops_of_the_oracle(gpu, rows, C, ld, index, div, ready):
    """`index`: u64 class indices, one-hot rows, or ("soft") probability rows with every class non-zero;
    `ready`: the weights are fetched before / after the kernel's dependency wait."""
    g = rng(rows * 31 + C)
    act0 = np.maximum(g.standard_normal((rows, H1)), 0).astype(np.float32)   # post-ReLU: about half zeros
    W1 = g.uniform(-0.2, 0.2, (H2, H1)).astype(np.float32)
    b1 = g.uniform(-0.1, 0.1, H2).astype(np.float32)
    W2 = g.uniform(-0.3, 0.3, (C, H2)).astype(np.float32)
    b2 = g.uniform(-0.1, 0.1, C).astype(np.float32)
    lab = g.integers(0, C, rows)
    T = np.eye(C, dtype=np.float32)[lab]
    if index == "soft":
        e = np.exp(g.standard_normal((rows, C))).astype(np.float32)
        T = (e / e.sum(1, keepdims=True)).astype(np.float32)
    want = tail_oracle(act0, W1, b1, W2, b2, T, div)
    be = GpuBackend(gpu)
    d_act0, d_W1, d_b1, d_W2, d_b2 = be.up(act0), be.up(W1), be.up(b1), be.up(W2), be.up(b2)
    d_lab = be.up(lab.astype(np.uint64), np.uint64) if index is True else be.up(T)
    sentinel = 7.5  # padding columns of logits / dlogits must not be touched
    d_act1, d_logits, d_dlog = be.up(np.zeros((rows, H2))), be.up(np.full((rows, ld), sentinel)), be.up(np.full((rows, ld), sentinel))
    d_dact1, d_dact0 = be.up(np.zeros((rows, H2))), be.up(np.zeros((rows, H1)))
    db0_init = g.standard_normal(H1).astype(np.float32)                      # bias gradients are ADDED
    d_db2, d_db1, d_db0, d_loss = be.up(np.zeros(C)), be.up(np.zeros(H2)), be.up(db0_init), be.up(np.full(1, -1.0))
    assert gpu.mlp_tail_supported(SINGLE, H1, H2, C)
    gpu.dispatch(opspec.mlp_tail(d_act0, d_W1, d_b1, d_W2, d_b2, d_lab, rows, H1, H2, C, ld, float(div), d_act1, d_logits, d_loss, d_dlog,
                                 d_dact1, d_dact0, d_db2, d_db1, d_db0, weights_ready=ready))
    got_act1 = gpu.to_numpy(d_act1, (rows, H2))
    got_logits, got_dlog = gpu.to_numpy(d_logits, (rows, ld)), gpu.to_numpy(d_dlog, (rows, ld))
    got_dact1, got_dact0 = gpu.to_numpy(d_dact1, (rows, H2)), gpu.to_numpy(d_dact0, (rows, H1))
    got_db2, got_db1, got_db0 = gpu.to_numpy(d_db2), gpu.to_numpy(d_db1), gpu.to_numpy(d_db0)
    got_loss = float(be.down(d_loss)[0])                                     # also checks the guard regions of every operand
    act1, logits, loss, dlog, dact1, dact0, db2, db1, db0 = want
    assert abs(got_loss - loss) <= 1e-5 * abs(loss), (got_loss, loss)
    assert np.all(got_logits[:, C:] == sentinel) and np.all(got_dlog[:, C:] == sentinel)
    np.testing.assert_array_equal(np.argmax(got_logits[:, :C], 1), np.argmax(logits, 1))
    # a pre-activation within rounding of zero may land on the other side of the ReLU: compare where the masks agree
    flip = (got_act1 > 0) != (act1 > 0)
    assert flip.mean() <= 1e-4 and np.all(np.maximum(got_act1, act1)[flip] <= 1e-5)
    touched = flip.any(1)
    for name, a, b in (("act1", got_act1, act1), ("logits", got_logits[:, :C], logits), ("dlogits", got_dlog[:, :C], dlog),
                       ("dact1", np.where(flip, 0, got_dact1), np.where(flip, 0, dact1)), ("dact0", got_dact0[~touched], dact0[~touched])):
        assert rel_err(a, b) <= 1e-4, (name, rel_err(a, b))
    for name, a, b in (("db2", got_db2, db2), ("db1", got_db1, db1), ("db0", got_db0 - db0_init, db0)):
        assert np.abs(a - b).max() <= 1e-4 * max(np.abs(b).max(), np.abs(dlog).max()) + 1e-6 * np.abs(db0_init).max(), (name, a[:4], b[:4])


def test_tail_refuses_other_widths(dev):
    from zigrad_b200 import abi
    assert not dev.mlp_tail_supported(SINGLE, 256, 64, 10)
    assert not dev.mlp_tail_supported(SINGLE, 128, 64, 17)
    L = abi.lib()
    L.zg_clear_error()
    x = dev.from_numpy(np.zeros(16, np.float32))
    L.zg_mlp_tail_fwd_bwd(SINGLE, dev.stream, 1, 256, 64, 10, x.ptr, x.ptr, x.ptr, x.ptr, x.ptr, x.ptr, 0, 10, 1.0, x.ptr, x.ptr, x.ptr,
                          x.ptr, x.ptr, x.ptr, x.ptr, x.ptr, x.ptr, 0)
    assert L.zg_last_error() == 5  # kUnsupported, nothing launched
    L.zg_clear_error()
    dev.mem_cache_free(x)
