"""Mixed-precision MLP step (the wide-MLP configuration in miniature): bf16
inputs, weights and hidden activations, fp32 accumulation, fp32 logits / loss /
parameter gradients, fp32 master weights updated by Adam with a bf16 copy.

The reference is fp32/fp64 only, so the oracle here is the CPU restatement run
on bf16-ROUNDED operands (fp32 BLAS over values that are exactly representable
in bf16), rounding to bf16 at the same points as the device path.

Tolerances (max |got - want| / max |want| per tensor), stated separately from
the fp32 path as the specification allows:
  fp32 tensors computed from bf16 operands (logits, dW, db)   2e-3
  tensors STORED in bf16 (hidden activations, their grads)    1e-2  (one bf16 ulp = 3.9e-3
      of the element; a 1e-6 accumulation difference can flip a rounding)
  loss                                                        1e-3 relative
"""
import numpy as np
import pytest

import oracle
from zigrad_b200.mlp import MlpTrainer, kaiming_uniform

from .test_gpu_ops import rel_err, rng

pytestmark = pytest.mark.gpu


def r16(x):
    x = np.ascontiguousarray(x, np.float32)
    return oracle.round_bf16(x.ravel()).reshape(x.shape)


def bits(x):
    return (r16(x).view(np.uint32) >> 16).astype(np.uint16)


def mm(A, B, ta, tb):
    m = A.shape[1] if ta else A.shape[0]
    k = A.shape[0] if ta else A.shape[1]
    n = B.shape[0] if tb else B.shape[1]
    C = np.zeros((m, n), np.float32)
    return oracle.matmul(np.ascontiguousarray(A), np.ascontiguousarray(B), C, m, n, k, ta, tb, A.shape[1], B.shape[1], n, 1.0, 0.0)


def bf16_step_oracle(dims, Ws, bs, X, labels, loss_div, masks=None):
    """Forward/backward of the mixed-precision step on the CPU.  ``masks[l]``
    (bool, True where layer l's activation counts as positive) replaces the
    oracle's own ReLU mask in the backward pass when given."""
    L = len(dims) - 1
    Wb = [r16(w) for w in Ws]
    act, inp = [], r16(X)
    for l in range(L):
        z = mm(inp, Wb[l], False, True) + bs[l][None, :]
        if l + 1 < L:
            z = r16(np.maximum(z, 0))
        act.append(z.astype(np.float32))
        inp = act[-1]
    T = np.eye(dims[-1], dtype=np.float32)[labels]
    loss, sm = oracle.softmax_ce_fwd(act[-1], T, loss_div)
    dlog = ((sm - T) / np.float32(loss_div)).astype(np.float32)
    dW, db, dact = [None] * L, [None] * L, [None] * L
    db[L - 1] = dlog.sum(0)
    dy = r16(dlog)
    dact[L - 1] = dlog
    for l in range(L - 1, -1, -1):
        a_in = r16(X) if l == 0 else act[l - 1]
        if l > 0:
            dx = mm(dy, Wb[l], False, False)
            dx[(act[l - 1] <= 0) if masks is None else ~masks[l - 1]] = 0
            db[l - 1] = dx.sum(0)
            dact[l - 1] = r16(dx)
        dW[l] = mm(dy, a_in, True, False)
        if l > 0:
            dy = dact[l - 1]
    return loss, act, dact, dW, db


@pytest.mark.parametrize("dims,B", [([256, 256, 128, 1000], 512), ([512, 384, 64], 1024)])
def test_bf16_step_forward_backward(gpu, dims, B):
    g = rng(B + sum(dims))
    Ws, bs = kaiming_uniform(dims, 3)
    bs = [g.standard_normal(b.size).astype(np.float32) * 0.1 for b in bs]
    X = g.standard_normal((B, dims[0])).astype(np.float32)
    labels = g.integers(0, dims[-1], B)
    want_loss, act, dact, dW, db = bf16_step_oracle(dims, Ws, bs, X, labels, B)
    tr = MlpTrainer(gpu, dims, B, Ws, bs, "none", fused=True, bf16=True)
    Xd, Td = gpu.from_numpy(bits(X)), gpu.from_numpy(labels.astype(np.uint64))
    tr.step(Xd, Td)
    assert abs(tr.read_loss() - want_loss) <= 1e-3 * abs(want_loss)
    L = len(dims) - 1
    for l in range(L):
        tol = 2e-3 if l + 1 == L else 1e-2
        assert rel_err(tr.act_numpy(l), act[l]) <= tol, ("act", l, rel_err(tr.act_numpy(l), act[l]))
        assert rel_err(tr.act_numpy(l, grad=True), dact[l]) <= tol, ("dact", l)
    np.testing.assert_array_equal(np.argmax(tr.act_numpy(L - 1), 1), np.argmax(act[L - 1], 1)) if dims[-1] <= 64 else None
    gW, gb = tr.get_grads()
    for l in range(L):
        assert rel_err(gW[l], dW[l]) <= 2e-3, ("dW", l, rel_err(gW[l], dW[l]))
        assert rel_err(gb[l], db[l]) <= 2e-3, ("db", l, rel_err(gb[l], db[l]))
    tr.free()
    gpu.mem_cache_free(Xd)
    gpu.mem_cache_free(Td)


def test_bf16_adam_keeps_master_and_copy_in_step(gpu):
    dims, B = [256, 128, 64], 256
    g = rng(77)
    Ws, bs = kaiming_uniform(dims, 5)
    X = g.standard_normal((B, dims[0])).astype(np.float32)
    labels = g.integers(0, dims[-1], B)
    tr = MlpTrainer(gpu, dims, B, Ws, bs, "adam", lr=1e-3, fused=True, bf16=True, clip=True)
    Xd, Td = gpu.from_numpy(bits(X)), gpu.from_numpy(labels.astype(np.uint64))
    losses = []
    for _ in range(5):
        tr.step(Xd, Td)
        losses.append(tr.read_loss())
    assert losses[-1] < losses[0]
    master = gpu.to_numpy(tr.params)
    copy = gpu.to_numpy(tr.params_bf16)
    np.testing.assert_array_equal(copy, bits(master))  # the bf16 copy is the RNE rounding of the master, bit for bit
    assert tr.t == 4 * 5
    tr.free()
    gpu.mem_cache_free(Xd)
    gpu.mem_cache_free(Td)


@pytest.mark.parametrize("clip", [False, True])
def test_adam_a_layer_at_a_time_during_backward_equals_one_update_after_it(gpu, clip):
    """update_by_layer: every layer's tensors are updated on a side stream as soon as the layer's
    gradients are final and nothing reads its weights any more.  Same kernels and segment positions
    as one Adam launch over the whole model; the step counts agree exactly, parameters and moments
    to the run-to-run spread of the split-K weight gradients (their partial products are summed in
    an order that varies), eagerly and from a replayed graph."""
    dims, B = [256, 384, 128, 64], 512
    g = rng(31)
    Ws, bs = kaiming_uniform(dims, 8)
    X = g.standard_normal((B, dims[0])).astype(np.float32)
    labels = g.integers(0, dims[-1], B)
    one = MlpTrainer(gpu, dims, B, Ws, bs, "adam", lr=1e-3, fused=True, bf16=True, clip=clip, max_norm=0.05, update_by_layer=False)
    lay = MlpTrainer(gpu, dims, B, Ws, bs, "adam", lr=1e-3, fused=True, bf16=True, clip=clip, max_norm=0.05, update_by_layer=True)
    Xd, Td = gpu.from_numpy(bits(X)), gpu.from_numpy(labels.astype(np.uint64))
    for _ in range(3):
        one.step(Xd, Td)
        lay.step(Xd, Td)
    graphs = []
    for tr in (one, lay):
        gpu.sync()
        gpu.capture.open()
        tr.step(Xd, Td)
        gpu.capture.save()
        graphs.append(gpu.capture.detach())
    for _ in range(2):
        for gr in graphs:
            gr.run()
    gpu.sync()
    assert one.read_t() == lay.read_t() == 6 * 5  # six tensors, five steps (three eager, two replays; capturing runs nothing)
    for name, tol in (("params", 1e-5), ("m", 1e-4), ("v", 1e-4)):
        assert rel_err(gpu.to_numpy(getattr(lay, name)), gpu.to_numpy(getattr(one, name))) <= tol, name
    widen = lambda a: (a.astype(np.uint32) << 16).view(np.float32)
    assert rel_err(widen(gpu.to_numpy(lay.params_bf16)), widen(gpu.to_numpy(one.params_bf16))) <= 8e-3  # a bf16 ulp where a rounding flips
    np.testing.assert_array_equal(gpu.to_numpy(lay.params_bf16), bits(gpu.to_numpy(lay.params)))  # the copy is the rounding of ITS master
    assert abs(one.read_loss() - lay.read_loss()) <= 1e-5 * abs(one.read_loss())
    for gr in graphs:
        gr.free()
    one.free()
    lay.free()
    gpu.mem_cache_free(Xd)
    gpu.mem_cache_free(Td)


def test_wide_mlp_full_size_shard_against_the_oracle(gpu):
    """The wide-MLP configuration at its real size: one GPU's 8192-row shard of
    4096->4096->4096->4096->1000 (the persistent 128x256-tile bf16 kernels and the
    staged softmax kernel at the shapes the benchmark runs), one forward/backward
    against the CPU oracle on bf16-rounded operands.  About 2.4 TFLOP of OpenBLAS
    on the host cores: seconds."""
    dims, B = [4096, 4096, 4096, 4096, 1000], 8192
    oracle.set_threads(__import__("os").cpu_count() or 1)
    g = rng(4096)
    Ws, bs = kaiming_uniform(dims, 5)
    bs = [g.standard_normal(b.size).astype(np.float32) * 0.05 for b in bs]
    X = g.standard_normal((B, dims[0])).astype(np.float32)
    labels = g.integers(0, dims[-1], B)
    tr = MlpTrainer(gpu, dims, B, Ws, bs, "none", fused=True, bf16=True, loss_div=65536)
    Xd, Td = gpu.from_numpy(bits(X)), gpu.from_numpy(labels.astype(np.uint64))
    tr.step(Xd, Td)
    L = len(dims) - 1
    got_act = [tr.act_numpy(l) for l in range(L)]
    # ReLU is discontinuous in its mask: among 33.5 M pre-activations per layer some lie within an
    # accumulation-order difference of zero and land on different sides, which switches that element's
    # gradient on or off -- and, one layer further down, shifts the WHOLE row of dX = dY.W that the
    # element feeds.  Behind the first layer the inputs themselves differ by bf16 roundings (one ulp on
    # a fraction of a percent of them), which moves a pre-activation by about 1e-3 of its spread, so a
    # few 1e-4 of the elements flip.  The forward pass is compared as it stands, the flips must stay
    # that rare and confined to activations near zero, and the backward pass of the oracle then runs on
    # the DEVICE's masks, so that every gradient is compared in full at the stated tolerance.
    want_loss, act, dact, dW, db = bf16_step_oracle(dims, Ws, bs, X, labels, 65536, masks=[a > 0 for a in got_act[:-1]])
    assert abs(tr.read_loss() - want_loss) <= 1e-3 * abs(want_loss), (tr.read_loss(), want_loss)
    # Tolerances as in the miniature test, except the logits: they sit behind three bf16-rounded layers
    # of 4096 terms each, and an activation that rounds to a neighbouring bf16 value on one side moves
    # 4096 products of the next layer: 4e-3 of the largest logit instead of 2e-3.
    for l in range(L):
        tol = 4e-3 if l + 1 == L else 1e-2
        assert rel_err(got_act[l], act[l]) <= tol, ("act", l, rel_err(got_act[l], act[l]))
        if l + 1 < L:
            flip = (got_act[l] > 0) != (act[l] > 0)
            assert flip.mean() <= 1e-3, ("mask flips", l, flip.mean())
            assert np.all(np.maximum(got_act[l], act[l])[flip] <= 1e-2 * np.abs(act[l]).max()), ("flip away from zero", l)
        gd = tr.act_numpy(l, grad=True)
        assert rel_err(gd, dact[l]) <= tol, ("dact", l, rel_err(gd, dact[l]))
    # The weight gradients sum 8192 rows of bf16-stored dY whose entries differ from the oracle's by a
    # rounding here and there (the 1e-2 above); three layers down that is 3e-3 of the largest entry of
    # dW[0], so 5e-3 here instead of the miniature's 2e-3.
    gW, gb = tr.get_grads()
    for l in range(L):
        assert rel_err(gW[l], dW[l]) <= 5e-3, ("dW", l, rel_err(gW[l], dW[l]))
        assert rel_err(gb[l], db[l]) <= 5e-3, ("db", l, rel_err(gb[l], db[l]))
    tr.free()
    gpu.mem_cache_free(Xd)
    gpu.mem_cache_free(Td)
