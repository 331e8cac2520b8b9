"""Whole-step parity for the MLP configurations: every activation, gradient
and updated parameter after one step from identical seeded state, the loss
curve over 100 SGD steps, graph replay, Adam, clipping, and the equivalence of
a sharded (data-parallel) step with the full-batch step."""
import numpy as np
import pytest

from oracle import MlpOracle
from zigrad_b200 import opspec
from zigrad_b200.abi import SINGLE
from zigrad_b200.mlp import MlpTrainer, kaiming_uniform

from .test_gpu_ops import rel_err, rng

pytestmark = pytest.mark.gpu
DIMS = [784, 128, 64, 10]


def batch(B, seed, dims=DIMS):
    g = rng(seed)
    X = g.uniform(0.0, 1.0, (B, dims[0])).astype(np.float32)
    lab = g.integers(0, dims[-1], B)
    T = np.zeros((B, dims[-1]), np.float32)
    T[np.arange(B), lab] = 1.0
    return X, T, lab


def assert_close(name, got, want, tol=1e-4):
    e = rel_err(got, want)
    assert e <= tol, "%s: max rel err %.3g > %.1g" % (name, e, tol)


@pytest.mark.parametrize("fused", [False, True], ids=["reference-op-sequence", "fused-epilogues"])
@pytest.mark.parametrize("B", [64, 1024])
def test_one_sgd_step_every_tensor(gpu, fused, B):
    Ws, bs = kaiming_uniform(DIMS, 81761)
    bs = [rng(5 + i).standard_normal(b.size).astype(np.float32) * 0.1 for i, b in enumerate(bs)]  # non-trivial biases
    X, T, _ = batch(B, 1)
    orc = MlpOracle(DIMS, Ws, bs, "sgd", lr=0.01)
    want_loss = orc.step(X, T)
    tr = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.01, fused=fused)
    Xd, Td = gpu.from_numpy(X), gpu.from_numpy(T)
    tr.step(Xd, Td)
    got_loss = tr.read_loss()
    assert abs(got_loss - want_loss) <= 1e-4 * abs(want_loss)
    for l in range(3):
        assert_close("act%d" % l, tr.act_numpy(l), orc.act[l])
        assert_close("dact%d" % l, tr.act_numpy(l, grad=True), orc.dact[l])
    # predictions: argmax of the logits is bit-exact
    np.testing.assert_array_equal(np.argmax(tr.act_numpy(2), 1), np.argmax(orc.act[2], 1))
    gW, gb = tr.get_grads()
    pW, pb = tr.get_params()
    for l in range(3):
        assert_close("dW%d" % l, gW[l], orc.dW[l])
        assert_close("db%d" % l, gb[l], orc.db[l])
        assert_close("W%d" % l, pW[l], orc.W[l], 1e-6)
        assert_close("b%d" % l, pb[l], orc.b[l], 1e-6)
    tr.free()
    gpu.mem_cache_free(Xd)
    gpu.mem_cache_free(Td)


def test_update_that_clears_gradients_trains_like_zero_grad(gpu):
    """zero_grads_in_update: no zero_grad launch from the second step on; losses and
    parameters follow the plain trainer (same kernels otherwise; the weight
    gradients are summed with atomics, hence a tolerance), eagerly and from a
    captured graph."""
    B = 1024
    Ws, bs = kaiming_uniform(DIMS, 4242)
    plain = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.05)
    fast = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.05, zero_grads_in_update=True)
    bufs = []
    for i in range(3):
        X, T, _ = batch(B, 50 + i)
        Xd, Td = gpu.from_numpy(X), gpu.from_numpy(T)
        bufs += [Xd, Td]
        plain.step(Xd, Td)
        fast.step(Xd, Td)
        assert abs(plain.read_loss() - fast.read_loss()) <= 1e-5 * abs(plain.read_loss())
    assert not gpu.to_numpy(fast.grads).any()
    gpu.sync()
    gpu.capture.open()
    fast.step(bufs[0], bufs[1])
    gpu.capture.save()
    graph = gpu.capture.detach()
    gpu.capture.open()
    plain.step(bufs[0], bufs[1])
    gpu.capture.save()
    graph_plain = gpu.capture.detach()
    # no fill of the gradient buffer; with the tail path the three weight updates also ride in their GEMMs' epilogues
    assert graph.kernel_count() <= graph_plain.kernel_count() - 1
    for _ in range(2):
        graph.run()
        graph_plain.run()
    gpu.sync()
    pW, pb = plain.get_params()
    fW, fb = fast.get_params()
    for l in range(3):
        assert_close("W%d" % l, fW[l], pW[l], 1e-5)
        assert_close("b%d" % l, fb[l], pb[l], 1e-5)
    graph.free()
    graph_plain.free()
    plain.free()
    fast.free()
    for b_ in bufs:
        gpu.mem_cache_free(b_)


def test_update_behind_each_weight_gradient_equals_the_update_after_the_join(gpu):
    """fuse_update (the default of the tail path): every tensor is updated by an SGD launch right
    behind its gradient, on that gradient's stream.  Same kernels, same arithmetic per element as one
    SGD launch over all tensors after the join; the weight gradients are summed by reductions whose
    order varies from run to run, hence a tolerance."""
    B = 2048
    Ws, bs = kaiming_uniform(DIMS, 99)
    after = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.05, zero_grads_in_update=True, fuse_update=False)
    behind = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.05, zero_grads_in_update=True, fuse_update=True)
    assert behind.tail and behind.fuse_update
    bufs = []
    for i in range(4):
        X, T, _ = batch(B, 70 + i)
        Xd, Td = gpu.from_numpy(X), gpu.from_numpy(T)
        bufs += [Xd, Td]
        after.step(Xd, Td)
        behind.step(Xd, Td)
        assert abs(after.read_loss() - behind.read_loss()) <= 1e-5 * abs(after.read_loss())
    assert not gpu.to_numpy(behind.grads).any()  # every gradient was cleared by the launch that applied it
    aW, ab = after.get_params()
    bW, bb = behind.get_params()
    for l in range(3):
        assert_close("W%d" % l, bW[l], aW[l], 1e-5)
        assert_close("b%d" % l, bb[l], ab[l], 1e-5)
    after.free()
    behind.free()
    for b_ in bufs:
        gpu.mem_cache_free(b_)


def test_loss_over_100_sgd_steps_config2(gpu):
    """784-128-64-10 at batch 8192, 100 SGD steps over a fixed set of seeded
    batches: per-step loss within 1e-3 relative of the CPU path."""
    B, n_batches = 8192, 4
    Ws, bs = kaiming_uniform(DIMS, 81761)
    data = [batch(B, 100 + i) for i in range(n_batches)]
    orc = MlpOracle(DIMS, Ws, bs, "sgd", lr=0.01)
    want = [orc.step(*data[s % n_batches][:2]) for s in range(100)]
    tr = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.01, fused=True)
    dev = [(gpu.from_numpy(X), gpu.from_numpy(T)) for X, T, _ in data]
    got = []
    for s in range(100):
        tr.step(*dev[s % n_batches])
        got.append(tr.read_loss())
    got, want = np.asarray(got), np.asarray(want)
    assert want[-1] < want[0], "the loss should go down"
    assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-3, np.max(np.abs(got - want) / np.abs(want))
    pW, _ = tr.get_params()
    for l in range(3):
        assert_close("W%d after 100 steps" % l, pW[l], orc.W[l], 1e-4)
    tr.free()
    for a, b in dev:
        gpu.mem_cache_free(a)
        gpu.mem_cache_free(b)


def test_captured_step_replays_like_eager(gpu):
    B = 256
    Ws, bs = kaiming_uniform(DIMS, 7)
    X, T, _ = batch(B, 3)
    Xd, Td = gpu.from_numpy(X), gpu.from_numpy(T)
    eager = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.05)
    for _ in range(5):
        eager.step(Xd, Td)
    graph = MlpTrainer(gpu, DIMS, B, Ws, bs, "sgd", lr=0.05)
    graph.step(Xd, Td)  # warm-up outside the capture (workspaces grow here)
    gpu.capture.open()
    graph.step(Xd, Td)
    gpu.capture.save()
    for _ in range(4):  # nothing executes while capturing: 1 eager + 4 replays = the 5 eager steps
        gpu.capture.run()
    gpu.sync()
    # split-K weight gradients add with atomics, so two runs agree to rounding, not bit for bit
    assert abs(graph.read_loss() - eager.read_loss()) <= 1e-5 * abs(eager.read_loss())
    for a, b in zip(graph.get_params()[0], eager.get_params()[0]):
        assert_close("W", a, b, 1e-5)
    gpu.capture.free()
    eager.free()
    graph.free()
    gpu.mem_cache_free(Xd)
    gpu.mem_cache_free(Td)


@pytest.mark.parametrize("clip", [False, True])
def test_adam_steps_with_per_tensor_counter(gpu, clip):
    B = 128
    Ws, bs = kaiming_uniform(DIMS, 11)
    X, T, _ = batch(B, 4)
    orc = MlpOracle(DIMS, Ws, bs, "adam", lr=1e-3, clip=clip, max_norm=0.5 if clip else 10.0)
    tr = MlpTrainer(gpu, DIMS, B, Ws, bs, "adam", lr=1e-3, clip=clip, max_norm=0.5 if clip else 10.0)
    Xd, Td = gpu.from_numpy(X), gpu.from_numpy(T)
    for s in range(3):
        want = orc.step(X, T)
        tr.step(Xd, Td)
        assert abs(tr.read_loss() - want) <= 1e-4 * abs(want)
        gW, gb = tr.get_grads()
        for l in range(3):  # forward/backward tensors of every step: the 1e-4 bound
            assert_close("step %d dW%d" % (s, l), gW[l], orc.dW[l])
            assert_close("step %d db%d" % (s, l), gb[l], orc.db[l])
    assert tr.t == orc.t.value == 18  # 6 tensors x 3 steps
    # Updated parameters: Adam divides by sqrt(v), so an element whose gradient is
    # at rounding-noise level moves by ~lr whatever the size of that noise; the
    # update itself is checked tightly on identical inputs in test_gpu_ops.py.
    pW, pb = tr.get_params()
    for l in range(3):
        assert_close("W%d" % l, pW[l], orc.W[l], 2e-2)
        assert_close("b%d" % l, pb[l], orc.b[l], 2e-2)
    tr.free()
    gpu.mem_cache_free(Xd)
    gpu.mem_cache_free(Td)


def test_sharded_step_equals_full_batch(gpu):
    """Two row shards with the loss divided by the GLOBAL batch, gradients
    summed (what the all-reduce does), give the full-batch gradients."""
    B = 512
    Ws, bs = kaiming_uniform(DIMS, 13)
    X, T, _ = batch(B, 6)
    orc = MlpOracle(DIMS, Ws, bs, "none")
    full_loss = orc.step(X, T)
    shards = []
    for r in range(2):
        tr = MlpTrainer(gpu, DIMS, B // 2, Ws, bs, "none", loss_div=B)
        Xd, Td = gpu.from_numpy(X[r * 256:(r + 1) * 256]), gpu.from_numpy(T[r * 256:(r + 1) * 256])
        tr.step(Xd, Td)
        shards.append((tr, tr.read_loss()))
    gpu.dispatch(opspec.add(shards[0][0].grads, shards[1][0].grads, shards[0][0].grads))
    assert abs(shards[0][1] + shards[1][1] - full_loss) <= 1e-5 * abs(full_loss)
    gW, gb = shards[0][0].get_grads()
    for l in range(3):
        assert_close("dW%d" % l, gW[l], orc.dW[l])
        assert_close("db%d" % l, gb[l], orc.db[l])
    for tr, _ in shards:
        tr.free()
