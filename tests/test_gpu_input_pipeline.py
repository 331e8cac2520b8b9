"""BatchStager: batches staged from pinned host memory on the copy stream reach
the step intact and in order, also when the copies overlap running steps."""
import numpy as np
import pytest

import oracle
from zigrad_b200.abi import SINGLE
from zigrad_b200.input_pipeline import BatchStager
from zigrad_b200.mlp import MlpTrainer, kaiming_uniform

pytestmark = pytest.mark.gpu


def test_staged_batches_give_the_same_losses_as_resident_batches(gpu):
    dims, B, steps = [64, 32, 10], 512, 6
    g = np.random.Generator(np.random.PCG64(8))
    Ws, bs = kaiming_uniform(dims, 4)
    data = []
    for i in range(steps):
        X = g.uniform(0, 1, (B, dims[0])).astype(np.float32)
        T = np.eye(dims[-1], dtype=np.float32)[g.integers(0, dims[-1], B)]
        data.append((X, T))
    cpu = oracle.MlpOracle(dims, Ws, bs, "sgd", lr=0.05)  # the reference's host path on the same batches
    want_cpu = [cpu.step(X, T) for X, T in data]
    ref = MlpTrainer(gpu, dims, B, Ws, bs, "sgd", lr=0.05)
    want = []
    for X, T in data:
        Xd, Td = gpu.from_numpy(X), gpu.from_numpy(T)
        ref.step(Xd, Td)
        want.append(ref.read_loss())
        gpu.mem_cache_free(Xd)
        gpu.mem_cache_free(Td)
    tr = MlpTrainer(gpu, dims, B, Ws, bs, "sgd", lr=0.05)
    st = BatchStager(gpu, [(B * dims[0], SINGLE), (B * dims[-1], SINGLE)])
    pinned = [(st.pinned_like(X), st.pinned_like(T)) for X, T in data]
    losses = gpu.from_numpy(np.zeros(steps, np.float32))
    st.put(pinned[0])
    for i in range(steps):
        if i + 1 < steps:
            st.put(pinned[i + 1])
        Xd, Td = st.get()
        tr.step(Xd, Td)
        gpu.mem_copy(tr.loss, losses.view(i, 1))
        st.release()
    got = gpu.to_numpy(losses)
    for a, b in zip(got, want):
        assert abs(a - b) <= 1e-6 * abs(b), (got, want)
    for a, b in zip(got, want_cpu):  # a stale or half-copied batch would show up as a different loss curve
        assert abs(a - b) <= 1e-4 * abs(b), (got, want_cpu)
    Wg, bg = tr.get_params()
    for l in range(len(dims) - 1):
        assert np.abs(Wg[l] - cpu.W[l]).max() <= 1e-4 * np.abs(cpu.W[l]).max()
    with pytest.raises(RuntimeError):
        st.get()
    st.close()
    ref.free()
    tr.free()
    gpu.mem_cache_free(losses)


def test_packed_batches_with_index_labels_follow_the_oracle(gpu):
    """One copy per batch (pixels and u64 class indices packed into one pinned buffer) and the
    documented put-before-get order: losses follow the CPU oracle fed with one-hot rows."""
    from zigrad_b200.device import USIZE
    dims, B, steps = [48, 32, 10], 256, 5
    g = np.random.Generator(np.random.PCG64(18))
    Ws, bs = kaiming_uniform(dims, 6)
    data = []
    for i in range(steps):
        X = g.uniform(0, 1, (B, dims[0])).astype(np.float32)
        lab = g.integers(0, dims[-1], B).astype(np.uint64)
        data.append((X, lab))
    cpu = oracle.MlpOracle(dims, Ws, bs, "sgd", lr=0.05)
    want = [cpu.step(X, np.eye(dims[-1], dtype=np.float32)[lab.astype(np.int64)]) for X, lab in data]
    tr = MlpTrainer(gpu, dims, B, Ws, bs, "sgd", lr=0.05, index_labels=True)
    st = BatchStager(gpu, [(B * dims[0], SINGLE), (B, USIZE)], packed=True)
    assert st.bytes_per_batch() == B * dims[0] * 4 + B * 8   # both sizes are multiples of 256 here: no padding
    packed = [st.pack([X, lab]) for X, lab in data]
    losses = gpu.from_numpy(np.zeros(steps, np.float32))
    st.put(packed[0])
    for i in range(steps):
        if i + 1 < steps:
            st.put(packed[i + 1])
        Xd, Td = st.get()
        tr.step(Xd, Td)
        gpu.mem_copy(tr.loss, losses.view(i, 1))
        st.release()
    got = gpu.to_numpy(losses)
    for a, b in zip(got, want):
        assert abs(a - b) <= 1e-4 * abs(b), (got, want)
    st.close()
    tr.free()
    gpu.mem_cache_free(losses)
