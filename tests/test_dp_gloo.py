"""Host-side logic of the data-parallel step on CPU: two gloo ranks shard one
global batch by rows, each computes its gradients with the loss divided by the
GLOBAL batch (the CPU oracle stands in for the device here), the flat gradient
buffer is all-reduced through zigrad_b200.dp, and every rank applies the same
update.  The result must equal the single-process full-batch step."""
import os
import socket

import numpy as np
import pytest
import torch.multiprocessing as mp

from zigrad_b200.dp import shard_rows

DIMS = [20, 16, 8, 5]
GLOBAL_B = 37  # odd on purpose: ranks get 19 and 18 rows


def _data():
    g = np.random.Generator(np.random.PCG64(5))
    X = g.uniform(0, 1, (GLOBAL_B, DIMS[0])).astype(np.float32)
    T = np.eye(DIMS[-1], dtype=np.float32)[g.integers(0, DIMS[-1], GLOBAL_B)]
    Ws = [g.uniform(-0.3, 0.3, (o, i)).astype(np.float32) for i, o in zip(DIMS[:-1], DIMS[1:])]
    bs = [g.uniform(-0.1, 0.1, o).astype(np.float32) for o in DIMS[1:]]
    return X, T, Ws, bs


def _flat(Ws, bs):
    return np.concatenate([np.concatenate([w.ravel(), b.ravel()]) for w, b in zip(Ws, bs)])


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    import oracle
    from zigrad_b200.dp import GradAllReduce
    dist.init_process_group("gloo", rank=rank, world_size=world)
    X, T, Ws, bs = _data()
    lo, hi = shard_rows(GLOBAL_B, world, rank)
    model = oracle.MlpOracle(DIMS, Ws, bs, "none")
    loss = model.step(X[lo:hi], T[lo:hi], loss_div=GLOBAL_B)
    grads = _flat(model.dW, model.db)
    GradAllReduce().host(grads)  # one all-reduce of the flat gradient buffer
    params = _flat(model.W, model.b)
    oracle.sgd_update(params, grads, 0.05)  # update AFTER the reduction, on every rank
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), loss=loss, grads=grads, params=params)
    dist.destroy_process_group()


def test_shard_rows_partitions_the_batch():
    for B, W in [(8192, 8), (37, 2), (5, 8), (0, 4)]:
        spans = [shard_rows(B, W, r) for r in range(W)]
        assert spans[0][0] == 0 and spans[-1][1] == B
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def test_two_rank_step_equals_full_batch_step(tmp_path, orc):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    X, T, Ws, bs = _data()
    full = orc.MlpOracle(DIMS, Ws, bs, "sgd", lr=0.05)
    full_loss = full.step(X, T)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    # shard losses add up to the full-batch loss; reduced gradients are identical on both ranks
    assert abs(float(r0["loss"]) + float(r1["loss"]) - full_loss) <= 1e-6 * abs(full_loss)
    np.testing.assert_array_equal(r0["grads"], r1["grads"])
    np.testing.assert_array_equal(r0["params"], r1["params"])
    want_g = _flat(full.dW, full.db)
    assert np.max(np.abs(r0["grads"] - want_g)) <= 1e-6 * np.max(np.abs(want_g))
    want_p = _flat(full.W, full.b)
    assert np.max(np.abs(r0["params"] - want_p)) <= 1e-6 * np.max(np.abs(want_p))
