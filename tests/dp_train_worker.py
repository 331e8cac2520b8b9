"""Worker of tests/test_gpu_dp_train.py (torchrun, one process per GPU): 100 SGD
steps of the 784-128-64-10 MLP on ONE global batch of 8192 rows sharded over
the ranks (contiguous row blocks, loss divided by the global batch, one
all-reduce of the flat gradient buffer fused with the update), against the
CPU oracle training on the whole batch.  Checks: the summed shard losses follow
the oracle's loss curve within 1e-3 relative at every step, the final
weights agree within 5e-4 (biases 1e-2) per tensor, and the replicas are
bit-identical."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

DIMS, GLOBAL_B, STEPS, LR, SEED = [784, 128, 64, 10], 8192, 100, 0.01, 81761


def main():
    import torch
    import torch.distributed as dist
    import oracle
    from zigrad_b200.device import CudaDevice
    from zigrad_b200.dp import GradAllReduce, NcclComm, PeerAllReduce, shard_rows
    from zigrad_b200.mlp import MlpTrainer, kaiming_uniform

    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    mode = sys.argv[1] if len(sys.argv) > 1 else "peer"
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # host channel only
    dev = CudaDevice(local)
    comm = NcclComm.from_torch_distributed(dev)
    g = np.random.Generator(np.random.PCG64(7))
    X = g.uniform(0, 1, (GLOBAL_B, DIMS[0])).astype(np.float32)
    T = np.eye(DIMS[-1], dtype=np.float32)[g.integers(0, DIMS[-1], GLOBAL_B)]
    Ws, bs = kaiming_uniform(DIMS, SEED)
    lo, hi = shard_rows(GLOBAL_B, world, rank)
    B = hi - lo
    tr = MlpTrainer(dev, DIMS, B, Ws, bs, "sgd", lr=LR, fused=True, loss_div=GLOBAL_B, zero_grads_in_update=(mode == "peer"))
    red = PeerAllReduce(dev, tr.n_params, comm) if mode == "peer" else GradAllReduce(comm=comm)
    Xd, Td = dev.from_numpy(X[lo:hi]), dev.from_numpy(T[lo:hi])
    losses = dev.from_numpy(np.zeros(STEPS, np.float32))
    for s in range(STEPS):
        tr.step(Xd, Td, red)
        dev.mem_copy(tr.loss, losses.view(s, 1))
    comm.allreduce(losses)  # shard losses (each already divided by the global batch) add up to the batch loss
    got = dev.to_numpy(losses)
    ok = True
    if mode == "peer" and red.error():
        ok = False
        print("rank %d: the peer all-reduce gave up" % rank, flush=True)
    # replicas bit-identical: every rank's parameter bytes against rank 0's
    flat = dev.to_numpy(tr.params)
    everyone = [None] * world
    dist.all_gather_object(everyone, flat.tobytes())
    if any(b != everyone[0] for b in everyone):
        ok = False
        print("rank %d: replicas differ" % rank, flush=True)
    if rank == 0:
        oracle.set_threads(os.cpu_count() or 1)
        ref = oracle.MlpOracle(DIMS, Ws, bs, "sgd", lr=LR)
        want = np.array([ref.step(X, T) for _ in range(STEPS)], np.float32)
        rel = np.abs(got - want) / np.abs(want)
        print("loss curve: first %.6f -> last %.6f (oracle %.6f -> %.6f), max rel err %.2e" % (got[0], got[-1], want[0], want[-1], rel.max()), flush=True)
        if rel.max() > 1e-3:
            ok = False
            print("loss curve off by %.3e at step %d" % (rel.max(), int(rel.argmax())), flush=True)
        Wg, bg = tr.get_params()
        # 100 updates on: weights (dominated by their initial values) within 5e-4 of their largest entry;
        # biases, which start at zero and ARE the accumulated updates, within 1e-2 of theirs.  (The 1e-4
        # per-tensor bound is for one forward/backward; over 100 steps the bound is the loss curve above.)
        for l in range(len(DIMS) - 1):
            for name, a, b, tol in (("W", Wg[l], ref.W[l], 5e-4), ("b", bg[l], ref.b[l], 1e-2)):
                err = np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
                if err > tol:
                    ok = False
                    print("%s%d differs from the oracle by %.3e" % (name, l, err), flush=True)
    if mode == "peer":
        red.close()
    comm.close()
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        print("DP_TRAIN_OK" if all(flags) else "DP_TRAIN_FAILED", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
