"""Worker of tests/test_gpu_zero_dp.py (torchrun, one process per GPU): the
optimizer-sharded data-parallel step against the plain data-parallel step
(all-reduce + replicated Adam) on the same seeded inputs."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist
    from zigrad_b200.abi import BF16
    from zigrad_b200.device import CudaDevice
    from zigrad_b200.dp import NcclComm, OverlappedGradAllReduce, ZeroShardedAdam
    from zigrad_b200.mlp import MlpTrainer, kaiming_uniform

    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # host channel only: the collectives are the library's own (C ABI)
    dev = CudaDevice(local)
    comm = NcclComm.from_torch_distributed(dev)
    dims, B = [256, 256, 128, 64], 256
    Ws, bs = kaiming_uniform(dims, 5)
    g = np.random.Generator(np.random.PCG64(100 + rank))
    X = g.standard_normal((B, dims[0])).astype(np.float32)
    lab = g.integers(0, dims[-1], B).astype(np.uint64)
    xf = dev.from_numpy(X)
    Xd = dev.mem_cache_alloc(BF16, X.size)
    dev.cast(xf, Xd)
    Td = dev.from_numpy(lab)
    mk = lambda: MlpTrainer(dev, dims, B, Ws, bs, "adam", lr=1e-3, clip=True, max_norm=0.05, bf16=True, loss_div=B * world)
    a, b = mk(), mk()
    red, zopt = OverlappedGradAllReduce(comm), ZeroShardedAdam(b, comm)
    ok = True
    for step in range(3):
        a.forward(Xd); a.loss_and_grad(Td)
        a.backward(Xd, on_layer_grads=lambda l: red.start(a.layer_grads(l)))
        red.finish()
        a.update()
        b.forward(Xd); b.loss_and_grad(Td)
        b.backward(Xd, on_layer_grads=zopt.start)
        zopt.finish()
        dev.sync()
        la, lb = a.read_loss(), b.read_loss()
        wa = (dev.to_numpy(a.params_bf16).astype(np.uint32) << 16).view(np.float32)
        wb = (dev.to_numpy(b.params_bf16).astype(np.uint32) << 16).view(np.float32)
        err = np.abs(wa - wb).max() / np.abs(wa).max()
        # step 0 starts from identical weights; later steps differ by bf16 ulps of single weights (the
        # two collectives add in different orders and Adam turns a near-zero gradient's sign into +-lr)
        if abs(la - lb) > (1e-5 if step == 0 else 2e-3) * abs(la) or err > 1e-2:
            ok = False
            print("rank %d step %d: loss %g vs %g, bf16 weights rel err %g" % (rank, step, la, lb, err), flush=True)
        # fp32 master weights and first moments of the owned parts
        pa, pb = dev.to_numpy(a.params), dev.to_numpy(b.params)
        ma, mb = dev.to_numpy(a.m), dev.to_numpy(b.m)
        for off, n in zopt.owned:
            if not n:
                continue
            if np.abs(pa[off:off + n] - pb[off:off + n]).max() > 1e-2 * np.abs(pa).max():
                ok = False
                print("rank %d step %d: owned master slice at %d differs" % (rank, step, off), flush=True)
            tol = (1e-5 if step == 0 else 2e-2) * np.abs(ma).max()
            if np.abs(ma[off:off + n] - mb[off:off + n]).max() > tol:
                ok = False
                print("rank %d step %d: owned first moment at %d differs by %g (tol %g)" % (rank, step, off, np.abs(ma[off:off + n] - mb[off:off + n]).max(), tol), flush=True)
    assert a.read_t() == b.read_t() == 3 * 6
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        print("ZERO_DP_OK" if all(flags) else "ZERO_DP_FAILED", flush=True)
    comm.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
