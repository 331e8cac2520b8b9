"""Worker of tests/test_gpu_peer_allreduce.py: one process per GPU (torchrun).
Each rank fills a buffer with seeded values, all-reduces it with the
peer-memory kernel several times (eagerly and from a captured graph) and
compares with the sum computed on the host in rank order; then the library
collectives of the C ABI (zg_allreduce / zg_reduce_scatter / zg_all_gather).
ZG_ALLREDUCE=2 in the environment makes the kernel under test the two-shot
variant for buffers of 16384 elements and more."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist
    from zigrad_b200.device import CudaDevice
    from zigrad_b200.dp import NcclComm, PeerAllReduce

    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # host channel only: the data path is the kernel under test
    dev = CudaDevice(local)
    comm = NcclComm.from_torch_distributed(dev)  # carries the IPC handles of the comm regions
    ok = True
    for n in (1, 7, 1024, 109386, 300001):
        ar = PeerAllReduce(dev, n, comm)
        for rep in range(3):
            host = [np.random.Generator(np.random.PCG64(1000 * rep + 10 * r + n % 7)).standard_normal(n).astype(np.float32) for r in range(world)]
            want = np.zeros(n, np.float32)
            for r in range(world):
                want = want + host[r]  # rank order, fp32: what every rank must produce bit for bit
            buf = dev.from_numpy(host[rank])
            ar(buf)
            got = dev.to_numpy(buf)
            if not np.array_equal(got, want) or ar.error():
                ok = False
                print("rank %d: mismatch n=%d rep=%d maxdiff=%g err=%d" % (rank, n, rep, np.abs(got - want).max(), ar.error()), flush=True)
            dev.mem_cache_free(buf)
        # fused SGD: params += -lr * sum, same rounding as the stand-alone update (one fma)
        g = np.random.Generator(np.random.PCG64(n + 5))
        P0 = g.standard_normal(n).astype(np.float32)
        pbuf, gbuf = dev.from_numpy(P0), dev.from_numpy(host[rank])
        ar.reduce_and_sgd(gbuf, pbuf, 0.01)
        tot = np.zeros(n, np.float32)
        for r in range(world):
            tot = tot + host[r]
        wantp = (np.float32(-0.01).astype(np.float64) * tot.astype(np.float64) + P0.astype(np.float64)).astype(np.float32)
        if not np.array_equal(dev.to_numpy(gbuf), tot) or not np.array_equal(dev.to_numpy(pbuf), wantp):
            ok = False
            print("rank %d: fused SGD mismatch n=%d" % (rank, n), flush=True)
        dev.mem_cache_free(pbuf)
        dev.mem_cache_free(gbuf)
        # the same with zero_grads: identical parameters, the gradient buffer reads back as zeros
        pbuf, gbuf = dev.from_numpy(P0), dev.from_numpy(host[rank])
        ar.reduce_and_sgd(gbuf, pbuf, 0.01, True)
        if dev.to_numpy(gbuf).any() or not np.array_equal(dev.to_numpy(pbuf), wantp):
            ok = False
            print("rank %d: fused SGD + zero mismatch n=%d" % (rank, n), flush=True)
        dev.mem_cache_free(pbuf)
        dev.mem_cache_free(gbuf)
        # replay from a captured graph: the epoch counter lives on the device
        x = np.full(n, float(rank + 1), np.float32)
        buf = dev.from_numpy(x)
        ar(buf)  # eager warm-up -> buf = sum(1..world)
        dev.sync()
        dev.capture.open()
        ar(buf)
        dev.capture.save()
        g = dev.capture.detach()
        for _ in range(3):
            g.run()
        got = dev.to_numpy(buf)
        s1 = world * (world + 1) / 2.0
        want = np.full(n, s1 * world ** 3, np.float32)  # every replay multiplies the (replicated) values by world
        if not np.allclose(got, want, rtol=1e-6) or ar.error():
            ok = False
            print("rank %d: graph replay mismatch n=%d got %g want %g" % (rank, n, got[0], want[0]), flush=True)
        g.free()
        dev.mem_cache_free(buf)
        ar.close()
    if "--time" in sys.argv:  # launch cost of the kernel alone, ranks in lockstep
        n = 109386
        ar = PeerAllReduce(dev, n, comm)
        buf = dev.from_numpy(np.zeros(n, np.float32))
        for _ in range(20):
            ar(buf)
        dev.sync()
        dist.barrier()
        ts = torch.cuda.ExternalStream(dev.stream.ptr)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        for _ in range(500):
            ar(buf)
        e1.record(ts)
        dev.sync()
        print("rank %d: %.2f us per all-reduce of %d floats over %d ranks" % (rank, e0.elapsed_time(e1) * 2.0, n, world), flush=True)
        ar.close()
    # the library collectives of the same communicator against the host sum (tolerance: the library picks the order)
    for n in (5, 4096, 300001):
        host = [np.random.Generator(np.random.PCG64(77 + 10 * r + n % 7)).standard_normal(n).astype(np.float32) for r in range(world)]
        want = np.sum(np.stack(host).astype(np.float64), axis=0)
        buf = dev.from_numpy(host[rank])
        comm.allreduce(buf)
        got = dev.to_numpy(buf)
        if np.abs(got - want).max() > 1e-5 * max(1.0, np.abs(want).max()):
            ok = False
            print("rank %d: zg_allreduce mismatch n=%d" % (rank, n), flush=True)
        dev.mem_cache_free(buf)
    c = 1000
    full = [np.random.Generator(np.random.PCG64(300 + r)).standard_normal(c * world).astype(np.float32) for r in range(world)]
    buf = dev.from_numpy(full[rank])
    comm.reduce_scatter(buf, buf.view(rank * c, c))          # in place: my part of the sum lands in my slice
    got = dev.to_numpy(buf)[rank * c:(rank + 1) * c]
    want = np.sum(np.stack(full).astype(np.float64), axis=0)[rank * c:(rank + 1) * c]
    if np.abs(got - want).max() > 1e-5 * max(1.0, np.abs(want).max()):
        ok = False
        print("rank %d: zg_reduce_scatter mismatch" % rank, flush=True)
    dev.mem_fill(buf, 0.0)
    dev.mem_transfer_htod(np.full(c, float(rank + 1), np.float32), buf.view(rank * c, c))
    comm.all_gather(buf.view(rank * c, c), buf)              # in place
    if not np.array_equal(dev.to_numpy(buf), np.repeat(np.arange(1, world + 1, dtype=np.float32), c)):
        ok = False
        print("rank %d: zg_all_gather mismatch" % rank, flush=True)
    dev.mem_cache_free(buf)
    comm.close()
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        print("PEER_ALLREDUCE_OK" if all(flags) else "PEER_ALLREDUCE_FAILED", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
