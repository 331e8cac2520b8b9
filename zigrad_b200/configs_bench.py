"""Timing of the other benchmark configurations on one GPU (bench.py at the
repository root covers the headline one, the batch-8192 MLP, and calls run()
and run_c3_dp() of this module for its "configs" record).

    python -m zigrad_b200.configs_bench [--configs c1,c3,c4,c5]
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m zigrad_b200.configs_bench --dp

  c1  MLP 784-128-64-10, batch 64, fp32 (3xTF32), SGD           -> samples/s, us/step
  c3  MLP 4096-4096-4096-4096-1000, bf16 + fp32 master, Adam, one GPU's 8192-row
      shard of the global batch of 65536                         -> samples/s, TFLOP/s
  c4  2-layer GCN, dense adjacency, 2708 nodes, Adam, full batch -> steps/s
  c5  DQN 4-128-128-2 (policy + target), batch 256, Huber, Adam  -> us/step

Every step is captured into one CUDA graph and replayed; times come from CUDA
events on the device stream.  Inputs are seeded synthetic tensors
(zigrad_b200.synthetic).  A caller that wants a host-side timing of the same
step beside each row passes `host_leg(name, **inputs) -> dict`: it receives the
host arrays a configuration was built from and returns keys to merge into the
row (bench.py times the CPU path that way).  One JSON line per configuration.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np


def _graph_time(dev, ts, fn, reps):
    import torch
    fn()  # eager warm-up: workspaces grow here
    dev.sync()
    dev.capture.open()
    fn()
    dev.capture.save()
    g = dev.capture.detach()
    for _ in range(5):
        g.run()
    dev.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ts)
    for _ in range(reps):
        g.run()
    e1.record(ts)
    dev.sync()
    us = e0.elapsed_time(e1) * 1e3 / reps
    n = g.kernel_count()
    g.free()
    return us, n


def run(configs, reps=200, dev=None, ts=None, host_leg=None):
    import torch
    from . import synthetic
    from .device import CudaDevice
    from .dqn import DqnTrainer
    from .gcn import GcnTrainer
    from .mlp import MlpTrainer, kaiming_uniform

    if dev is None:
        ts = torch.cuda.Stream()
        dev = CudaDevice(0, stream=ts.cuda_stream)
    leg = host_leg or (lambda name, **kw: {})
    out = []

    if "c1" in configs:
        dims, B = [784, 128, 64, 10], 64
        Ws, bs = kaiming_uniform(dims, 81761)
        X, T, _ = synthetic.mlp_batch(B, 784, 10, 1)
        tr = MlpTrainer(dev, dims, B, Ws, bs, "sgd", lr=0.01, zero_grads_in_update=True)  # as the headline run: no zero_grad launch, updates inside the gradient GEMMs
        Xd, Td = dev.from_numpy(X), dev.from_numpy(T)
        us, n = _graph_time(dev, ts, lambda: tr.step(Xd, Td), reps * 5 if reps >= 50 else reps)
        row = {"config": "c1 MLP 784-128-64-10 b64 fp32 SGD", "us_per_step": us, "samples_per_s": B / us * 1e6, "kernels": n}
        row.update(leg("c1", dims=dims, Ws=Ws, bs=bs, X=X, T=T))
        out.append(row)
        tr.free()
        dev.mem_cache_free(Xd)
        dev.mem_cache_free(Td)

    if "c3" in configs:
        dims, B = [4096, 4096, 4096, 4096, 1000], 8192
        Ws, bs = kaiming_uniform(dims, 5)
        g = np.random.Generator(np.random.PCG64(2))
        X = g.standard_normal((B, dims[0])).astype(np.float32)
        lab = g.integers(0, 1000, B).astype(np.uint64)
        tr = MlpTrainer(dev, dims, B, Ws, bs, "adam", lr=1e-3, clip=True, bf16=True, loss_div=65536)
        xf = dev.from_numpy(X)
        from .abi import BF16
        Xd = dev.mem_cache_alloc(BF16, X.size)
        dev.cast(xf, Xd)
        Td = dev.from_numpy(lab)
        us, n = _graph_time(dev, ts, lambda: tr.step(Xd, Td), min(reps, 20))
        flops = 293011456.0 * B  # fwd + dW + dX, algorithmic
        row = {"config": "c3 MLP 4096x3-1000 bf16/fp32-acc Adam, 8192-row shard of global 65536", "us_per_step": us,
               "samples_per_s": B / us * 1e6, "TFLOPs": flops / us * 1e-6, "kernels": n}
        row.update(leg("c3", dims=dims, Ws=Ws, bs=bs, X=X, labels=lab))
        out.append(row)
        tr.free()
        for s_ in (xf, Xd, Td):
            dev.mem_cache_free(s_)

    if "c4" in configs:
        N, F, H, C, M = 2708, 1433, 16, 7, 140
        src, tgt = synthetic.gcn_graph(N, 10556, 81761)
        A = synthetic.gcn_dense_adjacency(src, tgt, N)
        X = synthetic.gcn_features(N, F)
        (W1, W2), (b1, b2) = kaiming_uniform([F, H, C], 11)
        g = np.random.Generator(np.random.PCG64(12))
        mask = np.sort(g.permutation(N)[:M]).astype(np.int64)
        T = np.eye(C, dtype=np.float32)[g.integers(0, C, M)]
        tr = GcnTrainer(dev, A, X, W1, b1, W2, b2, mask)
        Td = dev.from_numpy(T)
        us, n = _graph_time(dev, ts, lambda: tr.step(Td), reps)
        row = {"config": "c4 GCN dense 2708 nodes, 1433-16-7, Adam", "us_per_step": us, "steps_per_s": 1e6 / us,
               "GFLOPs": 924.8e6 / us * 1e-3, "kernels": n}
        row.update(leg("c4", A=A, W1=W1, b1=b1, W2=W2, b2=b2, X=X, T=T, mask=mask))
        out.append(row)
        tr.free()
        # the reference's own algorithm for the same graph: edge scatter (here: CSR walk) instead of the dense product
        deg = synthetic.gcn_degree_scale(tgt, N)
        trs = GcnTrainer(dev, None, X, W1, b1, W2, b2, mask, edges=(src, tgt, deg))
        us, n = _graph_time(dev, ts, lambda: trs.step(Td), reps)
        row = {"config": "c4s GCN sparse propagation (edge list, CSR walk), same graph", "us_per_step": us, "steps_per_s": 1e6 / us, "kernels": n}
        row.update(leg("c4s", src=src, tgt=tgt, deg=deg, W1=W1, b1=b1, W2=W2, b2=b2, X=X, T=T, mask=mask))
        out.append(row)
        trs.free()
        dev.mem_cache_free(Td)

    if "c5" in configs:
        dims = [4, 128, 128, 2]
        Ws, bs = kaiming_uniform(dims, 21)
        batch = synthetic.dqn_batch(256, 3)
        tr = DqnTrainer(dev, dims, 256, Ws, bs)
        devb = [dev.from_numpy(x) for x in batch]
        us, n = _graph_time(dev, ts, lambda: tr.step(*devb), reps * 5 if reps >= 50 else reps)
        row = {"config": "c5 DQN 4-128-128-2 x2 nets, b256, Huber, Adam", "us_per_step": us, "kernels": n}
        row.update(leg("c5", dims=dims, Ws=Ws, bs=bs, batch=batch))
        out.append(row)
        tr.free()
        for s_ in devb:
            dev.mem_cache_free(s_)
    return out


def run_c3_dp(steps=20, warmup=5, zero=False, dev=None, ts=None, comm=None, quiet=False):
    """Config c3 data-parallel: one process per GPU (torchrun), 8192 rows per
    GPU (the global batch of 65536 at 8 GPUs; weak scaling below that), the
    gradient of each layer reduced through the library's collectives
    (zg_allreduce, or zg_reduce_scatter with `zero`) on a communication stream
    as soon as its weight-gradient GEMM has been issued, Adam after the last
    reduction.  Eager launches (17 kernels of ~0.1 ms each per step).  Returns
    the result row on rank 0 (and prints it as one JSON line unless `quiet`);
    the time is the maximum over ranks of the CUDA-event time of `steps` steps."""
    import torch
    import torch.distributed as dist
    from .abi import BF16
    from .device import CudaDevice
    from .dp import NcclComm, OverlappedGradAllReduce, ZeroShardedAdam
    from .mlp import MlpTrainer, kaiming_uniform

    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")))
    own = dev is None
    if own:
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("gloo")  # host channel for the rendezvous id, barriers and the max over ranks
        ts = torch.cuda.Stream()
        dev = CudaDevice(local, stream=ts.cuda_stream)
        comm = NcclComm.from_torch_distributed(dev) if world > 1 else None
    dims, B = [4096, 4096, 4096, 4096, 1000], 8192
    Ws, bs = kaiming_uniform(dims, 5)  # same seed on every rank: replicated parameters
    g = np.random.Generator(np.random.PCG64(100 + rank))
    X = g.standard_normal((B, dims[0])).astype(np.float32)
    lab = g.integers(0, 1000, B).astype(np.uint64)
    tr = MlpTrainer(dev, dims, B, Ws, bs, "adam", lr=1e-3, clip=True, bf16=True, loss_div=B * world)
    xf = dev.from_numpy(X)
    Xd = dev.mem_cache_alloc(BF16, X.size)
    dev.cast(xf, Xd)
    Td = dev.from_numpy(lab)
    red = OverlappedGradAllReduce(comm) if (world > 1 and not zero) else None
    zopt = ZeroShardedAdam(tr, comm) if (world > 1 and zero) else None

    def step():
        tr.forward(Xd)
        tr.loss_and_grad(Td)
        if zopt:  # reduce-scatter per layer, Adam on the owned slices, all-gather of the bf16 weights
            tr.backward(Xd, on_layer_grads=zopt.start)
            zopt.finish()
            return
        tr.backward(Xd, on_layer_grads=(lambda l: red.start(tr.layer_grads(l))) if red else None)
        if red:
            red.finish()
        tr.update()

    def barrier():
        dev.sync()
        if world > 1:
            comm.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ts)
    for _ in range(steps):
        step()
    e1.record(ts)
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    loss = tr.read_loss()
    if world > 1:  # every rank holds its share of the global-batch loss
        t = torch.tensor([loss])
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        loss = float(t.item())
    row = None
    if rank == 0:
        us = ms * 1e3 / steps
        how = ("per-layer reduce-scatter (zg_reduce_scatter) overlapped with backward, Adam sharded over the ranks, all-gather of the bf16 weights"
               if zopt else "per-layer all-reduce (zg_allreduce) overlapped with backward")
        row = {"config": "c3 data-parallel, bf16 + fp32 master, Adam, " + how,
               "n_gpus": world, "global_batch": B * world, "us_per_step": us, "samples_per_s": B * world / us * 1e6,
               "TFLOPs_per_gpu": 293011456.0 * B / us * 1e-6, "allreduce_bytes_per_step": 4 * tr.n_params,
               "loss": loss, "scaling": "weak"}
        if not quiet:
            print(json.dumps(row), flush=True)
    if zopt:
        zopt.free()
    tr.free()
    for s_ in (xf, Xd, Td):
        dev.mem_cache_free(s_)
    if own and world > 1:
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
    return row


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c3,c4,c5")
    ap.add_argument("--reps", type=int, default=200, help="graph replays per timing")
    ap.add_argument("--dp", action="store_true", help="config c3 data-parallel under torchrun (one process per GPU)")
    ap.add_argument("--zero", action="store_true", help="with --dp: shard the optimizer over the ranks (reduce-scatter / all-gather)")
    a = ap.parse_args()
    if a.dp:
        run_c3_dp(zero=a.zero)
        raise SystemExit(0)
    for r in run(a.configs.split(","), reps=a.reps):
        print(json.dumps(r), flush=True)
