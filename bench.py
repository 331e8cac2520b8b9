#!/usr/bin/env python
"""Benchmark of the training hot path on the B200 device backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (the reference's MNIST benchmark scaled to a GPU-sized batch): MLP
784-128-64-10, Linear+ReLU, Linear+ReLU, Linear, softmax cross-entropy, SGD
lr 0.01, fp32, batch 8192 per GPU, synthetic seeded inputs (uniform [0,1)
pixels, uniform labels).  One step = forward + backward + update (+ gradient
all-reduce when N > 1).  Prints ONE JSON line (rank 0).

* `value`   whole-job samples/s with the input batches already in HBM.  The
            step is captured once per resident batch into a CUDA graph; the
            resident batches rotate and together exceed the L2 cache.
* `e2e`     the same step fed from pinned HOST memory: the H2D copy of every
            batch and the D2H read of every loss are inside the timed region
            (double-buffered on a copy stream).
* `roofline` the slowest kernel of the step, timed alone over the rotating
            batches, against the measured HBM / tensor peaks.
* `cpu_baseline` the CPU oracle (reference HostDevice restated, OpenBLAS) on
            the box's host cores, on a bounded sample of the same workload.

`--impl reference` times that CPU path alone (the reference itself is Zig and
cannot be built in an image without a Zig toolchain).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DIMS = [784, 128, 64, 10]
LR = 0.01
SEED = 81761  # the reference's global seed (src/zigrad.zig:66)
METRIC = "train samples/sec (fwd+bwd+SGD)"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu capture of the
# same full-size launches (the eight GEMMs of one eager step, ncu --set full); batch 8192 only
NCU_DRAM_TRAFFIC = {"layer-1 forward GEMM+bias+ReLU [B,784]x[128,784]^T": 26165504,
                    "layer-1 weight-gradient GEMM dY^T.X [128,B]x[B,784]": 30362624}


def make_batch(B, seed):
    g = np.random.Generator(np.random.PCG64(seed))
    X = g.uniform(0.0, 1.0, (B, DIMS[0])).astype(np.float32)
    lab = g.integers(0, DIMS[-1], B)
    T = np.zeros((B, DIMS[-1]), np.float32)
    T[np.arange(B), lab] = 1.0
    return X, T


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------
# CPU path (oracle): the reference arm and the cpu_baseline leg
# ----------------------------------------------------------------------------
def time_cpu_path(B, steps, warmup):
    import oracle
    from zigrad_b200.mlp import kaiming_uniform
    cores = os.cpu_count() or 1
    oracle.lib()
    oracle.set_threads(cores)
    Ws, bs = kaiming_uniform(DIMS, SEED)
    model = oracle.MlpOracle(DIMS, Ws, bs, "sgd", lr=LR)
    data = [make_batch(B, 1000 + i) for i in range(2)]
    for i in range(warmup):
        model.step(*data[i % 2])
    t0 = time.perf_counter()
    for i in range(steps):
        model.step(*data[i % 2])
    dt = time.perf_counter() - t0
    return steps * B / dt, dt / steps * 1e3, cores, oracle.blas_name


def run_reference(args, rank, world):
    if rank != 0:
        return
    B = args.batch
    steps = max(1, min(args.steps, 200))
    sps, ms, cores, blas = time_cpu_path(B, steps, max(1, min(args.warmup, 5)))
    out = {
        "impl": "reference", "metric": METRIC, "value": sps, "unit": "samples/s", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "MLP 784-128-64-10 softmax-CE SGD lr=0.01, batch %d, CPU path (HostDevice restated, %s)" % (B, blas)},
        "cpu_baseline": {"value": sps, "unit": "samples/s", "cores": cores, "kind": "port",
                         "sample": "%d full steps of batch %d on all host threads" % (steps, B)},
        "e2e": {"value": sps, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


# ----------------------------------------------------------------------------
# GPU path
# ----------------------------------------------------------------------------
def run_gpu(args, rank, local_rank, world):
    import torch
    from zigrad_b200 import opspec
    from zigrad_b200.abi import SINGLE
    from zigrad_b200.device import CudaDevice
    from zigrad_b200.dp import GradAllReduce, PeerAllReduce
    from zigrad_b200.mlp import MlpTrainer, kaiming_uniform

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ts = torch.cuda.Stream()           # compute stream, shared with the device object
    dev = CudaDevice(local_rank, stream=ts.cuda_stream)
    B = args.batch
    global_B = B * world               # weak scaling: per-GPU batch fixed
    R = args.resident
    Ws, bs = kaiming_uniform(DIMS, SEED)
    # the update kernel also clears the gradients it applied: zero_grad costs no launch of its own
    tr = MlpTrainer(dev, DIMS, B, Ws, bs, "sgd", lr=LR, fused=True, loss_div=global_B, zero_grads_in_update=True)
    # N > 1: the flat gradient buffer (437 KB) is latency-bound, so it is reduced by the
    # one-kernel peer-memory all-reduce, inside the same captured graph as the rest of the
    # step; --allreduce nccl selects the library collective between two graphs instead
    peer = args.allreduce == "peer"
    reducer = None
    if world > 1:
        reducer = PeerAllReduce(dev, tr.n_params) if peer else GradAllReduce()
    host = [make_batch(B, 1000 + rank * 100 + i) for i in range(R)]
    resident = [(dev.from_numpy(X), dev.from_numpy(T)) for X, T in host]

    def allreduce(grads):
        if peer:
            reducer(grads)
        else:
            reducer.device(grads, ts)

    if peer and world > 1:
        allreduce = reducer  # MlpTrainer.step then fuses the reduction with the SGD update (one kernel)

    one_graph = world == 1 or peer

    # ---- capture: one graph per resident batch (N=1: the whole step; N>1: the
    # all-reduce runs between a forward+backward graph and an update graph)
    tr.step(resident[0][0], resident[0][1], allreduce if world > 1 else None)  # eager warm-up: workspaces grow here
    dev.sync()
    graphs, update_graph = [], None

    def capture(fn):
        dev.capture.open()
        fn()
        dev.capture.save()
        return dev.capture.detach()

    for X, T in resident:
        if one_graph:
            graphs.append(capture(lambda: tr.step(X, T, allreduce if world > 1 else None)))
        else:
            graphs.append(capture(lambda: (tr.forward(X), tr.loss_and_grad(T), tr.backward(X))))
    if not one_graph:
        update_graph = capture(tr.update)
    kernels_per_step = graphs[0].kernel_count() + (update_graph.kernel_count() if update_graph else 0)

    def step(i):
        graphs[i % R].run()
        if not one_graph:
            allreduce(tr.grads)
            update_graph.run()

    def barrier():
        dev.sync()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- value: inputs resident in HBM
    for i in range(args.warmup):
        step(i)
    barrier()
    # The timed region lasts milliseconds, nvidia-smi samples every 100 ms: keep the
    # GPU under the SAME load (untimed steps) until the sampler has delivered a
    # sample, time the K steps, then keep the load on until a few more arrive.
    sampler = ClockSampler(local_rank)

    def load_until(n_samples, limit_s):
        t0 = time.time()
        j = 0
        if world > 1:  # ranks must stay in lockstep: a fixed number of steps instead of a condition only rank 0 sees
            for j in range(1500):
                step(j)
            dev.sync()
            return
        while len(sampler.lines) < n_samples and time.time() - t0 < limit_s:
            for _ in range(50):
                step(j)
                j += 1
            dev.sync()

    if rank == 0:
        sampler.start()
    load_until(2, 4.0)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ts)
    for i in range(args.steps):
        step(i)
    e1.record(ts)
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    load_until(len(sampler.lines) + 3, 2.0)
    clocks = sampler.stop() if rank == 0 else None
    value = args.steps * global_B / (ms / 1e3)
    loss_after = tr.read_loss()

    # ---- e2e: batches come from pinned host memory through the package's input pipeline
    # (copy stream, double-buffered), the loss of every step goes back to the host
    from zigrad_b200.input_pipeline import BatchStager
    st = BatchStager(dev, [(B * DIMS[0], SINGLE), (B * DIMS[-1], SINGLE)], depth=2)
    pin = [(st.pinned_like(X), st.pinned_like(T)) for X, T in host]
    loss_host = st.pinned((args.steps + args.warmup,), np.float32)
    for X, T in st.slots:  # defined contents before the graphs are captured
        dev.mem_fill(X, 0.5)
        dev.mem_fill(T, 0.1)
    slot_graphs = []
    for X, T in st.slots:
        if one_graph:
            slot_graphs.append(capture(lambda: tr.step(X, T, allreduce if world > 1 else None)))
        else:
            slot_graphs.append(capture(lambda: (tr.forward(X), tr.loss_and_grad(T), tr.backward(X))))
    h2d = st.bytes_per_batch()
    n_e2e = args.warmup + args.steps

    def e2e_step(i):
        if i + 1 < n_e2e:
            st.put(pin[(i + 1) % R])          # the copy of the next batch overlaps this step
        s = st.current_slot()
        st.get()                              # compute stream waits for this batch's copy
        slot_graphs[s].run()
        if not one_graph:
            allreduce(tr.grads)
            update_graph.run()
        dev.L.memcpy_DtoH(loss_host.ctypes.data + 4 * i, tr.loss.ptr, 4, dev.stream)
        st.release()

    st.put(pin[0])
    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    e0.record(ts)
    for i in range(args.warmup, n_e2e):
        e2e_step(i)
    e1.record(ts)
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    e2e_value = args.steps * global_B / (ms_e2e / 1e3)
    e2e_last_loss = float(loss_host[n_e2e - 1])
    st.close()

    # ---- roofline of the slowest kernel, timed alone over the rotating batches
    roofline, kernel_table = None, None
    if rank == 0:
        hbm, tflops, origin = measured_peaks()
        K0, N0 = DIMS[0], DIMS[1]
        cands = {
            "layer-1 forward GEMM+bias+ReLU [B,784]x[128,784]^T": (
                lambda X: dev.dispatch(opspec.linear(X, tr.W[0], tr.act[0], B, N0, K0, False, True, K0, K0, N0, 1.0, 0.0, "bias_relu", tr.b[0])),
                4.0 * (B * K0 + N0 * K0 + B * N0 + N0), 2.0 * B * K0 * N0),
            "layer-1 weight-gradient GEMM dY^T.X [128,B]x[B,784]": (
                # beta = 1: accumulating into the gradient buffer, the launch the training step makes
                lambda X: dev.dispatch(opspec.linear(tr.dact[0], X, tr.dW[0], N0, K0, B, True, False, N0, K0, K0, 1.0, 1.0)),
                4.0 * (B * N0 + B * K0 + N0 * K0), 2.0 * B * K0 * N0),
        }
        kernel_table = {}
        for name, (fn, nbytes, flops) in cands.items():
            fn(resident[0][0])
            dev.sync()
            g = capture(lambda: [fn(X) for X, _ in resident])
            launches_per_run = g.kernel_count()
            for _ in range(3):
                g.run()
            dev.sync()
            reps = 20
            e0.record(ts)
            for _ in range(reps):
                g.run()
            e1.record(ts)
            dev.sync()
            us = e0.elapsed_time(e1) * 1e3 / (reps * R)   # per op
            kernel_table[name] = {"us_per_op": us, "launches_per_op": launches_per_run / R, "GBps": nbytes / us * 1e-3,
                                  "TFLOPs": flops / us * 1e-6, "bytes": nbytes, "flops": flops}
            g.free()
        top = max(kernel_table, key=lambda k: kernel_table[k]["us_per_op"])
        kt = kernel_table[top]
        roofline = {"kernel": top, "bound": "hbm", "achieved": kt["GBps"], "peak": hbm, "unit": "GB/s", "frac": kt["GBps"] / hbm,
                    "traffic": NCU_DRAM_TRAFFIC.get(top) if B == 8192 else None, "peak_origin": "of " + origin, "us_per_launch": kt["us_per_op"],
                    "algorithmic_bytes": kt["bytes"], "tensor_TFLOPs_algorithmic": kt["TFLOPs"]}

    # ---- CPU baseline (bounded sample), rank 0 at N=1 only
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sps, cms, cores, blas = time_cpu_path(B, 20, 3)
        cpu = {"value": sps, "unit": "samples/s", "cores": cores, "kind": "port",
               "sample": "20 steps of batch %d (of the same workload) on %d host threads, %s; %.1f ms/step" % (B, cores, blas, cms)}

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "MLP 784-128-64-10 (Linear+ReLU, Linear+ReLU, Linear) softmax-CE SGD lr=0.01, fp32 (3xTF32 tensor-core GEMMs), batch %d per GPU" % B,
                       "global_batch": global_B, "per_gpu_batch": B, "parallelism": "dp%d" % world,
                       "l2_policy": "%d resident batches of %.1f MB rotate (%.0f MB > 126 MB L2)" % (R, h2d / 1e6, R * h2d / 1e6),
                       "step_launch": "CUDA graph per resident batch" + ("" if world == 1 else (
                           " incl. the one-kernel peer-memory (NVLink) all-reduce of the flat gradient buffer" if peer else
                           " + NCCL all-reduce of the flat gradient buffer + update graph"))},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e / args.steps, "last_loss_read_on_host": e2e_last_loss,
                    "api": "zigrad_b200.input_pipeline.BatchStager + MlpTrainer.step (captured graph per staging slot)"},
            "gpu_launches": int(kernels_per_step * args.steps),
            "kernels_per_step": int(kernels_per_step),
            "final_loss": loss_after,
            "roofline": roofline, "kernels": kernel_table, "cpu_baseline": cpu,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        if peer:
            err = reducer.error()
            reducer.close()
            if err:
                raise RuntimeError("the peer all-reduce gave up waiting for another rank")
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8192, help="rows per GPU")
    ap.add_argument("--resident", type=int, default=8, help="distinct batches kept in HBM and rotated")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"], help="N > 1: gradient all-reduce implementation")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    run_gpu(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
