#!/usr/bin/env python
"""Benchmark of the training hot path on the B200 device backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--scaling weak|strong] [--impl reference]

Workload (the reference's MNIST benchmark scaled to a GPU-sized batch): MLP
784-128-64-10, Linear+ReLU, Linear+ReLU, Linear, softmax cross-entropy, SGD
lr 0.01, fp32, batch 8192, synthetic seeded inputs (uniform [0,1) pixels,
uniform labels).  One step = forward + backward + update (+ gradient
all-reduce when N > 1).  `--scaling weak` (default) keeps 8192 rows per GPU;
`--scaling strong` shards ONE batch of 8192 over the N GPUs (8192/N rows each).
Prints ONE JSON line (rank 0).

* `value`   whole-job samples/s with the input batches already in HBM: the
            median of REPEATS timings of K steps each (`value_spread` holds
            min/max).  The resident batches rotate and together exceed L2;
            one CUDA graph holds a whole rotation (one step per batch, a
            launch per `--resident` steps; `--graph step` launches a graph
            per step instead).
* `e2e`     the same step fed from pinned HOST memory: the H2D copy of every
            batch and the D2H read of every loss are inside the timed region
            (double-buffered on a copy stream, one packed copy per batch).
* `roofline` the kernel with the largest share of the step (the split-K
            weight-gradient GEMM; its layer-1 launch), timed alone over the
            rotating batches, against the measured HBM peak; `kernels`
            holds the other two kernels of the critical path beside it.
* `cpu_baseline` the CPU oracle (reference HostDevice restated, OpenBLAS) on
            the box's host cores, on a bounded sample of the same workload.
* `dp_check` (N > 1) replicas bit-identical after the timed steps, and three
            further steps on a fixed global batch agree with the CPU oracle
            started from the same parameters.
* `strong`  (N > 1, weak run) the strong-scaling numbers of the same job.
* `configs` (N = 1) the other benchmark configurations, GPU and CPU side by
            side; at N > 1 the wide-MLP data-parallel step.

`--impl reference` times the CPU path alone (the reference itself is Zig and
cannot be built in an image without a Zig toolchain).
"""
from __future__ import annotations

import argparse
import hashlib
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
REPEATS = 5
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the committed ncu capture of the kernel
# instances the step launches (profiles/roofline_traffic.json names the capture each figure comes from)
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "roofline_traffic.json")


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
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


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
# CPU path (oracle): the reference arm, the cpu_baseline leg, the dp_check oracle
# and the host legs of the other configurations
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


def _cpu_us(fn, reps, warm=2):
    for _ in range(warm):
        fn()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    return (time.perf_counter() - t0) / reps * 1e6


def cpu_config_leg(name, **kw):
    """Host-side timing of one of the other configurations: the CPU oracle on
    the host arrays the GPU row was built from (a bounded number of steps)."""
    import oracle
    from oracle.nets import DqnOracle, GcnOracle, GcnSparseOracle
    cores = os.cpu_count() or 1
    oracle.lib()
    oracle.set_threads(cores)
    if name == "c1":
        m = oracle.MlpOracle(kw["dims"], kw["Ws"], kw["bs"], "sgd", lr=LR)
        us = _cpu_us(lambda: m.step(kw["X"], kw["T"]), 200)
        return {"cpu_us_per_step": us, "cpu_samples_per_s": kw["X"].shape[0] / us * 1e6, "cpu_cores": cores, "cpu_sample": "200 steps"}
    if name == "c3":
        # fp32 arithmetic on the same operands (the host backend has no bf16): ONE step of the 8192-row shard
        X, lab = kw["X"], kw["labels"]
        T = np.zeros((X.shape[0], kw["dims"][-1]), np.float32)
        T[np.arange(X.shape[0]), lab.astype(np.int64)] = 1.0
        m = oracle.MlpOracle(kw["dims"], kw["Ws"], kw["bs"], "adam", lr=1e-3, clip=True)
        us = _cpu_us(lambda: m.step(X, T, loss_div=65536), 1, warm=0)
        return {"cpu_us_per_step": us, "cpu_samples_per_s": X.shape[0] / us * 1e6, "cpu_cores": cores, "cpu_sample": "1 step, fp32"}
    if name == "c4":
        m = GcnOracle(kw["A"], kw["W1"], kw["b1"], kw["W2"], kw["b2"])
        return {"cpu_us_per_step": _cpu_us(lambda: m.step(kw["X"], kw["T"], kw["mask"]), 20), "cpu_cores": cores, "cpu_sample": "20 steps"}
    if name == "c4s":
        m = GcnSparseOracle(kw["src"], kw["tgt"], kw["deg"], kw["W1"], kw["b1"], kw["W2"], kw["b2"])
        return {"cpu_us_per_step": _cpu_us(lambda: m.step(kw["X"], kw["T"], kw["mask"]), 20), "cpu_cores": cores, "cpu_sample": "20 steps"}
    if name == "c5":
        m = DqnOracle(kw["dims"], kw["Ws"], kw["bs"])
        return {"cpu_us_per_step": _cpu_us(lambda: m.step(*kw["batch"]), 200), "cpu_cores": cores, "cpu_sample": "200 steps"}
    return {}


def run_reference(args, rank, world):
    if rank != 0:
        return
    B = args.batch
    steps = max(1, min(args.steps, 200))
    sps, ms, cores, blas = time_cpu_path(B, steps, max(1, min(args.warmup, 5)))
    out = {
        "impl": "reference", "metric": METRIC, "value": sps, "unit": "samples/s", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "MLP 784-128-64-10 softmax-CE SGD lr=0.01, batch %d, CPU path (HostDevice restated, %s)" % (B, blas)},
        "cpu_baseline": {"value": sps, "unit": "samples/s", "cores": cores, "kind": "port",
                         "sample": "%d full steps of batch %d on all host threads" % (steps, B)},
        "e2e": {"value": sps, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


# ----------------------------------------------------------------------------
# host topology (for the end-to-end leg: where the staging memory lives)
# ----------------------------------------------------------------------------
def gpu_numa_node(index):
    try:
        bus = subprocess.run(["nvidia-smi", "-i", str(index), "--query-gpu=pci.bus_id", "--format=csv,noheader"], capture_output=True,
                             text=True, timeout=20).stdout.strip().lower()
        if bus.startswith("0000"):
            bus = bus[4:]
        with open("/sys/bus/pci/devices/%s/numa_node" % bus) as f:
            return int(f.read().strip())
    except Exception:
        return None


def bind_to_numa_node(node):
    """Runs this process on the CPUs of `node`, so that the page-locked staging
    buffers allocated afterwards come from the memory next to the GPU."""
    try:
        if node is None or node < 0:
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


# ----------------------------------------------------------------------------
# GPU path
# ----------------------------------------------------------------------------
class Job:
    """One configuration of the data-parallel MLP step on this rank: trainer,
    reducer, resident batches, one captured graph per resident batch and one over a
    whole rotation of them."""

    def __init__(self, dev, comm, rank, world, B, global_B, resident, allreduce_kind, seed_base=1000, steps_per_graph=1):
        from zigrad_b200.dp import GradAllReduce, PeerAllReduce
        from zigrad_b200.mlp import MlpTrainer, kaiming_uniform
        self.dev, self.comm, self.rank, self.world, self.B, self.global_B = dev, comm, rank, world, B, global_B
        Ws, bs = kaiming_uniform(DIMS, SEED)
        # the update kernel also clears the gradients it applied: zero_grad costs no launch of its own
        self.tr = MlpTrainer(dev, DIMS, B, Ws, bs, "sgd", lr=LR, fused=True, loss_div=global_B, zero_grads_in_update=True)
        # N > 1: the flat gradient buffer (437 KB) is latency-bound, so it is reduced by the one-kernel
        # peer-memory all-reduce (fused with the update), inside the same captured graph as the rest of
        # the step; --allreduce nccl selects the library collective (also captured) + the update kernel
        self.peer = allreduce_kind == "peer"
        self.reducer = None
        if world > 1:
            self.reducer = PeerAllReduce(dev, self.tr.n_params, comm) if self.peer else GradAllReduce(comm=comm)
        self.host = [make_batch(B, seed_base + rank * 100 + i) for i in range(resident)]
        self.resident = [(dev.from_numpy(X), dev.from_numpy(T)) for X, T in self.host]
        self.step_eager(*self.resident[0])  # workspaces grow here, outside any capture
        dev.sync()
        self.graphs = [self.capture(lambda X=X, T=T: self.step_eager(X, T)) for X, T in self.resident]
        self.kernels_per_step = self.graphs[0].kernel_count()
        # one graph over a whole rotation of the resident batches (one step each, in order): a launch per
        # rotation instead of per step; steps that do not fill a rotation use the per-batch graphs
        self.rotation = self.capture(lambda: [self.step_eager(X, T) for X, T in self.resident]) if steps_per_graph > 1 else None
        self.cursor = 0

    def step_eager(self, X, T):
        self.tr.step(X, T, self.reducer)

    def capture(self, fn):
        self.dev.capture.open()
        fn()
        self.dev.capture.save()
        return self.dev.capture.detach()

    def step(self, i):
        self.graphs[i % len(self.graphs)].run()

    def run(self, steps):
        """`steps` steps, the resident batches in rotation: whole rotations as one graph launch each."""
        R, i = len(self.graphs), 0
        while i < steps:
            if self.rotation is not None and self.cursor % R == 0 and steps - i >= R:
                self.rotation.run()
                i += R
                self.cursor += R
            else:
                self.graphs[self.cursor % R].run()
                i += 1
                self.cursor += 1

    def close(self):
        for g in self.graphs + ([self.rotation] if self.rotation is not None else []):
            g.free()
        if self.peer and self.reducer is not None:
            self.reducer.close()
        for X, T in self.resident:
            self.dev.mem_cache_free(X)
            self.dev.mem_cache_free(T)
        self.tr.free()


def run_gpu(args, rank, local_rank, world):
    import torch
    from zigrad_b200 import opspec
    from zigrad_b200.abi import SINGLE
    from zigrad_b200.device import USIZE, CudaDevice
    from zigrad_b200.dp import NcclComm

    numa = gpu_numa_node(local_rank)
    bound_cpus = bind_to_numa_node(numa) if not args.no_numa_bind else None
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # host-side plumbing (barriers, max over ranks, the rendezvous id); the gradients travel
        # through the library's own entry points (zg_allreduce_sgd_oneshot / zg_allreduce)
        dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local_rank))
    ts = torch.cuda.Stream()           # compute stream, shared with the device object
    dev = CudaDevice(local_rank, stream=ts.cuda_stream)
    comm = NcclComm.from_torch_distributed(dev) if world > 1 else None
    strong = args.scaling == "strong"
    if strong and args.batch % world:
        raise SystemExit("--scaling strong needs a batch divisible by the number of GPUs")
    B = args.batch // world if strong else args.batch
    global_B = args.batch if strong else args.batch * world
    # resident batches: together larger than L2 whatever the per-rank batch is
    R = args.resident if not strong else args.resident * world
    job = Job(dev, comm, rank, world, B, global_B, R, args.allreduce, steps_per_graph=R if args.graph == "rotation" else 1)
    tr = job.tr

    def barrier():
        dev.sync()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(step_fn, steps, whole=False):
        """K steps between two events on the compute stream, a barrier and a
        synchronise on both sides; the maximum over the ranks, in ms.
        `whole`: step_fn takes the number of steps and runs them all."""
        barrier()
        e0.record(ts)
        if whole:
            step_fn(steps)
        else:
            for i in range(steps):
                step_fn(i)
        e1.record(ts)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # ---- value: inputs resident in HBM
    for i in range(args.warmup):
        job.step(i)
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
                job.step(j)
            dev.sync()
            return
        while len(sampler.lines) < n_samples and time.time() - t0 < limit_s:
            for _ in range(50):
                job.step(j)
                j += 1
            dev.sync()

    if rank == 0:
        sampler.start()
    load_until(2, 4.0)
    times = [timed(job.run, args.steps, whole=True) for _ in range(REPEATS)]
    load_until(len(sampler.lines) + 3, 2.0)
    clocks = sampler.stop() if rank == 0 else None
    ms = statistics.median(times)
    value = args.steps * global_B / (ms / 1e3)
    spread = {"repeats": REPEATS, "ms_per_step_min": min(times) / args.steps, "ms_per_step_max": max(times) / args.steps,
              "value_min": args.steps * global_B / (max(times) / 1e3), "value_max": args.steps * global_B / (min(times) / 1e3)}
    loss_after = sum_over_ranks(tr.read_loss())  # every rank holds its shard's share of the global-batch loss

    # ---- dp_check (N > 1): replicas identical; three more steps on a fixed global batch against the CPU oracle
    dp_check = None
    if world > 1:
        digest = hashlib.sha256(dev.to_numpy(tr.params).tobytes()).hexdigest()
        digests = [None] * world
        dist.all_gather_object(digests, digest)
        identical = all(d == digests[0] for d in digests)
        start_W, start_b = tr.get_params()
        Xc, Tc = make_batch(B, 555000 + rank)          # this rank's rows of the check batch
        dev.mem_transfer_htod(Xc.ravel(), job.resident[0][0])
        dev.mem_transfer_htod(Tc.ravel(), job.resident[0][1])
        dev.sync()
        gpu_losses = []
        for _ in range(3):
            job.graphs[0].run()
            gpu_losses.append(sum_over_ranks(tr.read_loss()))
        rows = [None] * world
        dist.gather_object((Xc, Tc), rows if rank == 0 else None, dst=0)
        loss_err = None
        if rank == 0:
            import oracle
            oracle.set_threads(os.cpu_count() or 1)
            ref = oracle.MlpOracle(DIMS, start_W, start_b, "sgd", lr=LR)
            Xg, Tg = np.concatenate([r[0] for r in rows]), np.concatenate([r[1] for r in rows])
            want = [ref.step(Xg, Tg) for _ in range(3)]
            loss_err = max(abs(a - b) / abs(b) for a, b in zip(gpu_losses, want))
        digest2 = hashlib.sha256(dev.to_numpy(tr.params).tobytes()).hexdigest()
        dist.all_gather_object(digests, digest2)
        identical = identical and all(d == digests[0] for d in digests)
        dp_check = {"replicas_identical": bool(identical), "loss_rel_err": loss_err, "loss_tolerance": 1e-4,
                    "how": "sha256 of the parameter bytes of every rank after the timed steps and after 3 further steps on a fixed "
                           "seeded global batch of %d rows; their summed shard losses against the CPU oracle started from the same parameters" % global_B}
        ok = identical and (rank != 0 or loss_err <= 1e-4)
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        if not all(flags):
            if rank == 0:
                print(json.dumps({"dp_check_failed": dp_check}), flush=True)
            raise SystemExit(3)
        # back to the benchmark batch
        dev.mem_transfer_htod(job.host[0][0].ravel(), job.resident[0][0])
        dev.mem_transfer_htod(job.host[0][1].ravel(), job.resident[0][1])
        dev.sync()

    # ---- e2e: batches come from pinned host memory through the package's input pipeline (copy stream,
    # double-buffered, ONE packed copy per batch: pixels + u64 class indices), the loss of every step goes back
    from zigrad_b200.input_pipeline import BatchStager
    st = BatchStager(dev, [(B * DIMS[0], SINGLE), (B, USIZE)], depth=2, packed=True)
    pin = [st.pack([X, np.argmax(T, 1).astype(np.uint64)]) for X, T in job.host]
    n_e2e = args.warmup + args.steps
    loss_host = st.pinned((n_e2e,), np.float32)
    for X, L_ in st.slots:  # defined contents before the graphs are captured
        dev.mem_fill(X, 0.5)
        dev.mem_transfer_htod(np.zeros(B, np.uint64), L_)
    dev.sync()
    slot_graphs = [job.capture(lambda X=X, L_=L_: job.step_eager(X, L_)) for X, L_ in st.slots]
    h2d = st.bytes_per_batch()

    def e2e_step(i):
        if i + 1 < n_e2e:
            st.put(pin[(i + 1) % R])          # the copy of the next batch overlaps this step
        s = st.current_slot()
        st.get()                              # the compute stream waits for THIS batch's copy only
        slot_graphs[s].run()
        dev.L.memcpy_DtoH(loss_host.ctypes.data + 4 * i, tr.loss.ptr, 4, dev.stream)
        st.release()

    st.put(pin[0])
    for i in range(args.warmup):
        e2e_step(i)
    ms_e2e = timed(lambda i: e2e_step(args.warmup + i), args.steps)
    e2e_value = args.steps * global_B / (ms_e2e / 1e3)
    e2e_last_loss = sum_over_ranks(float(loss_host[n_e2e - 1]))
    # the copy leg alone, per rank (all ranks copying at once): what the host side can feed
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cs = torch.cuda.ExternalStream(st.copy_stream.ptr)
    c0.record(cs)
    for i in range(10):
        dev.L.memcpy_HtoD(st._blocks[i % 2].ptr, pin[i % R].ctypes.data, h2d, st.copy_stream)
    c1.record(cs)
    dev.L.stream_synchronize(st.copy_stream)
    h2d_gbs = 10 * h2d / (c0.elapsed_time(c1) * 1e-3) / 1e9
    h2d_all = [None] * world
    if world > 1:
        dist.all_gather_object(h2d_all, (round(h2d_gbs, 1), numa))
    else:
        h2d_all = [(round(h2d_gbs, 1), numa)]
    for g in slot_graphs:
        g.free()
    st.close()

    # ---- roofline of the kernel with the largest share of the step, timed alone over the rotating batches
    roofline, kernel_table = None, None
    if rank == 0:
        hbm, tflops, _, origin = measured_peaks()
        K0, N0 = DIMS[0], DIMS[1]
        cands = {
            "layer-1 forward GEMM+bias+ReLU [B,784]x[128,784]^T": (
                lambda X: dev.dispatch(opspec.linear(X, tr.W[0], tr.act[0], B, N0, K0, False, True, K0, K0, N0, 1.0, 0.0, "bias_relu", tr.b[0])),
                4.0 * (B * K0 + N0 * K0 + B * N0 + N0), 2.0 * B * K0 * N0),
            "layer-1 weight-gradient GEMM dY^T.X [128,B]x[B,784]": (
                # the launch the training step makes: accumulating (beta = 1) with alpha = -lr, its split-K grid sized
                # for the SM share it has beside the other weight gradients (into the gradient buffer here, so that
                # timing it does not move the weights)
                lambda X: dev.dispatch(opspec.linear(tr.dact[0], X, tr.dW[0], N0, K0, B, True, False, N0, K0, K0, -LR, 1.0,
                                                     sm_budget=(tr._dw_sm_shares().get(0, 0) if tr.tail and tr.L == 3 else 0))),
                4.0 * (B * N0 + B * K0 + N0 * K0), 2.0 * B * K0 * N0),
        }
        if tr.tail:
            H1, H2, CC, LD = DIMS[1], DIMS[2], DIMS[3], tr.ld_out
            cands["fused tail: layer-2 fwd, layer-3 fwd, softmax-CE, dX3, dX2, bias gradients (not a roofline candidate: a dependent chain)"] = (
                lambda X: dev.dispatch(opspec.mlp_tail(tr.act[0], tr.W[1], tr.b[1], tr.W[2], tr.b[2], job.resident[0][1], B, H1, H2, CC, LD,
                                                       float(global_B), tr.act[1], tr.act[2], tr.loss, tr.dact[2], tr.dact[1], tr.dact[0],
                                                       tr.db[2], tr.db[1], tr.db[0], weights_ready=True)),
                4.0 * (2 * B * H1 + 2 * B * H2 + 2 * B * LD + B * CC + H2 * H1 + CC * H2), 2.0 * B * (2 * H1 * H2 + 2 * H2 * CC))
        traffic = {}
        if os.path.exists(TRAFFIC_FILE):
            traffic = json.load(open(TRAFFIC_FILE))
        kernel_table = {}
        for name, (fn, nbytes, flops) in cands.items():
            fn(job.resident[0][0])
            dev.sync()
            g = job.capture(lambda: [fn(X) for X, _ in job.resident])
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
            us = e0.elapsed_time(e1) * 1e3 / (reps * len(job.resident))   # per op
            kernel_table[name] = {"us_per_op": us, "launches_per_op": launches_per_run / len(job.resident), "GBps": nbytes / us * 1e-3,
                                  "TFLOPs": flops / us * 1e-6, "bytes": nbytes, "flops": flops}
            g.free()
        # the roofline kernel is the instance with the largest share of the step in the committed launch list
        # (profiles/bench_mlp_784-128-64-10_b8192_launch_list.md): the split-K weight-gradient GEMM; the
        # launch reported is its large one, dW0
        top = "layer-1 weight-gradient GEMM dY^T.X [128,B]x[B,784]"
        kt = kernel_table[top]
        tr_entry = traffic.get(top, {}) if B == 8192 else {}
        roofline = {"kernel": top, "bound": "hbm", "achieved": kt["GBps"], "peak": hbm, "unit": "GB/s", "frac": kt["GBps"] / hbm,
                    "traffic": tr_entry.get("dram_bytes_per_launch"), "traffic_source": tr_entry.get("source", "no capture for this batch size"),
                    "peak_origin": "of " + origin, "us_per_launch": kt["us_per_op"],
                    "algorithmic_bytes": kt["bytes"], "tensor_TFLOPs_algorithmic": kt["TFLOPs"],
                    "limiter": "shared-memory pipe: per 32-deep k-slab of a 128x128 tile 3xTF32 moves ~128 KB through it (TMA write, hi/lo "
                               "split, tensor-core reads of B: ~1000 cycles at 128 B/cycle) for 768 cycles of tensor work; DRAM traffic equals "
                               "the algorithmic bytes (profiles/gemm_tc_fp32x3_mlp_step_gemms_b8192.md)"}

    # ---- CPU baseline (bounded sample), rank 0 at N=1 only
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sps, cms, cores, blas = time_cpu_path(args.batch, 20, 3)
        cpu = {"value": sps, "unit": "samples/s", "cores": cores, "kind": "port",
               "sample": "20 steps of batch %d (of the same workload) on %d host threads, %s; %.1f ms/step" % (args.batch, cores, blas, cms)}

    kernels_per_step = job.kernels_per_step
    job.close()

    # ---- the other curve of the same job (N > 1, weak run): one batch of 8192 sharded over the ranks
    strong_row = None
    if world > 1 and not strong and args.batch % world == 0 and not args.no_strong:
        sj = Job(dev, comm, rank, world, args.batch // world, args.batch, args.resident * world, args.allreduce, seed_base=7000,
                 steps_per_graph=args.resident * world if args.graph == "rotation" else 1)
        for i in range(args.warmup):
            sj.step(i)
        stimes = [timed(sj.run, args.steps, whole=True) for _ in range(REPEATS)]
        sms = statistics.median(stimes)
        strong_row = {"scaling": "strong", "global_batch": args.batch, "per_gpu_batch": args.batch // world,
                      "value": args.steps * args.batch / (sms / 1e3), "unit": "samples/s", "ms_per_step": sms / args.steps,
                      "ms_per_step_min": min(stimes) / args.steps, "ms_per_step_max": max(stimes) / args.steps,
                      "kernels_per_step": int(sj.kernels_per_step), "final_loss": sum_over_ranks(sj.tr.read_loss())}
        sj.close()

    # ---- the other configurations BASELINE.json names (bounded: a few seconds each)
    configs = None
    if not args.no_configs:
        from zigrad_b200 import configs_bench
        if world == 1:
            rows = configs_bench.run(["c1", "c3", "c4", "c5"], reps=100, dev=dev, ts=ts, host_leg=None if args.no_cpu else cpu_config_leg)
            _, burst, sustained, origin = measured_peaks()
            configs = {}
            for r in rows:
                key = r["config"].split()[0]
                if key == "c3":
                    r["frac_of_bf16_peak_burst"] = r["TFLOPs"] / burst
                    r["frac_of_bf16_peak_sustained"] = r["TFLOPs"] / sustained
                    r["peak_origin"] = "of " + origin
                configs[{"c3": "c3_shard", "c4": "c4_dense", "c4s": "c4_sparse"}.get(key, key)] = r
        elif world >= 2 and not args.no_c3_dp:
            configs = {}
            for key, zero in (("c3_dp_allreduce", False), ("c3_dp_sharded_adam", True)):
                row = configs_bench.run_c3_dp(steps=10, warmup=3, zero=zero, dev=dev, ts=ts, comm=comm, quiet=True)
                if rank == 0:
                    configs[key] = row

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "value_spread": spread,
            "config": {"workload": "MLP 784-128-64-10 (Linear+ReLU, Linear+ReLU, Linear) softmax-CE SGD lr=0.01, fp32 (3xTF32 tensor-core GEMMs), "
                                   + ("one batch of %d sharded over the GPUs" % global_B if strong else "batch %d per GPU" % B),
                       "global_batch": global_B, "per_gpu_batch": B, "parallelism": "dp%d" % world,
                       "l2_policy": "%d resident batches of %.1f MB rotate (%.0f MB > 126 MB L2)" % (R, B * (DIMS[0] + DIMS[-1]) * 4 / 1e6, R * B * (DIMS[0] + DIMS[-1]) * 4 / 1e6),
                       "step_launch": ("one CUDA graph per rotation of the resident batches (%d steps per launch)" % R if job.rotation is not None
                                       else "CUDA graph per resident batch") + ("" if world == 1 else (
                           " incl. the one-kernel peer-memory (NVLink) all-reduce of the flat gradient buffer fused with the update" if job.peer else
                           " incl. the library all-reduce (zg_allreduce) of the flat gradient buffer and the update kernel"))},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e / args.steps, "last_loss_read_on_host": e2e_last_loss,
                    "h2d_GBps_per_rank_all_ranks_copying": [x[0] for x in h2d_all], "gpu_numa_node_per_rank": [x[1] for x in h2d_all],
                    "staging_bound_to_gpu_numa_cpus": bound_cpus,
                    "api": "zigrad_b200.input_pipeline.BatchStager (packed: pixels + u64 labels in one copy) + MlpTrainer.step (captured graph per staging slot)"},
            "gpu_launches": int(kernels_per_step * args.steps),
            "kernels_per_step": int(kernels_per_step),
            "final_loss": loss_after,
            "roofline": roofline, "kernels": kernel_table, "cpu_baseline": cpu,
            "dp_check": dp_check, "strong": strong_row, "configs": configs,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        comm.close()
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8192, help="rows per GPU (weak) or of the one global batch (strong)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--graph", choices=["rotation", "step"], default="rotation",
                    help="device-timed leg: one CUDA graph per rotation of the resident batches (a launch per --resident steps) or one per step")
    ap.add_argument("--resident", type=int, default=8, help="distinct batches kept in HBM and rotated")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU legs")
    ap.add_argument("--no-configs", action="store_true", help="skip the other configurations")
    ap.add_argument("--no-c3-dp", action="store_true", help="N > 1: skip the wide-MLP data-parallel step")
    ap.add_argument("--no-strong", action="store_true", help="N > 1, weak run: skip the strong-scaling numbers")
    ap.add_argument("--no-numa-bind", action="store_true", help="do not bind the process to the CPUs next to its GPU")
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
