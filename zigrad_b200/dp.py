"""Data-parallel training step: one process per GPU, the batch sharded by
contiguous row blocks, ONE all-reduce of the flat gradient buffer between
backward and the optimizer kernel.

The reference has no distributed code (its roadmap lists "Distributed comms"
as future work, ``docs/roadmap.norg:74-76``); this module is new.  Plumbing is
``torch.distributed``: NCCL over NVLink on GPUs, gloo for the CPU tests of the
host logic.  Parameters and optimizer state are replicated; every rank divides
its loss and logits gradient by the GLOBAL batch so that the summed gradients
equal the single-device gradients, and clipping/updates run after the
all-reduce, exactly as on one device.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np


def shard_rows(global_batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous row block [start, stop) of `rank`; the first
    (global_batch % world) ranks take one extra row."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class _CudaView:
    """Exposes raw device memory to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, n: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3}


class GradAllReduce:
    """Sum-all-reduce of a gradient buffer over a torch.distributed group."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self._views = {}

    def host(self, grads: np.ndarray) -> np.ndarray:
        """In-place sum over ranks of a host array (gloo path)."""
        import torch
        t = torch.from_numpy(grads)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)
        return grads

    def device(self, grads, torch_stream) -> None:
        """In-place sum over ranks of a DeviceSlice, enqueued on `torch_stream`
        (the stream the CudaDevice was created on), so it is ordered after
        the backward kernels and before the optimizer kernel."""
        import torch
        key = (grads.ptr, grads.len)
        t = self._views.get(key)
        if t is None:
            t = torch.as_tensor(_CudaView(grads.ptr, grads.len, "<f4"), device=torch_stream.device)
            self._views[key] = t
        with torch.cuda.stream(torch_stream):
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)


class OverlappedGradAllReduce:
    """Per-layer all-reduce that overlaps the backward pass.

    `start(slice, stream)` enqueues an asynchronous sum-all-reduce of one slice
    of the gradient buffer, ordered after the work already on `stream` (the
    device's side stream, where the layer's weight gradient was just issued);
    the collective runs on the communication library's own stream, so neither
    the side stream nor the main stream waits for it.  `finish(main_stream)`
    makes the main stream wait for every started reduction -- call it before
    the optimizer kernel."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self._views, self._pending = {}, []

    def start(self, grads, torch_stream) -> None:
        import torch
        key = (grads.ptr, grads.len)
        t = self._views.get(key)
        if t is None:
            t = torch.as_tensor(_CudaView(grads.ptr, grads.len, "<f4"), device=torch_stream.device)
            self._views[key] = t
        with torch.cuda.stream(torch_stream):
            self._pending.append(self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self, torch_stream) -> None:
        import torch
        with torch.cuda.stream(torch_stream):
            for w in self._pending:
                w.wait()
        self._pending = []


class PeerAllReduce:
    """Sum all-reduce of a small gradient buffer in one kernel per rank over
    peer memory (zg_allreduce_oneshot): for latency-bound buffers (up to a few
    MB) on the GPUs of one box.  A plain kernel launch on the device stream, so
    the whole data-parallel step -- backward, reduction, update -- can be
    captured into one CUDA graph.  The host-side exchange of the IPC handles
    goes through torch.distributed (any backend)."""

    def __init__(self, dev, n_elems: int, group=None):
        import ctypes as C
        import torch.distributed as dist
        self.dev, self.dist, self.group = dev, dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("PeerAllReduce supports up to 8 ranks")
        self.cap = (int(n_elems) + 3) // 4 * 4
        L = dev.L
        dev.make_current()
        self.region = L.zg_comm_alloc(self.cap, self.world)
        if not self.region:
            raise MemoryError("comm region")
        handle = (C.c_ubyte * 64)()
        L.zg_ipc_export(self.region, handle)
        from . import abi
        abi.check()
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._opened = []
        ptrs = (C.c_void_p * self.world)()
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs[r] = self.region
            else:
                buf = (C.c_ubyte * 64).from_buffer_copy(h)
                p = L.zg_ipc_open(buf)
                abi.check()
                self._opened.append(p)
                ptrs[r] = p
        self.ptrs = ptrs
        dist.barrier(group=group)  # every region is cleared and mapped before the first launch

    def __call__(self, grads) -> None:
        self.dev.L.zg_allreduce_oneshot(self.dev.stream, grads.ptr, grads.len, self.rank, self.world, self.ptrs, self.cap)

    def reduce_and_sgd(self, grads, params, lr: float, zero_grads: bool = False) -> None:
        """All-reduce fused with the plain SGD update (no clipping): one kernel.
        zero_grads leaves zeros instead of the summed gradient behind (the
        next step's zero_grad without a launch of its own)."""
        self.dev.L.zg_allreduce_sgd_oneshot(self.dev.stream, grads.ptr, params.ptr, grads.len, float(lr), self.rank, self.world,
                                            self.ptrs, self.cap, int(zero_grads))

    def error(self) -> int:
        return int(self.dev.L.zg_comm_error(self.region, self.dev.stream))

    def close(self) -> None:
        self.dev.sync()
        self.dist.barrier(group=self.group)  # nobody still reads a region that is about to go away
        for p in self._opened:
            self.dev.L.zg_ipc_close(p)
        self._opened = []
        if self.region:
            self.dev.L.zg_comm_free(self.region)
            self.region = None


class ZeroShardedAdam:
    """Data-parallel Adam with the optimizer sharded over the ranks (reduce-scatter
    of the gradients, Adam on the owned slices, all-gather of the bf16 weights).

    For the wide mixed-precision MLP the all-reduce + replicated Adam of the plain
    data-parallel step moves 2 x 218 MB over the links and spends 0.29 ms per step
    in an optimizer kernel that every rank repeats.  Here, per layer l:
      * `start(l)` (called on the side stream right after dW_l was issued) starts an
        asynchronous REDUCE-SCATTER of the layer's slice [dW_l ; db_l] of the flat
        gradient buffer: rank r receives the r-th 1/world part, in place;
      * `finish()` waits for the reductions, forms the per-tensor gradient norms
        (sum of squares of the owned parts, summed over the ranks, root) as the
        reference clips per tensor (src/device/host_device.zig:339-346), runs Adam
        (src/nn/optim.zig:177-234) over the owned parts only -- every tensor stays
        in the segment list, possibly empty, so the per-tensor step counter runs
        as on one device -- and ALL-GATHERS the updated bf16 weights in place.
    fp32 master weights and moments exist only for the owned parts (the rest of
    those buffers is unused); forward and backward read the bf16 copy.
    Layer slices must divide by the world size (true for 4096-wide layers at 8)."""

    def __init__(self, trainer, main_stream, side_stream, group=None):
        import torch
        import torch.distributed as dist
        if not trainer.bf16 or trainer.opt != "adam":
            raise ValueError("ZeroShardedAdam drives an MlpTrainer in bf16 mode with Adam")
        self.tr, self.dist, self.group, self.torch = trainer, dist, group, torch
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.main, self.side = main_stream, side_stream
        tr, W = trainer, self.world
        dev = torch.device("cuda", torch.cuda.current_device())
        self.g32 = torch.as_tensor(_CudaView(tr.grads.ptr, tr.grads.len, "<f4"), device=dev)
        self.w16 = torch.as_tensor(_CudaView(tr.params_bf16.ptr, tr.params_bf16.len, "<i2"), device=dev).view(torch.bfloat16)
        self.layers, self.owned = [], []
        for l in range(tr.L):
            (woff, wn), (boff, bn) = tr.segments[2 * l], tr.segments[2 * l + 1]
            n = wn + bn
            if n % W:
                raise ValueError("layer %d has %d parameters: not divisible by %d ranks" % (l, n, W))
            c = n // W
            lo, hi = woff + self.rank * c, woff + (self.rank + 1) * c
            self.layers.append((woff, n, c))
            # owned part of the weight tensor, owned part of the bias tensor (either may be empty)
            self.owned.append((lo, max(0, min(hi, woff + wn) - lo)))
            b0 = max(lo, boff)
            self.owned.append((b0, max(0, hi - b0)))
        self.sumsq = tr.dev.mem_cache_alloc(0, len(self.owned))
        self.sumsq_t = torch.as_tensor(_CudaView(self.sumsq.ptr, self.sumsq.len, "<f4"), device=dev)
        self._pending = []

    def start(self, l: int) -> None:
        off, n, c = self.layers[l]
        full = self.g32[off:off + n]
        mine = self.g32[off + self.rank * c: off + (self.rank + 1) * c]
        with self.torch.cuda.stream(self.side):
            self._pending.append(self.dist.reduce_scatter_tensor(mine, full, op=self.dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self) -> None:
        from . import opspec
        tr, d = self.tr, self.tr.dev
        with self.torch.cuda.stream(self.main):
            for w in self._pending:
                w.wait()
        self._pending = []
        clip = tr.clip
        if clip:
            d.segment_sumsq(tr.grads, self.owned, self.sumsq)
            with self.torch.cuda.stream(self.main):
                self.dist.all_reduce(self.sumsq_t, op=self.dist.ReduceOp.SUM, group=self.group)
            d.dispatch(opspec.sqrt_fwd(self.sumsq, self.sumsq))
        d.dispatch(opspec.adam(tr.params, tr.grads, tr.m, tr.v, self.owned, tr.t + 1, tr.lr, tr.beta1, tr.beta2, tr.eps,
                               "given" if clip else False, tr.max_norm, tr.delta, self.sumsq, tr.params_bf16, tr.t_dev))
        tr.t += len(self.owned)
        works = []
        with self.torch.cuda.stream(self.main):
            for off, n, c in self.layers:
                works.append(self.dist.all_gather_into_tensor(self.w16[off:off + n], self.w16[off + self.rank * c: off + (self.rank + 1) * c],
                                                              group=self.group, async_op=True))
            for w in works:
                w.wait()

    def free(self) -> None:
        self.tr.dev.mem_cache_free(self.sumsq)
