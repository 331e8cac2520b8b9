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

    def reduce_and_sgd(self, grads, params, lr: float) -> None:
        """All-reduce fused with the plain SGD update (no clipping): one kernel."""
        self.dev.L.zg_allreduce_sgd_oneshot(self.dev.stream, grads.ptr, params.ptr, grads.len, float(lr), self.rank, self.world,
                                            self.ptrs, self.cap)

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
