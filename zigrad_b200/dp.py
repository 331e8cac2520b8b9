"""Data-parallel training step: one process per GPU, the batch sharded by
contiguous row blocks, ONE all-reduce of the flat gradient buffer between
backward and the optimizer kernel.

The reference has no distributed code (its roadmap lists "Distributed comms"
as future work, ``docs/roadmap.norg:74-76``); this module is new.  On GPUs the
data plane is the library's own C ABI -- ``zg_allreduce`` / ``zg_reduce_scatter``
/ ``zg_all_gather`` (NCCL over NVLink, bound by the library at run time) and the
peer-memory kernel ``zg_allreduce_oneshot`` -- so a host in any language drives
the same calls; ``torch.distributed`` is used only as the HOST channel that
carries the 128-byte rendezvous id (and, with gloo, for the CPU tests of the
host logic).  Parameters and optimizer state are replicated; every rank divides
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


class NcclComm:
    """One communicator per process (= per GPU) through the C ABI.

    `exchange(id_bytes_or_None) -> id_bytes` is the host channel: rank 0 passes the
    128-byte id it created, the others pass None, everybody gets rank 0's bytes
    back.  `from_torch_distributed` builds that channel from an initialised
    process group (any backend)."""

    def __init__(self, dev, rank: int, world: int, exchange):
        import ctypes as C
        from . import abi
        self.dev, self.rank, self.world = dev, int(rank), int(world)
        L = dev.L
        if not L.zg_nccl_load(_bundled_nccl()):
            abi.check()
            raise RuntimeError("no NCCL library found")
        dev.make_current()
        ident = None
        if self.rank == 0:
            buf = (C.c_ubyte * 128)()
            L.zg_nccl_unique_id(buf)
            abi.check()
            ident = bytes(buf)
        ident = exchange(ident)
        self.comm = L.zg_comm_init_rank((C.c_ubyte * 128).from_buffer_copy(ident), self.rank, self.world)
        abi.check()
        self._one = dev.from_numpy(np.zeros(1, np.float32))
        self._streams = []

    @classmethod
    def from_torch_distributed(cls, dev, group=None):
        import torch.distributed as dist

        def exchange(ident):
            box = [ident]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            return box[0]
        return cls(dev, dist.get_rank(group), dist.get_world_size(group), exchange)

    # collectives: asynchronous on `stream` (default: the device's stream), in place
    def allreduce(self, s, stream=None) -> None:
        self.dev.L.zg_allreduce(self.comm, s.ptr, s.len, s.dtype, stream or self.dev.stream)

    def reduce_scatter(self, send, recv, stream=None) -> None:
        self.dev.L.zg_reduce_scatter(self.comm, send.ptr, recv.ptr, recv.len, recv.dtype, stream or self.dev.stream)

    def all_gather(self, send, recv, stream=None) -> None:
        self.dev.L.zg_all_gather(self.comm, send.ptr, recv.ptr, send.len, send.dtype, stream or self.dev.stream)

    def new_stream(self):
        """A stream for collectives that should overlap the compute streams."""
        st = self.dev.L.init_stream()
        self._streams.append(st)
        return st

    def barrier(self) -> None:
        """Host barrier: a one-element all-reduce, then a stream synchronise."""
        self.allreduce(self._one)
        self.dev.sync()

    def close(self) -> None:
        if self.comm is not None:
            self.dev.sync()
            for st in self._streams:
                self.dev.L.stream_synchronize(st)
                self.dev.L.deinit_stream(st)
            self._streams = []
            self.dev.mem_cache_free(self._one)
            self.dev.L.zg_comm_destroy(self.comm)
            self.comm = None


def _bundled_nccl():
    """Path of the NCCL that ships with the Python environment (the newest one
    around), or None to let the library search the loader path."""
    try:
        import importlib.util
        import os
        spec = importlib.util.find_spec("nvidia.nccl")
        for base in (spec.submodule_search_locations if spec else []):
            cand = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                return cand.encode()
    except Exception:
        pass
    return None


class GradAllReduce:
    """Sum-all-reduce of a gradient buffer: `host` over a torch.distributed group
    (gloo; CPU tests of the host logic), `device` over an NcclComm."""

    def __init__(self, group=None, comm: "NcclComm" = None):
        self.group, self.comm = group, comm

    def host(self, grads: np.ndarray) -> np.ndarray:
        """In-place sum over ranks of a host array (gloo path)."""
        import torch
        import torch.distributed as dist
        t = torch.from_numpy(grads)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return grads

    def device(self, grads, stream=None) -> None:
        """In-place sum over ranks of a DeviceSlice, enqueued on the device's
        stream: ordered after the backward kernels and before the optimizer."""
        self.comm.allreduce(grads, stream)

    __call__ = device


class OverlappedGradAllReduce:
    """Per-layer all-reduce that overlaps the backward pass.

    `start(slice)` enqueues a sum-all-reduce of one slice of the gradient buffer
    on a communication stream of its own, ordered after the work already on the
    device's CURRENT stream (the side stream, where the layer's weight gradient
    was just issued), so neither the side stream nor the main stream waits for
    it.  `finish()` makes the device's current (main) stream wait for every
    started reduction -- call it before the optimizer kernel."""

    def __init__(self, comm: NcclComm):
        self.comm, self.dev = comm, comm.dev
        self.stream = comm.new_stream()

    def start(self, grads) -> None:
        self.dev.L.zg_stream_wait(self.stream, self.dev.stream)
        self.comm.allreduce(grads, self.stream)

    def finish(self) -> None:
        self.dev.L.zg_stream_wait(self.dev.stream, self.stream)


class PeerAllReduce:
    """Sum all-reduce of a small gradient buffer in one kernel per rank over
    peer memory (zg_allreduce_oneshot): for latency-bound buffers (up to a few
    MB) on the GPUs of one box.  A plain kernel launch on the device stream, so
    the whole data-parallel step -- backward, reduction, update -- can be
    captured into one CUDA graph.  The IPC handles of the comm regions travel
    over the communicator (zg_comm_peer_regions)."""

    def __init__(self, dev, n_elems: int, comm: NcclComm):
        import ctypes as C
        from . import abi
        self.dev, self.comm = dev, comm
        self.rank, self.world = comm.rank, comm.world
        if self.world > 8:
            raise ValueError("PeerAllReduce supports up to 8 ranks")
        self.cap = (int(n_elems) + 3) // 4 * 4
        L = dev.L
        dev.make_current()
        self.region = L.zg_comm_alloc(self.cap, self.world)
        if not self.region:
            raise MemoryError("comm region")
        ptrs = (C.c_void_p * self.world)()
        rc = L.zg_comm_peer_regions(comm.comm, self.region, ptrs, dev.stream)
        abi.check()
        if rc != 0:
            raise RuntimeError("exchange of the comm regions failed")
        self.ptrs = ptrs
        self._opened = [ptrs[r] for r in range(self.world) if r != self.rank]
        comm.barrier()  # every region is cleared and mapped before the first launch

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
        self.comm.barrier()  # nobody still reads a region that is about to go away
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

    def __init__(self, trainer, comm: NcclComm):
        if not trainer.bf16 or trainer.opt != "adam":
            raise ValueError("ZeroShardedAdam drives an MlpTrainer in bf16 mode with Adam")
        self.tr, self.comm = trainer, comm
        self.rank, self.world = comm.rank, comm.world
        self.stream = comm.new_stream()
        tr, W = trainer, self.world
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

    def start(self, l: int) -> None:
        """Call on the side stream right after layer l's weight gradient was issued."""
        tr, d = self.tr, self.tr.dev
        off, n, c = self.layers[l]
        d.L.zg_stream_wait(self.stream, d.stream)
        self.comm.reduce_scatter(tr.grads.view(off, n), tr.grads.view(off + self.rank * c, c), self.stream)

    def finish(self) -> None:
        from . import opspec
        tr, d = self.tr, self.tr.dev
        d.L.zg_stream_wait(d.stream, self.stream)
        clip = tr.clip
        if clip:
            d.segment_sumsq(tr.grads, self.owned, self.sumsq)
            self.comm.allreduce(self.sumsq)
            d.dispatch(opspec.sqrt_fwd(self.sumsq, self.sumsq))
        d.dispatch(opspec.adam(tr.params, tr.grads, tr.m, tr.v, self.owned, tr.t + 1, tr.lr, tr.beta1, tr.beta2, tr.eps,
                               "given" if clip else False, tr.max_norm, tr.delta, self.sumsq, tr.params_bf16, tr.t_dev))
        tr.t += len(self.owned)
        for off, n, c in self.layers:
            self.comm.all_gather(tr.params_bf16.view(off + self.rank * c, c), tr.params_bf16.view(off, n))

    def free(self) -> None:
        self.tr.dev.mem_cache_free(self.sumsq)
