"""Input staging in front of the training step: batches travel from
page-locked host memory to the device on a COPY stream, double-buffered, while
the previous batch trains on the compute stream.

The reference's MNIST loader builds one tensor per sample from CSV text and the
step consumes host tensors directly (``examples/mnist/src/dataset.zig:11-67``);
on a GPU the host-to-device copy of a batch (26 MB at batch 8192) costs more
than the step itself, so it is overlapped here.  Ordering between the two
streams uses ``zg_stream_wait`` only (no host synchronisation in steady
state):

    stager = BatchStager(dev, [(B * 784, SINGLE), (B * 10, SINGLE)])
    stager.put([X0, T0])                       # pinned host arrays (stager.pinned_like / .pinned)
    for i in range(steps):
        if i + 1 < steps: stager.put(next_batch(i + 1))   # H2D of batch i+1 overlaps step i
        X, T = stager.get()                    # compute stream now waits for batch i's copy
        trainer.step(X, T)
        stager.release()                       # the slot may be overwritten once this step is done
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence, Tuple

import numpy as np

from . import abi
from .device import CudaDevice, DeviceSlice

_NP = {abi.SINGLE: np.float32, abi.DOUBLE: np.float64, abi.BF16: np.uint16, 100: np.uint64}


class BatchStager:
    def __init__(self, dev: CudaDevice, tensors: Sequence[Tuple[int, int]], depth: int = 2):
        """tensors: (element count, dtype id) per input tensor of a batch."""
        self.dev, self.depth = dev, int(depth)
        self.copy_stream = dev.L.init_stream()
        self.spec = [(int(n), int(dt)) for n, dt in tensors]
        self.slots: List[List[DeviceSlice]] = [[dev.mem_cache_alloc(dt, n) for n, dt in self.spec] for _ in range(self.depth)]
        self._pinned = []
        self._put = self._got = 0
        dev.sync()

    # ------------------------------------------------------------ host memory
    def pinned(self, shape, dtype=np.float32) -> np.ndarray:
        """A page-locked numpy array (freed by close())."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape)) * dtype.itemsize
        p = self.dev.L.zg_host_alloc_pinned(max(n, 1))
        abi.check()
        if not p:
            raise MemoryError("pinned host allocation of %d bytes" % n)
        self._pinned.append(p)
        buf = (C.c_ubyte * max(n, 1)).from_address(p)
        return np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def pinned_like(self, a: np.ndarray) -> np.ndarray:
        out = self.pinned(a.shape, a.dtype)
        out[...] = a
        return out

    # ----------------------------------------------------------------- stream
    def put(self, arrays: Sequence[np.ndarray]) -> None:
        """Enqueue the host-to-device copy of one batch into the next free slot
        (asynchronous when the arrays are page-locked)."""
        if self._put - self._got >= self.depth:
            raise RuntimeError("all %d slots hold batches that were not released yet" % self.depth)
        slot = self.slots[self._put % self.depth]
        for a, d in zip(arrays, slot):
            if a.nbytes != d.nbytes:
                raise ValueError("batch tensor of %d bytes, slot holds %d" % (a.nbytes, d.nbytes))
            self.dev.L.memcpy_HtoD(d.ptr, a.ctypes.data, a.nbytes, self.copy_stream)
        self._put += 1

    def get(self) -> List[DeviceSlice]:
        """The oldest staged batch; the compute stream waits for its copy."""
        if self._got >= self._put:
            raise RuntimeError("no staged batch")
        self.dev.L.zg_stream_wait(self.dev.stream, self.copy_stream)
        return self.slots[self._got % self.depth]

    def current_slot(self) -> int:
        """Index of the slot get() returns next (for callers that keep one captured graph per slot)."""
        return self._got % self.depth

    def release(self) -> None:
        """Call after the step that consumed get()'s batch was enqueued: later
        copies into that slot wait for the compute stream up to this point."""
        self.dev.L.zg_stream_wait(self.copy_stream, self.dev.stream)
        self._got += 1

    def bytes_per_batch(self) -> int:
        return sum(d.nbytes for d in self.slots[0])

    def close(self) -> None:
        self.dev.sync()
        self.dev.L.stream_synchronize(self.copy_stream)
        for slot in self.slots:
            for d in slot:
                self.dev.mem_cache_free(d)
        self.slots = []
        for p in self._pinned:
            self.dev.L.zg_host_free_pinned(p)
        self._pinned = []
        self.dev.L.deinit_stream(self.copy_stream)
