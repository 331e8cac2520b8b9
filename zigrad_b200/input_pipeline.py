"""Input staging in front of the training step: batches travel from
page-locked host memory to the device on a COPY stream, double-buffered, while
the previous batch trains on the compute stream.

The reference's MNIST loader builds one tensor per sample from CSV text and the
step consumes host tensors directly (``examples/mnist/src/dataset.zig:11-67``);
on a GPU the host-to-device copy of a batch (26 MB at batch 8192) costs more
than the step itself, so it is overlapped here.  Ordering between the two
streams uses one pair of events per staging slot (no host synchronisation in
steady state): ``put`` records the slot's "copied" event right after that
slot's copies and ``get`` makes the compute stream wait for the event of the
slot it returns -- not for copies enqueued later; ``release`` records the
slot's "consumed" event on the compute stream and the next ``put`` into that
slot makes the copy stream wait for it -- not for later steps:

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
_ALIGN = 256  # tensors of a packed batch start on this boundary (keeps 128-bit and TMA alignment)


class BatchStager:
    def __init__(self, dev: CudaDevice, tensors: Sequence[Tuple[int, int]], depth: int = 2, packed: bool = False):
        """tensors: (element count, dtype id) per input tensor of a batch.
        packed: the tensors of a batch live back to back in ONE device block per
        slot and ONE page-locked host buffer per batch (`pack`), so a batch
        travels as a single copy (one DMA set-up instead of one per tensor)."""
        self.dev, self.depth, self.packed = dev, int(depth), bool(packed)
        self.copy_stream = dev.L.init_stream()
        self.spec = [(int(n), int(dt)) for n, dt in tensors]
        self.slots: List[List[DeviceSlice]] = []
        if packed:
            self._offsets, off = [], 0
            for n, dt in self.spec:
                self._offsets.append(off)
                off += (n * np.dtype(_NP[dt]).itemsize + _ALIGN - 1) // _ALIGN * _ALIGN
            self._packed_bytes = off
            self._blocks = [dev.mem_cache_alloc(abi.SINGLE, off // 4) for _ in range(self.depth)]
            for blk in self._blocks:
                self.slots.append([DeviceSlice(blk.ptr + o, n, dt, 0) for o, (n, dt) in zip(self._offsets, self.spec)])
        else:
            self._blocks = []
            self.slots = [[dev.mem_cache_alloc(dt, n) for n, dt in self.spec] for _ in range(self.depth)]
        self._pinned = []
        self._put = self._got = 0
        self._copied = [dev.L.zg_event_create() for _ in range(self.depth)]
        self._consumed = [dev.L.zg_event_create() for _ in range(self.depth)]
        self._was_consumed = [False] * self.depth
        abi.check()
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

    def pack(self, arrays: Sequence[np.ndarray]) -> np.ndarray:
        """One page-locked byte buffer holding the tensors of a batch at the
        offsets of a packed slot (packed stagers only); pass it to put()."""
        if not self.packed:
            raise RuntimeError("pack() needs a stager created with packed=True")
        buf = self.pinned((self._packed_bytes,), np.uint8)
        buf[:] = 0
        for a, o, (n, dt) in zip(arrays, self._offsets, self.spec):
            a = np.ascontiguousarray(a, dtype=_NP[dt]).ravel()
            if a.size != n:
                raise ValueError("batch tensor of %d elements, slot holds %d" % (a.size, n))
            buf[o:o + a.nbytes] = a.view(np.uint8)
        return buf

    # ----------------------------------------------------------------- stream
    def put(self, arrays) -> None:
        """Enqueue the host-to-device copy of one batch into the next free slot
        (asynchronous when the arrays are page-locked).  `arrays`: the batch's
        tensors, or for a packed stager the buffer pack() returned."""
        if self._put - self._got >= self.depth:
            raise RuntimeError("all %d slots hold batches that were not released yet" % self.depth)
        k = self._put % self.depth
        slot = self.slots[k]
        if self._was_consumed[k]:  # the step that last read this slot must be done before it is overwritten
            self.dev.L.zg_stream_wait_event(self.copy_stream, self._consumed[k])
        if self.packed:
            if arrays.nbytes != self._packed_bytes:
                raise ValueError("packed batch of %d bytes, slot holds %d" % (arrays.nbytes, self._packed_bytes))
            self.dev.L.memcpy_HtoD(self._blocks[k].ptr, arrays.ctypes.data, arrays.nbytes, self.copy_stream)
            arrays = ()
        for a, d in zip(arrays, slot):
            if a.nbytes != d.nbytes:
                raise ValueError("batch tensor of %d bytes, slot holds %d" % (a.nbytes, d.nbytes))
            self.dev.L.memcpy_HtoD(d.ptr, a.ctypes.data, a.nbytes, self.copy_stream)
        self.dev.L.zg_event_record(self._copied[k], self.copy_stream)
        self._put += 1

    def get(self) -> List[DeviceSlice]:
        """The oldest staged batch; the compute stream waits for its copy."""
        if self._got >= self._put:
            raise RuntimeError("no staged batch")
        k = self._got % self.depth
        self.dev.L.zg_stream_wait_event(self.dev.stream, self._copied[k])
        return self.slots[k]

    def current_slot(self) -> int:
        """Index of the slot get() returns next (for callers that keep one captured graph per slot)."""
        return self._got % self.depth

    def release(self) -> None:
        """Call after the step that consumed get()'s batch was enqueued: the next
        copy into that slot waits for the compute stream up to this point."""
        k = self._got % self.depth
        self.dev.L.zg_event_record(self._consumed[k], self.dev.stream)
        self._was_consumed[k] = True
        self._got += 1

    def bytes_per_batch(self) -> int:
        """Bytes one put() copies."""
        return self._packed_bytes if self.packed else sum(d.nbytes for d in self.slots[0])

    def close(self) -> None:
        self.dev.sync()
        self.dev.L.stream_synchronize(self.copy_stream)
        for blk in self._blocks:
            self.dev.mem_cache_free(blk)
        for slot in ([] if self.packed else self.slots):
            for d in slot:
                self.dev.mem_cache_free(d)
        self.slots, self._blocks = [], []
        for p in self._pinned:
            self.dev.L.zg_host_free_pinned(p)
        self._pinned = []
        for ev in self._copied + self._consumed:
            self.dev.L.zg_event_destroy(ev)
        self._copied, self._consumed = [], []
        self.dev.L.deinit_stream(self.copy_stream)
