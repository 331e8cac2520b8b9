"""``CudaDevice``: the host-side device object of this backend.

Python mirror of ``src/device/cuda_device.zig`` (the Zig struct that sits
behind ``DeviceReference``): it owns one stream, the op contexts, the
stream-ordered cache and a capture object, offers the ``mem_*`` calls of
``src/device/device_reference.zig:29-131`` and one method per ``opspec`` name,
and forwards each of them to the C ABI of ``libamalgamate.so``.  There is no
other implementation behind it: without the library or without a GPU it raises.
"""
from __future__ import annotations

import contextlib
import os

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import abi
from .abi import BF16, DOUBLE, SINGLE

_NP2ID = {np.dtype(np.float32): SINGLE, np.dtype(np.float64): DOUBLE}
_ITEMSIZE = {SINGLE: 4, DOUBLE: 8, BF16: 2}
USIZE = 100  # pseudo dtype id for index buffers (u64); never passed to the library
U8 = 101     # pseudo dtype id for byte masks (mem_alloc_byte_mask); never passed to the library


@dataclass
class DeviceSlice:
    """A typed view of device memory: Zig's ``[]T`` (plus the cache block handle
    that ``DeviceData.ctx`` carries when the memory came from ``mem_cache_alloc``)."""
    ptr: int
    len: int
    dtype: int = SINGLE
    ctx: int = 0

    @property
    def itemsize(self) -> int:
        return 8 if self.dtype == USIZE else (1 if self.dtype == U8 else _ITEMSIZE[self.dtype])

    @property
    def nbytes(self) -> int:
        return self.len * self.itemsize

    def view(self, offset: int, length: int) -> "DeviceSlice":
        assert 0 <= offset and offset + length <= self.len
        return DeviceSlice(self.ptr + offset * self.itemsize, length, self.dtype, 0)


class DeviceOOM(MemoryError):
    """error.DeviceOOM of src/allocators/device_data.zig:44."""


def _shape(s: Sequence[int]):
    return (abi.len_t * len(s))(*[int(v) for v in s])


def _f32(v: float):
    return C.byref(C.c_float(v))


class ExecutionGraph:
    """CUDA-graph capture of the device stream (cuda_device.zig:558-611)."""

    def __init__(self, dev: "CudaDevice"):
        self.dev = dev
        self.wrapper = None
        self.saved = False

    def open(self):
        self.free()
        self.dev.sync()
        self.wrapper = self.dev.L.open_capture(self.dev.stream)
        abi.check()
        self.saved = False

    def save(self):
        if self.wrapper is not None and not self.saved:
            self.dev.L.save_capture(self.wrapper, self.dev.stream)
            abi.check()
            self.saved = True

    def run(self):
        if self.wrapper is None:
            raise RuntimeError("UndefinedCapture")
        if not self.saved:
            raise RuntimeError("CaptureInProgress")
        self.dev.L.run_capture(self.wrapper, self.dev.stream)

    def free(self):
        self.save()
        if self.wrapper is not None:
            self.dev.sync()
            self.dev.L.free_capture(self.wrapper, self.dev.stream)
            self.wrapper = None

    def empty(self) -> bool:
        return self.wrapper is None

    def kernel_count(self) -> int:
        """Kernel launches one run() performs."""
        return int(self.dev.L.zg_capture_kernel_count(self.wrapper)) if self.wrapper is not None else 0

    def detach(self):
        """Hand the saved graph to the caller (several graphs can then coexist,
        e.g. one per resident input batch); returns an object with run()/free()."""
        self.save()
        g = ExecutionGraph(self.dev)
        g.wrapper, g.saved = self.wrapper, self.saved
        self.wrapper, self.saved = None, False
        return g


class CudaDevice:
    def __init__(self, device_number: int = 0, cache_max_bytes: int = 0, stream: Optional[int] = None):
        self.L = abi.lib()
        if not self.L.zg_device_available():
            raise RuntimeError("CudaDevice: no CUDA device is available (this backend has no CPU fallback)")
        self.device_number = int(device_number)
        self.properties = self.L.init_device(self.device_number)
        abi.check()
        if stream is None:
            self.stream = self.L.init_stream()
            self._own_stream = True
        else:  # adopt a stream created elsewhere (e.g. by the process's communication library)
            self.stream = abi.StreamWrapper(stream)
            self._own_stream = False
        self.cublas = self.L.init_cublas_handle(self.stream)
        self.cudnn = self.L.init_cudnn_handle(self.stream)
        self.cutensor = self.L.init_cutensor_handle(self.stream)
        self.cache = self.L.zg_cache_create(self.device_number, cache_max_bytes)
        self.capture = ExecutionGraph(self)
        self._side = None  # second stream for branches of independent work, created on first use
        self._sides = {}   # further side streams by index (branch(k), k >= 1)
        self._forked = []  # side streams used since the last join()
        abi.check()

    # ------------------------------------------------------------ lifecycle
    def deinit(self):
        if self.L is None:
            return
        self.sync()
        self.capture.free()
        self.L.zg_cache_destroy(self.cache)
        self.L.deinit_cudnn_handle(self.cudnn)
        self.L.deinit_cublas_handle(self.cublas)
        self.L.deinit_cutensor_handle(self.cutensor)
        if self._side is not None:
            self.L.deinit_stream(self._side)
            self._side = None
        for st in self._sides.values():
            self.L.deinit_stream(st)
        self._sides = {}
        if self._own_stream:
            self.L.deinit_stream(self.stream)
        self.L = None

    def reference(self):
        return self

    def is_compatible(self, other: "CudaDevice") -> bool:
        return self.device_number == other.device_number

    def sync(self):
        self.L.stream_synchronize(self.stream)
        abi.check()

    def make_current(self):
        self.L.zg_set_device(self.device_number)

    @contextlib.contextmanager
    def branch(self, k: int = 0, after=()):
        """Ops issued inside the block go to the device's k-th side stream,
        ordered after everything issued so far on the main stream (and on the
        side streams listed in `after`); they may
        overlap what the main stream (and the other side streams) run next.
        `join()` makes the main stream wait for them (required before the
        results are used and before a capture is saved)."""
        if os.environ.get("ZG_NO_BRANCH") == "1":  # everything in issue order on the main stream
            yield
            return
        if k == 0:
            if self._side is None:
                self._side = self.L.init_stream()
            side = self._side
        else:
            if k not in self._sides:
                self._sides[k] = self.L.init_stream()
            side = self._sides[k]
        main = self.stream
        self.L.zg_stream_wait(side, main)
        for j in after:
            other = self._side if j == 0 else self._sides.get(j)
            if other is not None and other.ptr != side.ptr:
                self.L.zg_stream_wait(side, other)
        if all(side.ptr != f.ptr for f in self._forked):
            self._forked.append(side)
        self.stream = side
        try:
            yield
        finally:
            self.stream = main

    def join(self):
        """The main stream waits for every side stream used since the last join
        (only those: a wait on a stream that is not part of a running capture
        would break the capture)."""
        for st in self._forked:
            self.L.zg_stream_wait(self.stream, st)
        self._forked = []

    # --------------------------------------------------------------- memory
    def mem_cache_alloc(self, dtype: int, n: int) -> DeviceSlice:
        size = n * DeviceSlice(0, 0, dtype).itemsize
        blk = self.L.zg_cache_alloc(self.cache, max(size, 1), self.stream)
        if not blk.ptr:
            abi.check()
            raise DeviceOOM("mem_cache_alloc(%d bytes)" % size)
        return DeviceSlice(blk.ptr, n, dtype, blk.ctx)

    def mem_cache_free(self, data: DeviceSlice):
        if data.ctx:
            self.L.zg_cache_free(self.cache, abi.Block(data.ptr, data.ctx), self.stream)
            data.ctx = 0

    def mem_cache_dupe(self, src: DeviceSlice) -> DeviceSlice:
        dst = self.mem_cache_alloc(src.dtype, src.len)
        self.mem_copy(src, dst)
        return dst

    def mem_alloc(self, dtype: int, n: int) -> DeviceSlice:
        if n == 0:
            return DeviceSlice(0, 0, dtype)
        size = n * DeviceSlice(0, 0, dtype).itemsize
        p = self.L.mem_alloc(size, self.stream)
        if not p:
            abi.check()
            raise DeviceOOM("mem_alloc(%d bytes)" % size)
        return DeviceSlice(p, n, dtype)

    def mem_alloc_byte_mask(self, n: int) -> DeviceSlice:
        """One bit per element: ceil(n/8) bytes (device_reference.zig:41-43)."""
        nb = (n + 7) // 8
        if nb == 0:
            return DeviceSlice(0, 0, U8)
        p = self.L.mem_alloc(nb, self.stream)
        if not p:
            abi.check()
            raise DeviceOOM("mem_alloc_byte_mask(%d bytes)" % nb)
        return DeviceSlice(p, nb, U8)

    def mem_free(self, s: DeviceSlice):
        if s.len:
            self.L.mem_free(s.ptr, self.stream)

    def mem_scratch(self, dtype: int, n: int) -> DeviceSlice:
        if n == 0:
            return DeviceSlice(0, 0, dtype)
        p = self.L.zg_cache_scratch(self.cache, n * _ITEMSIZE[dtype], self.stream)
        if not p:
            abi.check()
            raise DeviceOOM("mem_scratch")
        return DeviceSlice(p, n, dtype)

    def mem_fill(self, s: DeviceSlice, value: float):
        v = C.c_float(value) if s.dtype == SINGLE else C.c_double(value)
        self.L.mem_fill(s.dtype, s.ptr, s.len, C.byref(v), self.stream)

    def mem_sequence(self, s: DeviceSlice, initial: float, step: float):
        T = C.c_float if s.dtype == SINGLE else C.c_double
        self.L.mem_sequence(s.dtype, s.ptr, s.len, C.byref(T(initial)), C.byref(T(step)), self.stream)

    def mem_random(self, s: DeviceSlice, op: str, seed: int):
        self.L.mem_random(s.dtype, s.ptr, s.len, abi.NORMAL if op == "normal" else abi.UNIFORM, seed & 0xFFFFFFFF, self.stream)

    def mem_copy(self, src: DeviceSlice, dst: DeviceSlice):
        assert src.nbytes == dst.nbytes
        self.L.memcpy_DtoD(dst.ptr, src.ptr, src.nbytes, self.stream)

    def mem_transfer_htod(self, host: np.ndarray, dst: DeviceSlice):
        assert host.flags["C_CONTIGUOUS"] and host.nbytes == dst.nbytes, (host.nbytes, dst.nbytes)
        self.L.memcpy_HtoD(dst.ptr, host.ctypes.data, host.nbytes, self.stream)

    def mem_transfer_dtoh(self, src: DeviceSlice, host: np.ndarray):
        assert host.flags["C_CONTIGUOUS"] and host.nbytes == src.nbytes
        self.L.memcpy_DtoH(host.ctypes.data, src.ptr, src.nbytes, self.stream)

    def mem_take(self, src: DeviceSlice, idxs: DeviceSlice, dst: DeviceSlice):
        assert dst.len >= idxs.len
        self.L.mem_take(src.dtype, src.ptr, src.len, idxs.ptr, idxs.len, dst.ptr, self.stream)

    def clear_cache(self):
        self.L.zg_cache_clear(self.cache)

    # numpy conveniences used by the tests and drivers -----------------------
    def from_numpy(self, a: np.ndarray, cached: bool = True) -> DeviceSlice:
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint64:
            dt = USIZE
        elif a.dtype == np.uint16:
            dt = BF16  # raw bfloat16 bit patterns
        elif a.dtype == np.uint8:
            dt = U8    # byte masks
        else:
            dt = _NP2ID[a.dtype]
        s = self.mem_cache_alloc(dt, a.size) if cached else self.mem_alloc(dt, a.size)
        if a.size:
            self.mem_transfer_htod(a, s)
            self.sync()  # the host array may be a temporary
        return s

    def to_numpy(self, s: DeviceSlice, shape=None) -> np.ndarray:
        npdt = {SINGLE: np.float32, DOUBLE: np.float64, USIZE: np.uint64, BF16: np.uint16, U8: np.uint8}[s.dtype]
        out = np.empty(s.len, npdt)
        if s.len:
            self.mem_transfer_dtoh(s, out)
        self.sync()
        return out if shape is None else out.reshape(shape)

    # -------------------------------------------------------------- dispatch
    def dispatch(self, params):
        """DeviceReference.dispatch: select the method by the op's name."""
        name = type(params).op_name
        fn = getattr(self, name, None)
        if fn is None:
            raise NotImplementedError("Unimplemented: CudaDevice." + name)
        return fn(params)

    # element-wise ------------------------------------------------------------
    def _binary(self, fn, p):
        fn(p.z.dtype, self.stream, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len)

    def add(self, p):
        self._binary(self.L.addition, p)

    def sub(self, p):
        self._binary(self.L.subtraction, p)

    def mul(self, p):
        self._binary(self.L.multiplication, p)

    def div(self, p):
        self._binary(self.L.division, p)

    # linear algebra ---------------------------------------------------------
    def dot(self, p):
        self.L.dot(p.x.dtype, self.cublas, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len)

    def axpy(self, p):
        if isinstance(p.alpha, DeviceSlice):
            self.L.axpy(p.x.dtype, self.cublas, p.x.ptr, p.y.ptr, p.x.len, p.alpha.ptr)
        else:
            a = C.c_float(p.alpha) if p.x.dtype == SINGLE else C.c_double(p.alpha)
            self.L.axpy(p.x.dtype, self.cublas, p.x.ptr, p.y.ptr, p.x.len, C.cast(C.byref(a), C.c_void_p))

    def outer(self, p):
        self.L.ger(p.x.dtype, self.cublas, p.x.ptr, p.y.ptr, p.A.ptr, p.x.len, p.y.len, p.y.len, p.alpha)

    def transpose(self, p):
        self.L.zg_transpose(p.A.dtype, self.stream, p.A.ptr, p.B.ptr, p.m, p.n, p.alpha)

    def matvec(self, p):
        self.L.gemv(p.A.dtype, self.cublas, p.A.ptr, p.x.ptr, p.y.ptr, p.m, p.n, p.trans_a, p.alpha, p.beta)

    def matmul(self, p):
        self.L.gemm(p.A.dtype, self.cublas, p.A.ptr, p.B.ptr, p.C.ptr, p.m, p.n, p.k, p.trans_a, p.trans_b,
                    p.lda, p.ldb, p.ldc, p.alpha, p.beta)

    def bmm_acc(self, p):
        self.L.zg_bmm(p.A.dtype, p.C.dtype, self.stream, p.A.ptr, p.B.ptr, p.C.ptr,
                      p.A_shape[0], p.B_shape[0], p.C_shape[0], p.C_shape[1], p.C_shape[2], p.A_shape[2],
                      p.trans_a, p.trans_b, p.lda, p.ldb, p.ldc, p.alpha, p.beta, abi.EPI_NONE, None, None, None)

    def linear(self, p):
        epi = {"none": abi.EPI_NONE, "bias": abi.EPI_BIAS, "bias_relu": abi.EPI_BIAS_RELU, "relu_mask": abi.EPI_RELU_MASK}[p.epilogue]
        nA, nB, nC = p.n_batch
        if p.sm_budget:
            self.L.zg_bmm_sm_budget(p.sm_budget)
        self.L.zg_bmm(p.A.dtype, p.C.dtype, self.stream, p.A.ptr, p.B.ptr, p.C.ptr, nA, nB, nC, p.m, p.n, p.k,
                      p.trans_a, p.trans_b, p.lda, p.ldb, p.ldc, p.alpha, p.beta, epi,
                      p.bias.ptr if p.bias is not None else None, p.mask_src.ptr if p.mask_src is not None else None,
                      p.colsum.ptr if p.colsum is not None else None)

    def sum(self, p):
        self.L.reduce_sum(p.x.dtype, self.cublas, p.x.ptr, p.y.ptr, p.x.len)

    def scale(self, p):
        self.L.scale(p.x.dtype, self.cublas, p.x.ptr, p.x.len, p.alpha)

    def nrm2(self, p):
        self.L.nrm2(p.x.dtype, self.cublas, p.x.ptr, p.y.ptr, p.x.len)

    def clip_nrm2(self, p):
        scratch = self.mem_scratch(p.x.dtype, 1)
        self.L.clip_nrm2(p.x.dtype, self.cublas, p.x.ptr, scratch.ptr, p.x.len, p.max_norm, p.delta)

    # non-linear ---------------------------------------------------------------
    def _unary(self, op, p, param=0.0):
        self.L.zg_unary_fwd(p.x.dtype, self.stream, op, p.x.ptr, p.y.ptr, p.x.len, param)

    def exp_fwd(self, p):
        self._unary(abi.UN_EXP, p)

    def sqrt_fwd(self, p):
        self._unary(abi.UN_SQRT, p)

    def rsqrt_fwd(self, p):
        self._unary(abi.UN_RSQRT, p, p.eps)

    def tanh_fwd(self, p):
        self._unary(abi.UN_TANH, p)

    def sigm_fwd(self, p):
        self._unary(abi.UN_SIGM, p)

    def exp_bwd(self, p):
        self.L.zg_unary_bwd(p.y.dtype, self.stream, abi.UN_EXP, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0.0)

    def tanh_bwd(self, p):
        self.L.zg_unary_bwd(p.y.dtype, self.stream, abi.UN_TANH, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0.0)

    def sigm_bwd(self, p):
        self.L.zg_unary_bwd(p.y.dtype, self.stream, abi.UN_SIGM, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0.0)

    def sqrt_bwd(self, p):
        self.L.zg_unary_bwd(p.x.dtype, self.stream, abi.UN_SQRT, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.eps)

    def rsqrt_bwd(self, p):
        self.L.zg_unary_bwd(p.x.dtype, self.stream, abi.UN_RSQRT, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.eps)

    def pow_fwd(self, p):
        self.L.zg_unary_fwd(p.x.dtype, self.stream, abi.UN_POW, p.x.ptr, p.y.ptr, p.x.len, p.exp)

    def pow_fwd_(self, p):
        self.L.zg_unary_fwd(p.x.dtype, self.stream, abi.UN_POW, p.x.ptr, p.x.ptr, p.x.len, p.exp)

    def pow_bwd(self, p):
        self.L.zg_pow_bwd(p.x.dtype, self.stream, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.exp, p.eps)

    def sqrt_fwd_(self, p):
        self.L.zg_unary_fwd(p.x.dtype, self.stream, abi.UN_SQRT, p.x.ptr, p.x.ptr, p.x.len, 0.0)

    def tanh_inplace_bwd(self, p):
        self.L.zg_unary_inplace_bwd(p.x.dtype, self.stream, abi.UN_TANH, p.x.ptr, p.x_g.ptr, p.x.len)

    def sigm_inplace_bwd(self, p):
        self.L.zg_unary_inplace_bwd(p.x.dtype, self.stream, abi.UN_SIGM, p.x.ptr, p.x_g.ptr, p.x.len)

    def relu_mask_fwd(self, p):
        self.L.zg_relu_mask_fwd(p.x.dtype, self.stream, p.x.ptr, p.mask.ptr, p.x.len)

    def relu_mask_bwd(self, p):
        self.L.zg_relu_mask_bwd(p.x_g.dtype, self.stream, p.x_g.ptr, p.mask.ptr, p.x_g.len)

    def clamp_mask_fwd(self, p):
        self.L.zg_clamp_mask_fwd(p.x.dtype, self.stream, p.x.ptr, p.y.ptr, p.mask.ptr, p.x.len, p.min, p.max)

    def clamp_mask_bwd(self, p):
        self.L.zg_clamp_mask_bwd(p.x_g.dtype, self.stream, p.x_g.ptr, p.y_g.ptr, p.mask.ptr, p.x_g.len)

    def relu_fwd(self, p):
        self.L.relu_fwd(p.x.dtype, self.stream, p.x.ptr, p.y.ptr, p.x.len)

    def relu_bwd(self, p):
        self.L.relu_bwd(p.x.dtype, self.stream, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len)

    def relu_inplace_bwd(self, p):
        self.L.zg_relu_inplace_bwd(p.x.dtype, self.stream, p.x.ptr, p.x_g.ptr, p.x.len)

    def max_fwd(self, p):
        self.L.max_fwd(p.x.dtype, self.stream, p.x.ptr, p.y.ptr, p.x.len)

    def max_bwd(self, p):
        self.L.max_bwd(p.x.dtype, self.stream, p.x.ptr, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len)

    def clamp_fwd(self, p):
        self.L.clamp(p.x.dtype, self.stream, p.x.ptr, p.y.ptr, p.x.len, p.min, p.max)

    def clamp_bwd(self, p):
        self.L.zg_clamp_bwd(p.x.dtype, self.stream, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.min, p.max)

    # reductions ---------------------------------------------------------------
    def unbroadcast(self, p):
        self.L.zg_unbroadcast(p.x.dtype, self.stream, p.x.ptr, _shape(p.x_shape), len(p.x_shape), p.y.ptr,
                              _shape(p.y_shape), len(p.y_shape), p.scratch.ptr if p.scratch is not None and p.scratch.len else None,
                              p.alpha, p.beta)

    def broadcast(self, p):
        self.L.zg_broadcast(p.x.dtype, self.stream, p.x.ptr, p.x.len, p.y.ptr, p.y.len, p.alpha, p.beta)

    def sum_along(self, p):
        self.L.zg_sum_along(p.x.dtype, self.stream, p.x.ptr, _shape(p.x_shape), len(p.x_shape), p.dim, p.y.ptr, p.alpha, p.beta)

    def max_along(self, p):
        self.L.zg_max_along(p.x.dtype, self.stream, p.x.ptr, _shape(p.x_shape), len(p.x_shape), p.dim, p.y.ptr)

    # index ----------------------------------------------------------------------
    def scatter_add(self, p):
        self.L.zg_scatter_add(p.src.dtype, self.stream, p.src.ptr, p.offsets.ptr, p.src.len, p.dst.ptr)

    def scatter_add_2d(self, p):
        self.L.zg_scatter_add_2d(p.src.dtype, self.stream, p.src.ptr, p.indices.ptr, p.indices.len, p.stride, p.dst.ptr)

    def scatter_add_csr(self, p):
        self.L.zg_scatter_add_csr(p.src.dtype, self.stream, p.src.ptr, p.row_ptr.ptr, p.src.len, p.dst.ptr)

    def segment_sum_csr(self, p):
        self.L.zg_segment_sum_csr(p.src.dtype, self.stream, p.src.ptr, p.row_offsets.ptr, p.dst.len, p.dst.ptr)

    def scatter_gcn_deg_scaled(self, p):
        self.L.zg_scatter_gcn_deg_scaled(p.h.dtype, self.stream, p.dst.ptr, p.h.ptr, p.deg.ptr, p.src_indices.ptr,
                                         p.tgt_indices.ptr, p.stride, p.n_edge)

    def scatter_gcn_deg_scaled_bwd(self, p):
        self.L.zg_scatter_gcn_deg_scaled_bwd(p.h.dtype, self.stream, p.grad_output.ptr, p.h.ptr, p.deg.ptr,
                                             p.src_indices.ptr, p.tgt_indices.ptr, p.grad_h.ptr, p.grad_deg.ptr,
                                             p.stride, p.n_edge)

    def csr_gcn_propagate(self, p):
        epi = {"none": abi.EPI_NONE, "bias": abi.EPI_BIAS, "bias_relu": abi.EPI_BIAS_RELU}[p.epilogue]
        self.L.zg_csr_gcn_propagate(p.x.dtype, self.stream, p.out.ptr, p.x.ptr, p.deg.ptr, p.row_ptr.ptr, p.col_idx.ptr, p.n_rows, p.n_feat,
                                    p.ld_x, p.ld_out, 1 if p.transpose else 0, epi, p.bias.ptr if p.bias is not None else None)

    def gather_rows(self, src: DeviceSlice, idx: DeviceSlice, rows: int, cols: int, dst: DeviceSlice,
                    offsets_out: Optional[DeviceSlice] = None):
        self.L.zg_gather_rows(src.dtype, self.stream, src.ptr, idx.ptr, rows, cols, dst.ptr,
                              offsets_out.ptr if offsets_out is not None else None)

    # added ops -----------------------------------------------------------------
    def softmax_ce(self, p):
        kind = abi.LABEL_INDEX if p.labels.dtype == USIZE else abi.LABEL_ONEHOT
        div = float(p.loss_div if p.loss_div is not None else p.rows)
        self.L.zg_softmax_ce_fwd_bwd(p.logits.dtype, self.stream, p.logits.ptr, p.labels.ptr, kind, p.rows, p.classes, p.ld, div,
                                     p.loss.ptr, p.grad.ptr if p.grad is not None else None, int(p.accumulate),
                                     p.probs.ptr if p.probs is not None else None,
                                     p.bias_grad.ptr if p.bias_grad is not None else None)

    def sm_count(self) -> int:
        return int(self.L.zg_sm_count())

    def mlp_tail_supported(self, dtype: int, h1: int, h2: int, classes: int) -> bool:
        return bool(self.L.zg_mlp_tail_supported(dtype, h1, h2, classes))

    def mlp_tail(self, p):
        kind = abi.LABEL_INDEX if p.labels.dtype == USIZE else abi.LABEL_ONEHOT
        self.L.zg_mlp_tail_fwd_bwd(p.act0.dtype, self.stream, p.rows, p.h1, p.h2, p.classes, p.act0.ptr, p.W1.ptr, p.b1.ptr, p.W2.ptr,
                                   p.b2.ptr, p.labels.ptr, kind, p.ld_out, float(p.loss_div), p.act1.ptr, p.logits.ptr, p.loss.ptr,
                                   p.dlogits.ptr, p.dact1.ptr, p.dact0.ptr, p.db2.ptr, p.db1.ptr, p.db0.ptr, int(p.weights_ready))

    def smooth_l1(self, p):
        self.L.zg_smooth_l1_fwd_bwd(p.pred.dtype, self.stream, p.pred.ptr, p.target.ptr, p.pred.len, p.beta, p.loss.ptr,
                                    p.grad.ptr if p.grad is not None else None)

    @staticmethod
    def _segments(segs):
        arr = (abi.Segment * len(segs))()
        for i, (off, ln) in enumerate(segs):
            arr[i].offset, arr[i].len = int(off), int(ln)
        return arr

    def sgd(self, p):
        self.L.zg_sgd_step(p.params.dtype, self.stream, p.params.ptr, p.grads.ptr, self._segments(p.segments), len(p.segments),
                           p.lr, int(p.clip), p.max_norm, p.delta, p.norms.ptr if p.norms is not None else None,
                           int(bool(getattr(p, 'zero_grads', False))))

    def adam(self, p):
        self.L.zg_adam_step_part(p.params.dtype, self.stream, p.params.ptr, p.grads.ptr, p.m.ptr, p.v.ptr,
                                 self._segments(p.segments), len(p.segments), p.t_first, p.lr, p.beta1, p.beta2, p.eps,
                                 2 if p.clip == "given" else int(bool(p.clip)), p.max_norm, p.delta,
                                 p.norms.ptr if p.norms is not None else None,
                                 p.bf16_copy.ptr if p.bf16_copy is not None else None,
                                 p.step_counter.ptr if p.step_counter is not None else None, 1 if p.advance_counter else 0)

    def segment_sumsq(self, x: DeviceSlice, segments, out: DeviceSlice):
        self.L.zg_segment_sumsq(x.dtype, self.stream, x.ptr, self._segments(segments), len(segments), out.ptr)

    def soft_update(self, src: DeviceSlice, target: DeviceSlice, tau: float):
        self.L.zg_soft_update(src.dtype, self.stream, src.ptr, target.ptr, src.len, tau)

    def cast(self, src: DeviceSlice, dst: DeviceSlice):
        self.L.zg_cast(src.dtype, dst.dtype, self.stream, src.ptr, dst.ptr, src.len)
