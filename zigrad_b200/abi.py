"""ctypes binding of the C ABI exported by ``libamalgamate.so``.

This is the Python twin of what ``src/cuda/root.zig`` does with ``@cImport``
in the reference: every function declared in ``include/*.h`` gets its argument
and result types here, nothing more.  The library is loaded from the package
directory (``zigrad_b200/lib``); a missing library is an error -- there is no
fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libamalgamate.so")

len_t = C.c_ulong
dtype_t = C.c_ubyte
SINGLE, DOUBLE, BF16 = 0, 1, 2
vp = C.c_void_p
dbl = C.c_double
i32 = C.c_int
b8 = C.c_bool
u8 = C.c_ubyte
lenp = C.POINTER(len_t)


class _Handle(C.Structure):
    _fields_ = [("ptr", vp)]


class StreamWrapper(_Handle):
    pass


class CublasWrapper(_Handle):
    pass


class CutensorWrapper(_Handle):
    pass


class CudnnWrapper(_Handle):
    pass


class GraphWrapper(_Handle):
    pass


class DevicePropertiesWrapper(_Handle):
    pass


class MemmapWrapper(_Handle):
    pass


class CacheWrapper(_Handle):
    pass


class CommWrapper(_Handle):
    pass


class CutensorPlanWrapper(C.Structure):
    _fields_ = [("plan", vp), ("scratch_len", len_t)]


class Block(C.Structure):
    _fields_ = [("ptr", vp), ("ctx", len_t)]


class Segment(C.Structure):
    _fields_ = [("offset", len_t), ("len", len_t)]


ADD, MIN, MAX, MUL = 0, 1, 2, 3
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_RELU_MASK = 0, 1, 2, 3
MATH_FP32X3, MATH_TF32, MATH_FFMA = 0, 1, 2
UN_EXP, UN_SQRT, UN_RSQRT, UN_TANH, UN_SIGM, UN_POW = 0, 1, 2, 3, 4, 5
LABEL_ONEHOT, LABEL_INDEX = 0, 1
SMAX_FAST, SMAX_MAX, SMAX_LOG = 0, 1, 2
RDX_NONE, RDX_MEAN, RDX_SUM = 0, 1, 2
UNIFORM, NORMAL = 0, 1

S, CB, CT, CD = StreamWrapper, CublasWrapper, CutensorWrapper, CudnnWrapper
u8p = C.POINTER(C.c_ubyte)

# name -> (restype, [argtypes]); one entry per declaration in include/*.h
SIGNATURES = {
    # ---- cuda_utils.h
    "mem_alloc": (vp, [len_t, S]),
    "mem_free": (None, [vp, S]),
    "memcpy_HtoD": (None, [vp, vp, len_t, S]),
    "memcpy_DtoH": (None, [vp, vp, len_t, S]),
    "memcpy_DtoD": (None, [vp, vp, len_t, S]),
    "mem_fill": (None, [dtype_t, vp, len_t, vp, S]),
    "mem_sequence": (None, [dtype_t, vp, len_t, vp, vp, S]),
    "mem_random": (None, [dtype_t, vp, len_t, u8, C.c_uint, S]),
    "mem_take": (None, [dtype_t, vp, len_t, vp, len_t, vp, S]),
    "mem_page_size": (len_t, [C.c_uint]),
    "init_device": (DevicePropertiesWrapper, [C.c_uint]),
    "check_last_error": (None, []),
    "device_synchronize": (None, []),
    "device_total_memory": (len_t, [C.c_uint]),
    "device_count": (C.c_uint, []),
    "init_stream": (S, []),
    "deinit_stream": (None, [S]),
    "stream_synchronize": (None, [S]),
    "zg_stream_wait": (None, [S, S]),
    "zg_event_create": (vp, []),
    "zg_event_destroy": (None, [vp]),
    "zg_event_record": (None, [vp, S]),
    "zg_stream_wait_event": (None, [S, vp]),
    "zg_host_alloc_pinned": (vp, [len_t]),
    "zg_host_free_pinned": (None, [vp]),
    "init_cublas_handle": (CB, [S]),
    "deinit_cublas_handle": (None, [CB]),
    "init_cudnn_handle": (CD, [S]),
    "deinit_cudnn_handle": (None, [CD]),
    "init_cutensor_handle": (CT, [S]),
    "deinit_cutensor_handle": (None, [CT]),
    "open_capture": (GraphWrapper, [S]),
    "save_capture": (None, [GraphWrapper, S]),
    "free_capture": (None, [GraphWrapper, S]),
    "run_capture": (None, [GraphWrapper, S]),
    "mem_map": (vp, [C.c_uint, C.c_size_t]),
    "mem_unmap": (None, [C.c_uint, vp, C.c_size_t]),
    "init_memmap": (MemmapWrapper, [C.c_uint]),
    "reset_memmap": (None, [MemmapWrapper]),
    "deinit_memmap": (None, [MemmapWrapper]),
    "mem_map_alloc": (None, [MemmapWrapper, vp, len_t]),
    # ---- blas_conflux.h
    "dot": (None, [dtype_t, CB, vp, vp, vp, len_t]),
    "gemv": (None, [dtype_t, CB, vp, vp, vp, len_t, len_t, b8, dbl, dbl]),
    "gemm": (None, [dtype_t, CB, vp, vp, vp, len_t, len_t, len_t, b8, b8, len_t, len_t, len_t, dbl, dbl]),
    "ger": (None, [dtype_t, CB, vp, vp, vp, len_t, len_t, len_t, dbl]),
    "nrm2": (None, [dtype_t, CB, vp, vp, len_t]),
    "clip_nrm2": (None, [dtype_t, CB, vp, vp, len_t, dbl, dbl]),
    "max_fwd": (None, [dtype_t, S, vp, vp, len_t]),
    "max_bwd": (None, [dtype_t, S, vp, vp, vp, vp, len_t]),
    "reduce_sum": (None, [dtype_t, CB, vp, vp, len_t]),
    "scale": (None, [dtype_t, CB, vp, len_t, dbl]),
    "axpy": (None, [dtype_t, CB, vp, vp, len_t, vp]),
    "addition": (None, [dtype_t, S, vp, vp, vp, len_t, len_t, len_t]),
    "subtraction": (None, [dtype_t, S, vp, vp, vp, len_t, len_t, len_t]),
    "multiplication": (None, [dtype_t, S, vp, vp, vp, len_t, len_t, len_t]),
    "division": (None, [dtype_t, S, vp, vp, vp, len_t, len_t, len_t]),
    "get_contraction_plan": (CutensorPlanWrapper, [CT, dtype_t, lenp, u8p, len_t, lenp, u8p, len_t, lenp, u8p, len_t]),
    "get_reduce_plan": (CutensorPlanWrapper, [CT, dtype_t, lenp, u8p, len_t, lenp, u8p, len_t, i32]),
    "get_permutate_plan": (CutensorPlanWrapper, [CT, dtype_t, lenp, u8p, len_t, lenp, u8p, len_t]),
    "reduce": (None, [CT, vp, vp, vp, vp, len_t, vp, vp]),
    "permutate": (None, [CT, vp, vp, vp, vp, len_t, vp]),
    "contraction": (None, [CT, vp, vp, vp, vp, vp, len_t, vp, vp]),
    # ---- nn_conflux.h
    "relu_fwd": (None, [dtype_t, S, vp, vp, len_t]),
    "relu_bwd": (None, [dtype_t, S, vp, vp, vp, len_t]),
    "smax_vec_fwd": (None, [dtype_t, CD, vp, vp, len_t, u8]),
    "smax_vec_bwd": (None, [dtype_t, CD, vp, vp, vp, len_t]),
    "smax_2D_row_fwd": (None, [dtype_t, CD, vp, vp, len_t, len_t]),
    "smax_2D_row_bwd": (None, [dtype_t, CD, vp, vp, vp, len_t, len_t]),
    "clamp": (None, [dtype_t, S, vp, vp, len_t, dbl, dbl]),
    "nll_loss_1D_index_fwd": (None, [dtype_t, CD, vp, len_t, vp, len_t, b8, u8]),
    "nll_loss_1D_index_bwd": (None, [dtype_t, CD, vp, vp, len_t, len_t, u8]),
    "nll_loss_1D_encode_fwd": (None, [dtype_t, CD, vp, vp, vp, len_t, b8, u8]),
    "nll_loss_1D_encode_bwd": (None, [dtype_t, CD, vp, vp, vp, len_t, u8]),
    "pow_exp": (None, [dtype_t, S, vp, vp, len_t]),
    # ---- zg_b200.h
    "zg_last_error": (i32, []),
    "zg_last_error_message": (C.c_char_p, []),
    "zg_clear_error": (None, []),
    "zg_device_available": (i32, []),
    "zg_set_device": (None, [C.c_uint]),
    "zg_capture_kernel_count": (len_t, [GraphWrapper]),
    "zg_set_math_mode": (None, [i32]),
    "zg_get_math_mode": (i32, []),
    "zg_bmm_sm_budget": (None, [i32]),
    "zg_sm_count": (i32, []),
    "zg_bmm": (None, [dtype_t, dtype_t, S, vp, vp, vp, len_t, len_t, len_t, len_t, len_t, len_t, b8, b8, len_t, len_t, len_t,
                      dbl, dbl, i32, vp, vp, vp]),
    "zg_relu_inplace_bwd": (None, [dtype_t, S, vp, vp, len_t]),
    "zg_clamp_bwd": (None, [dtype_t, S, vp, vp, vp, len_t, dbl, dbl]),
    "zg_unary_fwd": (None, [dtype_t, S, i32, vp, vp, len_t, dbl]),
    "zg_unary_bwd": (None, [dtype_t, S, i32, vp, vp, vp, len_t, dbl]),
    "zg_pow_bwd": (None, [dtype_t, S, vp, vp, vp, len_t, dbl, dbl]),
    "zg_unary_inplace_bwd": (None, [dtype_t, S, i32, vp, vp, len_t]),
    "zg_relu_mask_fwd": (None, [dtype_t, S, vp, vp, len_t]),
    "zg_relu_mask_bwd": (None, [dtype_t, S, vp, vp, len_t]),
    "zg_clamp_mask_fwd": (None, [dtype_t, S, vp, vp, vp, len_t, dbl, dbl]),
    "zg_clamp_mask_bwd": (None, [dtype_t, S, vp, vp, vp, len_t]),
    "zg_transpose": (None, [dtype_t, S, vp, vp, len_t, len_t, dbl]),
    "zg_fold_rows": (None, [dtype_t, S, vp, vp, len_t, len_t, dbl, dbl]),
    "zg_fold_rows_noalloc": (None, [dtype_t, S, vp, vp, len_t, len_t, dbl, dbl]),
    "zg_fold_cols": (None, [dtype_t, S, vp, vp, len_t, len_t, dbl, dbl]),
    "zg_sum_along": (None, [dtype_t, S, vp, lenp, len_t, len_t, vp, dbl, dbl]),
    "zg_max_along": (None, [dtype_t, S, vp, lenp, len_t, len_t, vp]),
    "zg_unbroadcast": (None, [dtype_t, S, vp, lenp, len_t, vp, lenp, len_t, vp, dbl, dbl]),
    "zg_broadcast": (None, [dtype_t, S, vp, len_t, vp, len_t, dbl, dbl]),
    "zg_softmax_ce_fwd_bwd": (None, [dtype_t, S, vp, vp, i32, len_t, len_t, len_t, dbl, vp, vp, i32, vp, vp]),
    "zg_smooth_l1_fwd_bwd": (None, [dtype_t, S, vp, vp, len_t, dbl, vp, vp]),
    "zg_mlp_tail_supported": (i32, [dtype_t, len_t, len_t, len_t]),
    "zg_mlp_tail_fwd_bwd": (None, [dtype_t, S, len_t, len_t, len_t, len_t, vp, vp, vp, vp, vp, vp, i32, len_t, dbl,
                                   vp, vp, vp, vp, vp, vp, vp, vp, vp, i32]),
    "zg_sgd_step": (None, [dtype_t, S, vp, vp, C.POINTER(Segment), len_t, dbl, i32, dbl, dbl, vp, i32]),
    "zg_adam_step": (None, [dtype_t, S, vp, vp, vp, vp, C.POINTER(Segment), len_t, len_t, dbl, dbl, dbl, dbl, i32, dbl, dbl, vp, vp, vp]),
    "zg_adam_step_part": (None, [dtype_t, S, vp, vp, vp, vp, C.POINTER(Segment), len_t, len_t, dbl, dbl, dbl, dbl, i32, dbl, dbl, vp, vp, vp, i32]),
    "zg_segment_sumsq": (None, [dtype_t, S, vp, C.POINTER(Segment), len_t, vp]),
    "zg_soft_update": (None, [dtype_t, S, vp, vp, len_t, dbl]),
    "zg_cast": (None, [dtype_t, dtype_t, S, vp, vp, len_t]),
    # ---- peer-memory all-reduce
    "zg_comm_alloc": (vp, [len_t, C.c_uint]),
    "zg_comm_free": (None, [vp]),
    "zg_ipc_export": (None, [vp, u8p]),
    "zg_ipc_open": (vp, [u8p]),
    "zg_ipc_close": (None, [vp]),
    "zg_comm_error": (C.c_int, [vp, S]),
    "zg_comm_set_spin_limit": (None, [C.c_uint]),
    "zg_allreduce_oneshot": (None, [S, vp, len_t, C.c_uint, C.c_uint, C.POINTER(vp), len_t]),
    "zg_allreduce_sgd_oneshot": (None, [S, vp, vp, len_t, dbl, C.c_uint, C.c_uint, C.POINTER(vp), len_t, i32]),
    # ---- library collectives (NCCL bound at run time)
    "zg_nccl_load": (C.c_int, [C.c_char_p]),
    "zg_nccl_unique_id": (None, [u8p]),
    "zg_comm_init_rank": (CommWrapper, [u8p, C.c_uint, C.c_uint]),
    "zg_comm_destroy": (None, [CommWrapper]),
    "zg_comm_rank": (C.c_uint, [CommWrapper]),
    "zg_comm_world": (C.c_uint, [CommWrapper]),
    "zg_allreduce": (None, [CommWrapper, vp, len_t, dtype_t, S]),
    "zg_reduce_scatter": (None, [CommWrapper, vp, vp, len_t, dtype_t, S]),
    "zg_all_gather": (None, [CommWrapper, vp, vp, len_t, dtype_t, S]),
    "zg_comm_peer_regions": (C.c_int, [CommWrapper, vp, C.POINTER(vp), S]),
    "zg_scatter_add": (None, [dtype_t, S, vp, vp, len_t, vp]),
    "zg_scatter_add_2d": (None, [dtype_t, S, vp, vp, len_t, len_t, vp]),
    "zg_scatter_add_csr": (None, [dtype_t, S, vp, vp, len_t, vp]),
    "zg_segment_sum_csr": (None, [dtype_t, S, vp, vp, len_t, vp]),
    "zg_gather_rows": (None, [dtype_t, S, vp, vp, len_t, len_t, vp, vp]),
    "zg_scatter_gcn_deg_scaled": (None, [dtype_t, S, vp, vp, vp, vp, vp, len_t, len_t]),
    "zg_scatter_gcn_deg_scaled_bwd": (None, [dtype_t, S, vp, vp, vp, vp, vp, vp, vp, len_t, len_t]),
    "zg_csr_gcn_propagate": (None, [dtype_t, S, vp, vp, vp, vp, vp, len_t, len_t, len_t, len_t, C.c_int, C.c_int, vp]),
    "zg_cache_create": (CacheWrapper, [C.c_uint, len_t]),
    "zg_cache_destroy": (None, [CacheWrapper]),
    "zg_cache_alloc": (Block, [CacheWrapper, len_t, S]),
    "zg_cache_free": (None, [CacheWrapper, Block, S]),
    "zg_cache_scratch": (vp, [CacheWrapper, len_t, S]),
    "zg_cache_clear": (None, [CacheWrapper]),
    "zg_cache_stats": (None, [CacheWrapper, lenp]),
}

_lib = None


class LibraryMissing(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load libamalgamate.so and type every entry point.  Raises if the
    library has not been built (``python -m zigrad_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            "%s not found: build it with `python -m zigrad_b200.build` (there is no CPU fallback)" % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError here = a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


class DeviceError(RuntimeError):
    """Raised by ``check()`` when the library's sticky status is set; the Zig
    shim panics at the same point (the reference exits the process)."""

    def __init__(self, code: int, message: str):
        super().__init__("zigrad-b200 error %d: %s" % (code, message))
        self.code = code


def check() -> None:
    L = lib()
    code = L.zg_last_error()
    if code != 0:
        msg = L.zg_last_error_message().decode(errors="replace")
        L.zg_clear_error()
        raise DeviceError(code, msg)
