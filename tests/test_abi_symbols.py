"""CPU-only checks of the drop-in boundary: the library loads without a GPU,
exports every symbol that include/*.h declares, and the ctypes table covers
exactly those declarations.  No compute call is made here."""
import ctypes
import os
import re

import pytest

from zigrad_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")


def declared_symbols():
    names = {}
    for h in sorted(os.listdir(INC)):
        if not h.endswith(".h"):
            continue
        text = open(os.path.join(INC, h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"EXTERN_C\s+[^;(]*?\b(\w+)\s*\(", text):
            names[m.group(1)] = h
    return names


def test_library_builds_and_loads():
    from zigrad_b200 import build
    path = build.build()
    assert os.path.exists(path)
    assert abi.lib() is not None


def test_every_declared_symbol_is_exported():
    decl = declared_symbols()
    assert len(decl) > 90, len(decl)
    L = ctypes.CDLL(abi.LIB_PATH)
    missing = [n for n in decl if not hasattr(L, n)]
    assert not missing, missing


def test_ctypes_table_matches_headers():
    decl = set(declared_symbols())
    table = set(abi.SIGNATURES)
    assert decl - table == set(), "declared in include/*.h but not bound: %s" % sorted(decl - table)
    assert table - decl == set(), "bound but not declared: %s" % sorted(table - decl)


def test_reference_abi_names_are_kept():
    """The 67 entry points of the reference's three headers (cuda_utils.h,
    blas_conflux.h, nn_conflux.h) keep their names."""
    ref = """mem_alloc memcpy_HtoD memcpy_DtoH memcpy_DtoD mem_fill mem_sequence mem_random mem_free mem_take mem_page_size
    init_device check_last_error device_synchronize device_total_memory device_count init_stream deinit_stream
    stream_synchronize init_cublas_handle deinit_cublas_handle init_cudnn_handle deinit_cudnn_handle init_cutensor_handle
    deinit_cutensor_handle open_capture save_capture free_capture run_capture mem_map mem_unmap init_memmap reset_memmap
    deinit_memmap mem_map_alloc dot gemv gemm ger nrm2 clip_nrm2 max_fwd max_bwd reduce_sum scale axpy addition subtraction
    multiplication division get_contraction_plan get_reduce_plan get_permutate_plan reduce permutate contraction relu_fwd
    relu_bwd smax_vec_fwd smax_vec_bwd smax_2D_row_fwd smax_2D_row_bwd clamp nll_loss_1D_index_fwd nll_loss_1D_index_bwd
    nll_loss_1D_encode_fwd nll_loss_1D_encode_bwd pow_exp""".split()
    assert len(ref) == 67
    decl = declared_symbols()
    assert [n for n in ref if n not in decl] == []


def test_status_calls_work_without_a_gpu():
    L = abi.lib()
    L.zg_clear_error()
    assert L.zg_last_error() == 0
    assert L.zg_device_available() in (0, 1)
    assert L.zg_get_math_mode() == abi.MATH_FP32X3


def test_device_object_refuses_to_run_without_gpu():
    from zigrad_b200.device import CudaDevice
    if abi.lib().zg_device_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        CudaDevice(0)
