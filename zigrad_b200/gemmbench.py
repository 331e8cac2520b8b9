"""Timing of single GEMMs through the `linear` op (zg_bmm).

    python -m zigrad_b200.gemmbench                       # the shapes of the wide bf16 MLP (config c3) + the headline MLP's
    python -m zigrad_b200.gemmbench --m 8192 --n 4096 --k 4096 --dtype bf16 --epi bias_relu [--ta] [--tb] [--c-bf16]   # --dtype: bf16 | f32 (3xTF32) | tf32 | ffma (fp32 FFMA kernel)

Each GEMM runs on 4 distinct A operands in turn (so the inputs of consecutive
launches differ), is captured into a CUDA graph and timed with CUDA events on
the device stream.  TFLOP/s = 2 m n k / time; with --cublas the same shape is
also timed through torch.matmul (the library GEMM) for reference.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import abi, opspec
from .abi import BF16, SINGLE
from .device import CudaDevice

C3 = [
    ("c3 fwd hidden", 8192, 4096, 4096, False, True, "bf16", True, "bias_relu", 0.0),
    ("c3 fwd out", 8192, 1000, 4096, False, True, "bf16", False, "bias", 0.0),
    ("c3 dX hidden", 8192, 4096, 4096, False, False, "bf16", True, "relu_mask", 0.0),
    ("c3 dX out", 8192, 4096, 1000, False, False, "bf16", True, "relu_mask", 0.0),
    ("c3 dW hidden", 4096, 4096, 8192, True, False, "bf16", False, "none", 1.0),
    ("c3 dW out", 1000, 4096, 8192, True, False, "bf16", False, "none", 1.0),
    ("mlp L1 fwd fp32x3", 8192, 128, 784, False, True, "f32", False, "bias_relu", 0.0),
    ("mlp L2 fwd fp32x3", 8192, 64, 128, False, True, "f32", False, "bias_relu", 0.0),
    ("mlp dW1 fp32x3", 128, 784, 8192, True, False, "f32", False, "none", 1.0),
    ("square 4096 fp32x3", 4096, 4096, 4096, False, True, "f32", False, "none", 0.0),
    ("square 4096 tf32", 4096, 4096, 4096, False, True, "tf32", False, "none", 0.0),
]


def run_one(dev, ts, name, m, n, k, ta, tb, dtype, c_bf16, epi, beta, reps=10, cublas=False, R=4):
    import torch
    bf16 = dtype == "bf16"
    dev.L.zg_set_math_mode(abi.MATH_TF32 if dtype == "tf32" else (abi.MATH_FFMA if dtype == "ffma" else abi.MATH_FP32X3))
    a_shape = (k, m) if ta else (m, k)
    b_shape = (n, k) if tb else (k, n)
    g = np.random.default_rng(0)

    def mk(shape):
        f = dev.from_numpy(g.standard_normal(shape).astype(np.float32))
        if not bf16:
            return f
        b = dev.mem_cache_alloc(BF16, int(np.prod(shape)))
        dev.cast(f, b)
        dev.sync()
        dev.mem_cache_free(f)
        return b

    As = [mk(a_shape) for _ in range(R)]
    B = mk(b_shape)
    Cb = dev.mem_cache_alloc(BF16 if c_bf16 else SINGLE, m * n)
    if not c_bf16:
        dev.mem_fill(Cb, 0.0)
    bias = dev.from_numpy(np.zeros(n, np.float32))
    mask = None
    if epi == "relu_mask":
        mask = dev.mem_cache_alloc(BF16 if c_bf16 else SINGLE, m * n)
        if c_bf16:
            t = dev.from_numpy(np.ones(m * n, np.float32))
            dev.cast(t, mask)
            dev.sync()
            dev.mem_cache_free(t)
        else:
            dev.mem_fill(mask, 1.0)

    def op(A):
        dev.dispatch(opspec.linear(A, B, Cb, m, n, k, ta, tb, a_shape[1], b_shape[1], n, 1.0, beta, epi,
                                   bias if epi.startswith("bias") else None, mask))

    op(As[0])
    dev.sync()
    dev.capture.open()
    for A in As:
        op(A)
    dev.capture.save()
    gr = dev.capture.detach()
    nk = gr.kernel_count()
    for _ in range(2):
        gr.run()
    dev.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ts)
    for _ in range(reps):
        gr.run()
    e1.record(ts)
    dev.sync()
    us = e0.elapsed_time(e1) * 1e3 / (reps * R)
    gr.free()
    row = {"gemm": name, "m": m, "n": n, "k": k, "trans": ("T" if ta else "N") + ("T" if tb else "N"), "dtype": dtype,
           "out": "bf16" if c_bf16 else "f32", "epilogue": epi, "beta": beta, "us": round(us, 2),
           "TFLOPs": round(2.0 * m * n * k / us * 1e-6, 1), "kernels_per_gemm": nk / R}
    if cublas:
        td = torch.bfloat16 if bf16 else torch.float32
        if dtype == "tf32":
            torch.backends.cuda.matmul.allow_tf32 = True
        ta_ = torch.randn(a_shape, device="cuda", dtype=td)
        tb_ = torch.randn(b_shape, device="cuda", dtype=td)
        f = lambda: torch.matmul(ta_.T if ta else ta_, tb_.T if tb else tb_)
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(reps * R):
            f()
        s1.record()
        torch.cuda.synchronize()
        us2 = s0.elapsed_time(s1) * 1e3 / (reps * R)
        row["library_us"] = round(us2, 2)
        row["library_TFLOPs"] = round(2.0 * m * n * k / us2 * 1e-6, 1)
        torch.backends.cuda.matmul.allow_tf32 = False
    for s in As + [B, Cb, bias] + ([mask] if mask is not None else []):
        dev.mem_cache_free(s)
    dev.L.zg_set_math_mode(abi.MATH_FP32X3)
    print(json.dumps(row), flush=True)
    return row


if __name__ == "__main__":
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int)
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--ta", action="store_true")
    ap.add_argument("--tb", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32", "tf32", "ffma"])
    ap.add_argument("--c-bf16", action="store_true")
    ap.add_argument("--epi", default="none", choices=["none", "bias", "bias_relu", "relu_mask"])
    ap.add_argument("--beta", type=float, default=0.0)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul on the same shape")
    ap.add_argument("--operands", type=int, default=4, help="distinct A operands used in turn (1 keeps A in L2 when it fits)")
    a = ap.parse_args()
    ts = torch.cuda.Stream()
    dev = CudaDevice(0, stream=ts.cuda_stream)
    if a.m:
        run_one(dev, ts, "custom", a.m, a.n, a.k, a.ta, a.tb, a.dtype, a.c_bf16, a.epi, a.beta, a.reps, a.cublas, R=a.operands)
    else:
        for cfg in C3:
            run_one(dev, ts, *cfg, reps=a.reps, cublas=a.cublas)
