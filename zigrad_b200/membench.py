"""Achieved HBM bandwidth of the memory-bound device ops at sizes well above L2.

    python -m zigrad_b200.membench [--mib 1024] [--reps 10] [--only add,adam]

Each op runs on its own buffers (working set >= 4x the 126 MB L2 unless
--mib shrinks it), is warmed up, captured into a CUDA graph and timed with
CUDA events on the device stream.  GB/s = ALGORITHMIC bytes (every operand
read once, every result written once) / time.  One JSON line per op.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import opspec
from .abi import BF16, SINGLE
from .device import CudaDevice


def run(mib=1024, reps=10, only=None):
    import torch
    ts = torch.cuda.Stream()
    dev = CudaDevice(0, stream=ts.cuda_stream)
    n = mib * (1 << 20) // 4            # fp32 elements of one "big" operand
    rows_w = 4096                        # matrix view [n / rows_w, rows_w]
    R = n // rows_w
    out = []

    def time_op(name, nbytes, fn, note=""):
        if only and name not in only:
            return
        fn()
        dev.sync()
        dev.capture.open()
        fn()
        dev.capture.save()
        g = dev.capture.detach()
        g.run()
        dev.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        for _ in range(reps):
            g.run()
        e1.record(ts)
        dev.sync()
        us = e0.elapsed_time(e1) * 1e3 / reps
        row = {"op": name, "bytes": nbytes, "us": round(us, 2), "GBps": round(nbytes / us * 1e-3, 1), "kernels": g.kernel_count()}
        if note:
            row["note"] = note
        g.free()
        out.append(row)
        print(json.dumps(row), flush=True)

    f = lambda k: dev.mem_cache_alloc(SINGLE, k)
    x, y, z = f(n), f(n), f(n)
    dev.mem_random(x, "normal", 1)
    dev.mem_random(y, "normal", 2)
    dev.mem_fill(z, 0.0)
    rowv, colv, one = f(rows_w), f(R), f(1)
    dev.mem_random(rowv, "normal", 3)
    dev.mem_fill(colv, 0.0)
    B4 = 4 * n

    time_op("fill", B4, lambda: dev.mem_fill(z, 1.0))
    time_op("copy", 2 * B4, lambda: dev.mem_copy(x, z))
    time_op("add", 3 * B4, lambda: dev.dispatch(opspec.add(x, y, z)))
    time_op("mul_inplace", 3 * B4, lambda: dev.dispatch(opspec.mul(x, z, z)))
    time_op("add_row_broadcast", 2 * B4, lambda: dev.dispatch(opspec.add(rowv, x, z)), "bias [4096] + matrix")
    time_op("relu_fwd", 2 * B4, lambda: dev.dispatch(opspec.relu_fwd(x, z)))
    time_op("relu_bwd", 4 * B4, lambda: dev.dispatch(opspec.relu_bwd(x, z, y)), "x_g += mask(x) * y_g")
    time_op("relu_inplace_bwd", 3 * B4, lambda: dev.dispatch(opspec.relu_inplace_bwd(x, z)))
    time_op("exp_fwd", 2 * B4, lambda: dev.dispatch(opspec.exp_fwd(y, z)))
    time_op("tanh_fwd", 2 * B4, lambda: dev.dispatch(opspec.tanh_fwd(y, z)))
    time_op("clamp_fwd", 2 * B4, lambda: dev.dispatch(opspec.clamp_fwd(y, z, -1.0, 1.0)))
    time_op("scale", 2 * B4, lambda: dev.dispatch(opspec.scale(z, 0.5)))
    time_op("axpy", 3 * B4, lambda: dev.dispatch(opspec.axpy(x, z, 0.5)))
    time_op("dot", 2 * B4, lambda: dev.dispatch(opspec.dot(x, y, one)))
    time_op("sum", B4, lambda: dev.dispatch(opspec.sum(x, one)))
    time_op("nrm2", B4, lambda: dev.dispatch(opspec.nrm2(x, one)))
    time_op("max_fwd", B4, lambda: dev.dispatch(opspec.max_fwd(x, one)))
    time_op("sum_along_rows", B4, lambda: dev.dispatch(opspec.sum_along(x, [R, rows_w], rowv, [1, rows_w], 0)), "[R,4096] -> [4096]")
    time_op("sum_along_cols", B4, lambda: dev.dispatch(opspec.sum_along(x, [R, rows_w], colv, [R, 1], 1)), "[R,4096] -> [R]")
    time_op("max_along_cols", B4, lambda: dev.dispatch(opspec.max_along(x, [R, rows_w], colv, [R, 1], 1)))
    time_op("unbroadcast_bias", B4, lambda: dev.dispatch(opspec.unbroadcast(x, [R, rows_w], rowv, [rows_w], None, 1.0, 0.0)))
    time_op("transpose", 2 * B4, lambda: dev.dispatch(opspec.transpose(x, z, R, rows_w, 0.0)))

    # bf16 cast
    xb = dev.mem_cache_alloc(BF16, n)
    time_op("cast_f32_bf16", 6 * n, lambda: dev.cast(x, xb))
    time_op("cast_bf16_f32", 6 * n, lambda: dev.cast(xb, z))
    dev.mem_cache_free(xb)

    # fused softmax + cross-entropy forward/backward over index labels
    for C in (1000, 10, 64, 128):
        rows = n // C
        lab = dev.from_numpy(np.random.Generator(np.random.PCG64(C)).integers(0, C, rows).astype(np.uint64))
        lg = x.view(0, rows * C)
        dl = z.view(0, rows * C)
        db = f(C)
        time_op("softmax_ce_C%d" % C, 8 * rows * C + 8 * rows,
                lambda: dev.dispatch(opspec.softmax_ce(lg, lab, rows, C, one, dl, 65536.0, accumulate=False, bias_grad=db)),
                "logits read + dlogits written, u64 labels, fused bias gradient, loss divisor 65536 (a global batch)")
        dev.mem_cache_free(lab)
        dev.mem_cache_free(db)

    # optimizers over a flat buffer of 8 tensors
    m_, v_ = f(n), f(n)
    dev.mem_fill(m_, 0.0)
    dev.mem_fill(v_, 0.0)
    seg = [(i * (n // 8), n // 8) for i in range(8)]
    norms = f(8)
    time_op("sgd", 3 * B4, lambda: dev.dispatch(opspec.sgd(z, y, seg, 0.01)))
    time_op("sgd_clip", 4 * B4, lambda: dev.dispatch(opspec.sgd(z, y, seg, 0.01, True, 10.0, 1e-6, norms)), "norm pass + update that rewrites grads")
    time_op("adam", 7 * B4, lambda: dev.dispatch(opspec.adam(z, y, m_, v_, seg, 1, 1e-3)))
    pb = dev.mem_cache_alloc(BF16, n)
    cnt = dev.from_numpy(np.zeros(1, np.uint64))
    time_op("adam_clip_bf16copy", 8 * B4 + 2 * n,
            lambda: dev.dispatch(opspec.adam(z, y, m_, v_, seg, 1, 1e-3, 0.9, 0.999, 1e-8, True, 10.0, 1e-6, norms, pb, cnt)),
            "norm pass (grads read) + update (p,g,m,v read; p,m,v written; bf16 copy written)")
    time_op("soft_update", 3 * B4, lambda: dev.soft_update(x, z, 0.005))

    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=1024, help="size of one big fp32 operand")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    run(a.mib, a.reps, set(a.only.split(",")) if a.only else None)
