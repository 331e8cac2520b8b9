"""In-tree build of the device library (``zigrad_b200/lib/libamalgamate.so``).

Every ``csrc/*.cu`` is compiled for sm_100a only and linked into ONE shared
library whose name is the one the reference's build links against
(``build.zig:195-197``: ``libamalgamate``).  nvcc cross-compiles, so this
works on a machine without a GPU.

    python -m zigrad_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "lib", "obj")
LIB = os.path.join(HERE, "lib", "libamalgamate.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
          "--expt-relaxed-constexpr", "-I", INCLUDE]
# Memory-bound kernels are compiled without FMA contraction so that multi-step
# formulas (Adam, alpha*x+beta*y) round like the CPU loops they restate; the
# GEMM file keeps FMA.
NO_FMAD = {"elementwise.cu", "reduce.cu", "loss.cu", "optim.cu", "index.cu", "runtime.cu", "allocator.cu"}


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC)")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest(src: str, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for name in sorted(os.listdir(CSRC)) + sorted(os.listdir(INCLUDE)):
        if name.endswith((".cuh", ".h")) or name == src:
            base = CSRC if os.path.exists(os.path.join(CSRC, name)) else INCLUDE
            with open(os.path.join(base, name), "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _compile(src: str, force: bool, verbose: bool) -> str:
    flags = ARCH + COMMON + (["--fmad=false"] if src in NO_FMAD else [])
    if verbose:
        flags = flags + ["-Xptxas", "-v"]
    obj = os.path.join(OBJ, src[:-3] + ".o")
    stamp = obj + ".sha"
    dig = _digest(src, flags)
    if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj
    cmd = [nvcc()] + flags + ["-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    if verbose:
        sys.stderr.write(r.stderr)
    with open(stamp, "w") as f:
        f.write(dig)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        cmd = [nvcc()] + ARCH + ["-shared", "-o", LIB] + objs + ["-Xcompiler", "-fPIC", "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB


HOST_EXAMPLE = os.path.join(HERE, "lib", "mlp_step_main")


def build_host_example(force: bool = False) -> str:
    """The C++ host side (zigrad_b200/host/*.hpp) linked against the library:
    the MLP-step program that tests/test_gpu_cpp_host.py runs.  g++ only."""
    src = os.path.join(os.path.dirname(HERE), "tests", "cpp", "mlp_step_main.cpp")
    deps = [src, LIB] + [os.path.join(HERE, "host", f) for f in sorted(os.listdir(os.path.join(HERE, "host")))]
    if not force and os.path.exists(HOST_EXAMPLE) and os.path.getmtime(HOST_EXAMPLE) >= max(os.path.getmtime(d) for d in deps):
        return HOST_EXAMPLE
    gxx = shutil.which("g++") or "g++"
    cmd = [gxx, "-std=c++17", "-O2", "-Wall", "-I", os.path.dirname(HERE), src, "-o", HOST_EXAMPLE, "-L", os.path.dirname(LIB),
           "-lamalgamate", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed for the C++ host example:\n%s\n%s" % (r.stdout, r.stderr))
    return HOST_EXAMPLE


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v (registers, spills, shared memory)")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    print(build_host_example(a.force))
