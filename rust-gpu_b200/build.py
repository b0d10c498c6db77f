"""Builds libt0b200 (shared + static) in-tree with nvcc for sm_100a.

    python rust-gpu_b200/build.py [--force] [--verbose]

Objects go to rust-gpu_b200/build/, the libraries to rust-gpu_b200/lib/.  nvcc cross-compiles
without a GPU.  Only files whose sources or headers changed are rebuilt.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

SOURCES = ["host_config.cpp", "cost_model.cpp", "tuner.cpp", "runtime.cu", "gemm_sm100.cu", "gemm_sm100_pair.cu", "gemm_sm100_splitk.cu", "aux_kernels.cu",
           "w4a16.cu", "w4a16_stream.cu", "w4a16_umma.cu", "multi_gpu.cu", "no_alloc.cu", "matmul_f32.cu", "host_pipeline.cu"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-Xptxas", "-v", "--expt-relaxed-constexpr"]
# extra compiler flags, e.g. T0_NVCC_EXTRA=-DT0_GEMM_TRACE (per-role time stamps in the pair GEMM kernel); use with --force
NVCC_FLAGS += os.environ.get("T0_NVCC_EXTRA", "").split()


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(HERE, "..", "include", "t0b200.h"))
    return hs


def _compile(src: str, force: bool, verbose: bool) -> str:
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    newest = max(os.path.getmtime(p) for p in [path] + _headers())
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj
    cmd = [NVCC] + NVCC_FLAGS + ["-x", "cu", "-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OBJ, os.path.splitext(src)[0] + ".ptxas.log")
    with open(log, "w") as f:
        f.write(r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"nvcc failed on {src}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    so = os.path.join(LIB, "libt0b200.so")
    a = os.path.join(LIB, "libt0b200.a")
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(so) or os.path.getmtime(so) < newest:
        subprocess.run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", so] + objs +
                       ["-cudart", "static", "-lpthread", "-ldl"], check=True)
    if force or not os.path.exists(a) or os.path.getmtime(a) < newest:
        if os.path.exists(a):
            os.remove(a)
        subprocess.run(["ar", "rcs", a] + objs, check=True)
    return so


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
