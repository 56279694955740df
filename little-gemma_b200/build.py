"""Build liblg_b200.so in-tree: host C (gcc) + sm_100a CUDA (nvcc), one shared library.

    python little-gemma_b200/build.py [--mtp-n 4] [--force] [--ptxas-v]

The library is compiled for sm_100a only; nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
INC = os.path.join(ROOT, "include")
HOST = os.path.join(HERE, "csrc", "host")
CUDA = os.path.join(HERE, "csrc", "cuda")
LIB = os.path.join(HERE, "liblg_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

HOST_SRC = ["lg_gguf.c", "lg_quant.c", "lg_setup.c", "lg_session.c"]
CUDA_SRC = ["lg_engine.cu"]
DEPS = [os.path.join(HOST, f) for f in HOST_SRC + ["lg_host.h"]] + \
       [os.path.join(CUDA, f) for f in CUDA_SRC + ["lg_kernels.cuh", "lg_capi.cuh", "lg_prefill.cuh", "lg_attn_deep.cuh", "lg_attn_cluster.cuh"]] + \
       [os.path.join(INC, "lg_abi.h"), os.path.join(INC, "lg_b200.h"), os.path.abspath(__file__)]


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in DEPS)


def build(mtp_n: int = 4, force: bool = False, ptxas_v: bool = False, stamps: bool = False) -> str:
    if not force and not stale():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    defs = [f"-DLG_MTP_N={mtp_n}"] + (["-DLG_STAMPS"] if stamps else [])     # stamps: profiling build with phase time stamps
    for f in HOST_SRC:
        o = os.path.join(objdir, f + ".o")
        subprocess.check_call(["gcc", "-O2", "-fPIC", "-std=gnu11", "-Wall", "-Wextra", *defs, f"-I{INC}", f"-I{HOST}",
                               "-c", os.path.join(HOST, f), "-o", o])
        objs.append(o)
    for f in CUDA_SRC:
        o = os.path.join(objdir, f + ".o")
        cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
               "-Xcompiler", "-fPIC", *defs, f"-I{INC}", f"-I{HOST}", f"-I{CUDA}", "-c", os.path.join(CUDA, f), "-o", o]
        if ptxas_v:
            cmd[1:1] = ["-Xptxas", "-v"]
        subprocess.check_call(cmd)
        objs.append(o)
    subprocess.check_call([NVCC, "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--mtp-n", type=int, default=4)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true")
    ap.add_argument("--stamps", action="store_true", help="profiling build: kernels record phase time stamps (lg_debug_stamps)")
    a = ap.parse_args()
    print(build(a.mtp_n, a.force or a.stamps, a.ptxas_v, a.stamps))
