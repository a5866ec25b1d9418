"""Build libfastface_b200.so in-tree: C99 host code (gcc) + sm_100a CUDA code (nvcc).

    python -m fastface_b200.build [--force]

The C99 side (model files, layer plan, public API) and the CUDA side (kernels,
device context) meet at the C-ABI declared in include/ff_cuda.h.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from typing import List

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
INC = os.path.join(ROOT, "include")
OBJ = os.path.join(PKG, "csrc", "_obj")
LIB = os.path.join(PKG, "libfastface_b200.so")
CLI = os.path.join(PKG, "fastface_int8_b200")     # reference-compatible command-line driver

HOST_SRCS = ["csrc/host/ff_model.c", "csrc/host/ff_plan.c", "csrc/host/fastface_api.c"]
CUDA_SRCS = ["csrc/cuda/ffcu_context.cu", "csrc/cuda/kernels_simt.cu", "csrc/cuda/conv_tc.cu",
             "csrc/cuda/conv_tc_generic.cu", "csrc/cuda/conv_tc_ws.cu", "csrc/cuda/conv_tc_pair.cu", "csrc/cuda/conv_tc_wsp.cu", "csrc/cuda/conv_tc_chain.cu", "csrc/cuda/conv_tc_sc.cu", "csrc/cuda/conv_tc_fc.cu", "csrc/cuda/conv_tc_stem.cu", "csrc/cuda/peak_probe.cu", "csrc/cuda/cos_sim.cu", "csrc/cuda/fc_small_noalloc.cu", "csrc/cuda/winograd_f23.cu"]

# -fmad=false: the epilogues state every fp32 rounding explicitly; the compiler must not fuse.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-fmad=false", "-Xcompiler", "-fPIC", "-I" + INC] + os.environ.get("FF_NVCC_EXTRA", "").split()
# -ffp-contract=off: 1/(s+1e-9f) and friends are evaluated exactly as written.
GCC_FLAGS = ["-std=c11", "-O2", "-fPIC", "-Wall", "-ffp-contract=off", "-I" + INC,
             "-I" + os.path.join(PKG, "csrc", "host")]


def _nvcc() -> str:
    for c in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: List[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers() -> List[str]:
    hs = [os.path.join(INC, f) for f in os.listdir(INC)]
    for sub in ("csrc/host", "csrc/cuda"):
        d = os.path.join(PKG, sub)
        hs += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".h", ".cuh"))]
    return hs


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    objs = []
    procs = []
    for rel in HOST_SRCS + CUDA_SRCS:
        src = os.path.join(PKG, rel)
        obj = os.path.join(OBJ, os.path.basename(rel) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            if rel.endswith(".cu"):
                cmd = [_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj]
            else:
                cmd = ["gcc"] + GCC_FLAGS + ["-c", src, "-o", obj]
            if verbose:
                print(" ".join(cmd))
            procs.append((rel, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for rel, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"compiling {rel} failed:\n{out.decode()}")
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart", "-lpthread", "-lm"]
        if verbose:
            print(" ".join(cmd))
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout.decode()}")
    cli_src = os.path.join(PKG, "csrc", "host", "fastface_cli.c")
    if force or _stale(CLI, [cli_src, LIB] + hdrs):
        cmd = ["gcc", "-std=c11", "-O2", "-Wall", "-I" + INC, cli_src, "-o", CLI, "-L" + PKG, "-lfastface_b200",
               "-Wl,-rpath,$ORIGIN", "-lm"]
        if verbose:
            print(" ".join(cmd))
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if r.returncode != 0:
            raise RuntimeError(f"building the CLI failed:\n{r.stdout.decode()}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
