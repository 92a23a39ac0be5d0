"""In-tree build of libnlh_b200.so (sm_100a only) with nvcc.

    python -m nl_hecate_b200.build [--force]

nvcc cross-compiles without a GPU. The shared library is written next to this
file so that it travels with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libnlh_b200.so")

SOURCES = ["runtime.cu", "memory_ffi.cu", "swa.cu", "swa_f32.cu", "adamw.cu",
           "static_scratch.cu", "wrapper.cu", "glue.cu", "opaque.cu", "opaque_rules.cu",
           "host_dispatch.cu", "mlp_memory.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libnlh_b200.so")
    return nvcc


def _deps(src: str):
    yield os.path.join(CSRC, src)
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".h")):
            yield os.path.join(CSRC, f)
    for f in os.listdir(INCLUDE):
        yield os.path.join(INCLUDE, f)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    objs, jobs = [], []
    for s in srcs:
        obj = os.path.join(OBJ_DIR, s.replace(".cu", ".o"))
        objs.append(obj)
        newest = max(os.path.getmtime(d) for d in _deps(s))
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < newest:
            jobs.append([nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, s), "-o", obj])

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)

    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
