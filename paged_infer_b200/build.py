"""Build ``libpaged_infer_cuda.so`` in-tree with nvcc for sm_100a.

``python -m paged_infer_b200.build`` compiles every ``csrc/*.cu`` (one object
per file, in parallel) and links them into
``paged_infer_b200/libpaged_infer_cuda.so``.  This is what a Rust ``build.rs``
would do for the reference crate; the object files are kept under
``paged_infer_b200/build/`` so that unchanged sources are not recompiled.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libpaged_infer_cuda.so")
HOST_SRC = os.path.join(HERE, "host", "pi_host_shim.cpp")
HOST_LIB = os.path.join(HERE, "libpaged_infer_host.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    # no --use_fast_math: the quantiser needs IEEE division and rounding
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _ccbin() -> list:
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + sorted(glob.glob(os.path.join(INCLUDE, "*.h")))
    jobs = []
    objects = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc()] + NVCC_FLAGS + _ccbin() + (["-Xptxas", "-v"] if ptxas_info else []) + ["-I", INCLUDE, "-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or ptxas_info or r.returncode != 0:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {cmd[-3]}")
    if jobs or _newer(LIB, objects):
        cmd = [nvcc(), "-shared"] + _ccbin() + ["-o", LIB] + objects + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("linking libpaged_infer_cuda.so failed")
    build_host()
    return LIB


def build_host() -> str:
    """``libpaged_infer_host.so``: the C ABI over the host-side block bookkeeping (g++ only, no CUDA)."""
    deps = [HOST_SRC, os.path.join(INCLUDE, "paged_infer_memory.hpp")]
    if _newer(HOST_LIB, deps):
        gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
        r = subprocess.run([gxx, "-std=c++17", "-O2", "-Wall", "-Wextra", "-fPIC", "-shared", HOST_SRC, "-o", HOST_LIB],
                           capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("building libpaged_infer_host.so failed")
    return HOST_LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
