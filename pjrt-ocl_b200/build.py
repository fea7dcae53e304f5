"""Builds libb2vm.so (C++ host runtime + the sm_100a megakernel) in-tree with nvcc.

Every source is compiled to its own object (in parallel, and only when it or a
header changed), then linked; the objects live in `build/` next to this file.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
SOURCES = ["vm_kernel.cu", "runtime.cc", "loader.cc", "vmprog.cc", "static_sum.cu"]
OUT = os.path.join(HERE, "libb2vm.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "b2vm.h"))
    return hs


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(nvcc: str, src: str, obj: str, verbose: bool) -> str:
    cmd = [nvcc, *ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-c"]
    if verbose and src.endswith(".cu"):
        cmd += ["-Xptxas", "-v"]
    cmd += [src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJ, exist_ok=True)
    heads = _headers()
    jobs = []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, os.path.splitext(s)[0] + ".o")
        if force or _newer(obj, [src, *heads]):
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            logs = list(ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs))
        if verbose:
            sys.stderr.write("".join(logs))
    objs = [os.path.join(OBJ, os.path.splitext(s)[0] + ".o") for s in SOURCES]
    if jobs or _newer(OUT, objs):
        r = subprocess.run([nvcc, *ARCH, "-shared", "-cudart", "static", *objs, "-o", OUT],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
