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
SOURCES = ["runtime.cc", "loader.cc", "vmprog.cc", "static_sum.cu"]
KERNEL = "vm_kernel.cu"      # compiled once per entry of csrc/variants.h
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


def variants():
    """[(name, family mask)] from csrc/variants.h (the one list the C++ side uses too)."""
    import re
    text = open(os.path.join(CSRC, "variants.h")).read()
    fam = {m.group(1): 1 << int(m.group(2))
           for m in re.finditer(r"(kFam\w+) = 1u << (\d+)", open(os.path.join(CSRC, "format.h")).read())}
    fam["kFamAll"] = 0xFFFFFFFF
    macros = {m.group(1): m.group(2) for m in re.finditer(r"#define (B2_FAMS_\w+) \((.*?)\)\n", text)}

    def mask(expr: str) -> int:
        for k, v in macros.items():
            expr = expr.replace(k, v)
        total = 0
        for tok in re.findall(r"kFam\w+", expr):
            total |= fam[tok]
        return total
    body = text[text.index("#define B2_VARIANT_LIST(X)"):]
    return [(m.group(1), mask(m.group(2))) for m in re.finditer(r"X\((\w+), ([^\\\n]*)\)\s*(?:\\|\n)", body)]


def _compile(nvcc: str, src: str, obj: str, verbose: bool, defines=()) -> str:
    cmd = [nvcc, *ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-c", *defines]
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
    units = [(os.path.join(CSRC, s), os.path.join(OBJ, os.path.splitext(s)[0] + ".o"), ()) for s in SOURCES]
    for name, mask in variants():
        units.append((os.path.join(CSRC, KERNEL), os.path.join(OBJ, f"vm_kernel_{name}.o"),
                      (f"-DB2_VARIANT={name}", f"-DB2_FAMILIES={mask:#x}u")))
    jobs = [u for u in units if force or _newer(u[1], [u[0], *heads])]
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            logs = list(ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose, j[2]), jobs))
        if verbose:
            for j, log in zip(jobs, logs):
                sys.stderr.write(f"==== {os.path.basename(j[1])}\n{log}")
    objs = [u[1] for u in units]
    if jobs or _newer(OUT, objs):
        r = subprocess.run([nvcc, *ARCH, "-shared", "-cudart", "static", *objs, "-o", OUT],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
