"""The boundary through a compiler: a plain-C translation unit that includes
include/b2vm.h, and the C++ adapter header (include/b2_runtime_adapter.h: the
reference's OclRuntime / VmProgram / LoadedProgram over the C ABI) driving the
reference's device test cases (pjrt_plugin/src/runtime_test.cc:136-267)."""
import os
import subprocess

import numpy as np
import pytest

import kat_programs as K
from conftest import package

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")
SRC = os.path.join(ROOT, "tests", "adapter")


def _libdir():
    return os.path.dirname(package().find_library())


def _link_args():
    d = _libdir()
    return ["-L" + d, "-l:libb2vm.so", "-Wl,-rpath," + d]


def test_header_is_plain_c_and_links(tmp_path):
    exe = str(tmp_path / "include_c")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I" + INC,
                    os.path.join(SRC, "include_c.c"), "-o", exe, *_link_args()], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "bad magic" in r.stdout


def test_adapter_header_compiles(tmp_path):
    subprocess.run(["g++", "-std=c++14", "-Wall", "-Wextra", "-Werror", "-I" + INC, "-c",
                    os.path.join(SRC, "runtime_test.cc"), "-o", str(tmp_path / "runtime_test.o")], check=True)


@pytest.mark.gpu
def test_reference_device_test_through_the_adapter(tmp_path):
    exe = str(tmp_path / "runtime_test")
    subprocess.run(["g++", "-std=c++14", "-O1", "-I" + INC, os.path.join(SRC, "runtime_test.cc"), "-o", exe,
                    *_link_args()], check=True)
    specs = []
    for name, build, rtol in (("A_two_level", K.kat_a_two_level, 0.0), ("B_while", K.kat_b_while, 0.0),
                              ("C_region_gelu", K.kat_c_region_gelu, 1e-5)):
        blob, ins, want = build()
        (tmp_path / f"{name}.blob").write_bytes(blob)
        for i, a in enumerate(ins):
            (tmp_path / f"{name}.in{i}").write_bytes(np.ascontiguousarray(a, dtype=np.float32).tobytes())
        for o, a in enumerate(want):
            (tmp_path / f"{name}.want{o}").write_bytes(np.ascontiguousarray(a, dtype=np.float32).tobytes())
        specs.append(f"{name}:{len(ins)}:{len(want)}:{rtol}")
    r = subprocess.run([exe, str(tmp_path), *specs], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("PASS ") == 3, r.stdout
