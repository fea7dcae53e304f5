"""CPU-side checks of the C ABI: the library loads, exports exactly what
include/b2vm.h declares, and the host-only half (parse + queries) behaves like
the reference parser (pjrt_plugin/src/runtime.cc:90-251;
tests/test_lowering.py:246-260 for the rejection cases). No compute calls."""
import os
import re
import struct

import numpy as np
import pytest

from conftest import ROOT, Golden, golden_names, package

import kat_programs as K


def test_header_and_library_agree_on_the_entry_points():
    vm = package()
    header = open(os.path.join(ROOT, "include", "b2vm.h")).read()
    code = re.sub(r"/\*.*?\*/", "", header, flags=re.S)          # declarations only, no comments
    declared = sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", code)))
    assert declared == sorted(vm.EXPORTS)
    lib = vm.lib()
    for name in declared:
        assert getattr(lib, name) is not None


@pytest.mark.parametrize("name", golden_names())
def test_parse_accepts_every_reference_blob(name):
    vm = package()
    g = Golden(name)
    p = vm.VmProgram.Parse(g.blob)
    assert p.n_outputs == len(g.expected) and p.n_inputs == len(g.args)
    for spec, exp in zip(p.outputs, g.expected):
        assert spec["bytes"] == exp.nbytes and spec["shape"] == exp.shape and spec["dtype"] == exp.dtype
    for spec, a in zip(p.inputs, g.args):
        assert spec["bytes"] == a.nbytes


def test_parse_rejects_malformed_blobs():
    vm = package()
    blob = Golden("golden_layout_kat").blob
    cases = {
        "bad magic": b"XXXX" + blob[4:],
        "unsupported version": blob[:4] + struct.pack("<I", 2) + blob[8:],
        "trailing bytes": blob + b"\0" * 8,
        "truncated": blob[:40],
    }
    for what, bad in cases.items():
        with pytest.raises(vm.InvalidArgument, match=what.split()[0]):
            vm.VmProgram.Parse(bad)
    with pytest.raises(vm.InvalidArgument):
        vm.VmProgram.Parse(b"")


def test_parse_rejects_schedule_errors():
    vm = package()
    from blobs import BARRIER, Builder
    b = Builder(2)
    x = b.buf(8)
    b.outputs, b.out_dims = [x], [[8]]
    t = b.task(0, x, x, x, 18, 8)
    b.ent(0, t, 0, 1)
    b.ent(0, BARRIER)          # lane 1 has no barrier: non-uniform
    b.ent(1, t, 0, 1)
    with pytest.raises(vm.InvalidArgument, match="non-uniform"):
        vm.VmProgram.Parse(b.serialize())
    b = Builder(1)
    x = b.buf(8)
    b.outputs, b.out_dims = [x], [[8]]
    b.task(99, x, x, x)
    with pytest.raises(vm.InvalidArgument, match="unknown tile_op"):
        vm.VmProgram.Parse(b.serialize())
    b = Builder(1)
    x = b.buf(8)
    b.outputs, b.out_dims = [x], [[8]]
    b.task(0, x, 7, x, 0, 8)   # buffer id out of range
    with pytest.raises(vm.InvalidArgument, match="out of range"):
        vm.VmProgram.Parse(b.serialize())
    b = Builder(1)
    b.ent(0, 5, 0, 1)          # entry refers to a task that does not exist
    with pytest.raises(vm.InvalidArgument, match="task index"):
        vm.VmProgram.Parse(b.serialize())


def test_hand_encoded_programs_parse():
    vm = package()
    for name, fn in K.ALL.items():
        blob = fn()[0]
        p = vm.VmProgram.Parse(blob)
        assert p.n_lanes >= 1 and p.n_tasks >= 1, name


def test_runtime_fails_loudly_without_a_device():
    """No CPU fallback: without a B200 the runtime refuses to come up."""
    vm = package()
    try:
        rt = vm.Runtime.Create(0)
    except vm.FailedPrecondition as e:
        assert "CUDA" in str(e) or "sm_" in str(e)
    else:
        rt.close()
        pytest.skip("a CUDA device is present")


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    import importlib
    rt_mod = importlib.import_module("pjrt-ocl_b200.runtime")
    monkeypatch.setattr(rt_mod, "_LIB", None)
    monkeypatch.setenv("B2VM_LIBRARY", str(tmp_path / "nope.so"))
    with pytest.raises(rt_mod.FailedPrecondition, match="no fallback"):
        rt_mod.lib()
    monkeypatch.setattr(rt_mod, "_LIB", None)
