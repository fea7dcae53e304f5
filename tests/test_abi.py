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


def test_byte_layout_golden_parses_field_by_field():
    """The reference's byte-layout known answer (tests/test_lowering.py:109-171):
    b3 = (b0 + b1) - [1, 2, 3] on 8 lanes. The blob the reference serializer wrote
    (fixture) must equal the bytes spelled out here from the format description,
    and the parser must report every count and shape in it."""
    vm = package()
    blob = Golden("golden_layout_kat").blob
    none, barrier = 0xFFFFFFFF, 0xFFFFFFFE
    want = struct.pack("<IIIIIIIIIIQ", 0x314D5056, 3, 4, 2, 1, 2, 2, 1, 0, 0, 256)
    for off in (0, 64, 128, 192):
        want += struct.pack("<QQII", off, 12, 0, 0)
    want += struct.pack("<II", 0, 1) + struct.pack("<I", 3) + b"\0" * 4
    want += struct.pack("<IIQ", 1, 0, 3) * 3
    want += struct.pack("<II", 2, 12) + np.array([1.0, 2.0, 3.0], "<f4").tobytes() + b"\0" * 4
    want += struct.pack("<8I", 1, 3, 0, 1, 3, 0, 0, 0) + struct.pack("<8I", 3, 3, 3, 2, 3, 0, 0, 0)
    assert len(want) == 296 and blob[:296] == want
    n_tasks, n_entries, n_flags, n_lanes = struct.unpack_from("<IIII", blob, 296)
    assert (n_tasks, n_entries, n_flags, n_lanes) == (2, 10, 0, 8)
    assert struct.unpack_from("<12I", blob, 312) == (0, 3, 0, 1, 0, 3, 0, 0, 0, 0, 0, 0)
    ent = 312 + 48 * 2 + 16 * 8
    assert struct.unpack_from("<8I", blob, ent) == (0, 0, 1, none, 0, none, 0, 0)
    assert struct.unpack_from("<8I", blob, ent + 32) == (barrier, 0, 0, none, 0, none, 0, 0)
    assert len(blob) == ent + 32 * 10
    p = vm.VmProgram.Parse(blob)
    assert (p.n_inputs, p.n_outputs, p.n_lanes, p.n_tasks, p.arena_bytes) == (2, 1, 8, 2, 256)
    for spec in p.inputs + p.outputs:
        assert spec["bytes"] == 12 and spec["shape"] == (3,) and spec["dtype"] == np.dtype("<f4")
    # a buffer that is not on a multiple of its element size is refused on the host
    bad = bytearray(blob)
    struct.pack_into("<QQII", bad, 48 + 24, 68, 8, 4, 0)        # buffer 1: i64 at offset 68
    with pytest.raises(vm.InvalidArgument, match="misaligned"):
        vm.VmProgram.Parse(bytes(bad))


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
