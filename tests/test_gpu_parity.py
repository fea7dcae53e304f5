"""Parity of the CUDA backend, through the C ABI, against (a) the golden
fixtures produced by the reference's two validators and (b) the C oracle on the
same seeded inputs. Integer / bool / index outputs bit-exact; f32 within rel 1e-5
class tolerances, bf16 / f16 within rel 2e-2 (exact numbers per fixture)."""
import numpy as np
import pytest

from conftest import Golden, check_outputs, golden_names, package

import kat_programs as K
import vmoracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    vm = package()
    r = vm.Runtime.Create(0)
    yield r
    r.close()


def _raw(arrs):
    return [np.ascontiguousarray(a).view(np.uint8).reshape(-1) for a in arrs]


@pytest.mark.parametrize("name", golden_names())
def test_execute_matches_reference_validators(rt, name):
    vm = package()
    g = Golden(name)
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
    out = lp.Execute(g.args)
    check_outputs(g, _raw(out), "cuda")
    st = lp.Status()
    assert st["code"] == 0 and lp.launch_count == 1
    # twice in a row: the arena keeps the previous run's contents
    out2 = lp.Execute(g.args)
    for a, b in zip(_raw(out), _raw(out2)):
        np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("name", ["c2_int_chain_small", "c2_chain_f32_small", "c3_mlp_bf16_small",
                                  "c4_nbody_small", "c5_block_bf16_small", "dynslice",
                                  "while_loop_data_dependent", "c5_decode_in_place_bf16_small"])
def test_execute_device_matches_oracle(rt, name):
    """ExecuteDevice (device pointers in, pooled device buffers out) against the
    C oracle run on the same inputs."""
    vm = package()
    g = Golden(name)
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
    dins = []
    for a in g.args:
        a = np.ascontiguousarray(a)
        p = rt.AllocDevice(max(a.nbytes, 16))
        rt.WriteToDevice(p, a)
        dins.append((p, max(a.nbytes, 16)))
    douts = lp.ExecuteDevice([p for p, _ in dins])
    got = [rt.ReadFromDevice(p, s["bytes"]) for p, s in zip(douts, lp.prog.outputs)]
    for p, s in zip(douts, lp.prog.outputs):
        rt.PoolFree(p, s["bytes"])
    for p, n in dins:
        rt.PoolFree(p, n)
    check_outputs(g, got, "cuda-device")
    want = vmoracle.Program(g.blob).execute(g.args)
    for i, (a, b, e) in enumerate(zip(got, want, g.expected)):
        if g.meta.get("exact") or e.dtype.kind in "iub":
            np.testing.assert_array_equal(a, b, err_msg=f"{name} out {i} vs oracle")


@pytest.mark.parametrize("name", ["c5_decode_in_place_f32_small", "c5_decode_in_place_bf16_small"])
def test_in_out_buffers_are_updated_in_place(rt, name):
    """A KV cache that is argument and result of the program: with the same device address
    passed for both nothing is copied and the cache is updated where it lies; two steps in
    a row give the same answer (the step overwrites one position with the same values)."""
    vm = package()
    g = Golden(name)
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
    pairs = lp.InOutResults()
    assert pairs == {2: 1, 3: 2} and lp.stat("in_out_ports") == 2
    if name.endswith("bf16_small"):
        assert lp.stat("decode_flash") == 1
    dins = []
    for a in g.args:
        a = np.ascontiguousarray(a)
        p = rt.AllocDevice(max(a.nbytes, 16))
        rt.WriteToDevice(p, a)
        dins.append((p, max(a.nbytes, 16)))
    douts = []
    for o, s in enumerate(lp.prog.outputs):
        src = [i for i, r in pairs.items() if r == o]
        douts.append(dins[src[0]][0] if src else rt.AllocDevice(max(s["bytes"], 16)))
    for _ in range(2):
        lp.ExecuteDeviceAsync([p for p, _ in dins], douts)
        assert lp.Status()["code"] == 0
    got = [rt.ReadFromDevice(p, s["bytes"]) for p, s in zip(douts, lp.prog.outputs)]
    check_outputs(g, got, "cuda-in-place")
    # the cache argument itself now holds the updated cache
    np.testing.assert_array_equal(rt.ReadFromDevice(dins[2][0], lp.prog.outputs[1]["bytes"]), got[1])
    for o, (p, s) in enumerate(zip(douts, lp.prog.outputs)):
        if o not in pairs.values():
            rt.PoolFree(p, max(s["bytes"], 16))
    for p, n in dins:
        rt.PoolFree(p, n)


def test_phases_mixing_unit_costs_are_recut_over_all_lanes(rt):
    """Config 3's backward phases hold matmuls of different depth, regions and casts side by
    side; the scheduler's cost per tile is one constant per op class, so the loader re-cuts
    such phases evenly over all lanes. Values are those of the scheduler's own cut."""
    vm = package()
    g = Golden("c3_mlp_bf16_small")
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
    assert lp.stat("rebalanced_phases") >= 1
    check_outputs(g, [np.ascontiguousarray(o).view(np.uint8).reshape(-1) for o in lp.Execute(g.args)], "cuda-recut")
    # a phase of equal units keeps the scheduler's cut
    g2 = Golden("c2_chain_f32_small")
    assert vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g2.blob)).stat("rebalanced_phases") == 0


def test_row_local_phases_run_as_one_pipeline(rt, monkeypatch):
    """LayerNorm rows -> elementwise chain -> softmax rows over the same rows of one elementwise tile each:
    the loader removes the two grid barriers between them (every row depends only on the same row of its
    predecessor); with a block size the lane also interleaves the three units block by block. Same values."""
    vm = package()
    g = Golden("c2_chain_f32_small")
    for block in (None, "2"):
        if block:
            monkeypatch.setenv("B2VM_ROW_BLOCK", block)
        lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
        assert lp.stat("row_pipelines") == 1
        check_outputs(g, [np.ascontiguousarray(o).view(np.uint8).reshape(-1) for o in lp.Execute(g.args)], "cuda-rows")
        # 4 phases -> one: the pipeline, whose softmax also carries the sum (so the barrier before the sum goes too)
        assert lp.stat("carried_sums") == 1 and lp.stat("carried_barriers_removed") == 1
        assert lp.Status()["barriers"] == 1


def test_convert_feeding_a_full_sum_is_folded(rt, monkeypatch):
    """A full f32 sum over the f32 copy of a bf16 / f16 buffer reads the 16-bit source itself when nothing else
    wants the copy (two of the fixture's three sums; the third copy is also a program output and stays). Same
    values either way: convert to f32 per element, accumulate in f32 (vmreader.py convert + reduce)."""
    vm = package()
    g = Golden("reduce_full_16bit_source")
    for off, want in ((None, 2), ("1", 0)):
        with monkeypatch.context() as m:
            if off:
                m.setenv("B2VM_NO_CONVERT_FOLD", off)
            lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
            assert lp.stat("folded_converts") == want
            check_outputs(g, [np.ascontiguousarray(o).view(np.uint8).reshape(-1) for o in lp.Execute(g.args)], "cuda-fold")


@pytest.mark.parametrize("name,folds", [("rows_then_full_sum_f32", 0), ("rows_then_full_sum_bf16", 1), ("rows_then_full_sum_ragged", 0)])
def test_full_sum_carried_by_the_row_op(rt, monkeypatch, name, folds):
    """A full sum over what one softmax / layer-norm task wrote is taken from that task (each lane adds what it
    stores to its carry word) instead of streaming the rows again: same total as the streamed sum to f32
    summation-order accuracy, on the staged f32 and bf16 paths and on the short-row path, and again on a second
    execute (the carry words return to zero)."""
    vm = package()
    g = Golden(name)
    totals = {}
    for off in (None, "1"):
        with monkeypatch.context() as m:
            if off:
                m.setenv("B2VM_NO_CARRIED_SUM", off)
            lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
            assert lp.stat("carried_sums") == (0 if off else 1)
            assert lp.stat("carried_barriers_removed") == (0 if off else 1 + folds)   # the folded convert's empty phase goes too
            assert lp.stat("folded_converts") == folds
            first = lp.Execute(g.args)
            check_outputs(g, [np.ascontiguousarray(o).view(np.uint8).reshape(-1) for o in first], "cuda-carried")
            second = lp.Execute(g.args)
            totals[off] = [float(np.asarray(o[-1]).reshape(-1)[0]) for o in (first, second)]
    assert totals[None][0] == totals[None][1]
    np.testing.assert_allclose(totals[None][0], totals["1"][0], rtol=1e-5)


def test_decomposed_rms_norm_runs_as_one_row_op(rt, monkeypatch):
    """The block's RMS norm arrives as seven tile ops in five phases (convert, square, RED_SEG, a region on the row
    sums, two multiplies through broadcast views, convert); the loader runs it as one row op on the last
    convert's entries and drops the phases that empty. Same values as the separate ops, rows of 1024 and 256."""
    vm = package()
    g = Golden("rmsnorm_rows_bf16")
    barriers = {}
    for off, want in ((None, 2), ("1", 0)):
        with monkeypatch.context() as m:
            if off:
                m.setenv("B2VM_NO_RMS_FUSION", off)
            lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(g.blob))
            assert lp.stat("rms_rows") == want
            check_outputs(g, [np.ascontiguousarray(o).view(np.uint8).reshape(-1) for o in lp.Execute(g.args)], "cuda-rms")
            barriers[off] = (lp.Status()["barriers"], lp.stat("empty_phases_dropped"))
    assert barriers["1"][1] == 0 and barriers[None][1] > 0
    assert barriers[None][0] + barriers[None][1] == barriers["1"][0]


def test_point_to_point_entry_fields_are_refused(rt):
    """Tile entries whose reserved wait / signal words are set (scheduler.py:201-209 keeps them
    for point-to-point dependencies and emits "no flag") are refused at load, not ignored."""
    from blobs import Builder
    vm = package()
    b = Builder(2)
    ba, bb, bc = (b.buf(2 * 4096) for _ in range(3))
    b.inputs, b.outputs = [ba, bb], [bc]
    b.in_dims, b.out_dims = [[2 * 4096], [2 * 4096]], [[2 * 4096]]
    t0 = b.task(0, bc, ba, bb, 0, 2 * 4096)
    b.ent(0, t0, 0, 1, 3, 1)             # waits once on flag 3
    b.ent(1, t0, 1, 2)
    b.barrier_all()
    with pytest.raises(vm.Unimplemented, match="point-to-point"):
        vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(b.serialize()))


def test_operand_view_outside_its_buffer_is_refused(rt):
    """A view whose largest index lies beyond its buffer is a malformed program: refused on
    the host at load (INVALID_ARGUMENT), never run."""
    from blobs import Builder
    vm = package()
    n = 4096
    b = Builder(1)
    ba, bb, bc = (b.buf(n) for _ in range(3))
    b.inputs, b.outputs = [ba, bb], [bc]
    b.in_dims, b.out_dims = [[n], [n]], [[n]]
    b.aux = [0, 1, n, 2, 0]              # word 1..: rank 1, dims [n], strides [2], offset 0 -> indices up to 2n - 2
    t0 = b.task(0, bc, ba, bb, 0, n, 2)  # add, operand a through the view at aux[1]
    b.ent(0, t0, 0, 1)
    b.barrier_all()
    with pytest.raises(vm.InvalidArgument, match="outside buffer"):
        vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(b.serialize()))


@pytest.mark.parametrize("name", sorted(K.ALL))
def test_known_answer_programs(rt, name):
    vm = package()
    blob, args, expected = K.ALL[name]()
    out = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(blob)).Execute(args)
    for o, e in zip(out, expected):
        e = np.asarray(e)
        if name == "C_region_gelu":
            np.testing.assert_allclose(o.reshape(e.shape), e, rtol=1e-5, atol=1e-5)
        else:
            np.testing.assert_array_equal(o.reshape(e.shape), e)


@pytest.mark.parametrize("flag", [1.0, 0.0])
def test_for_zero_trip_and_if(rt, flag):
    vm = package()
    blob, x, expected = K.kat_for_zero_trip_and_if()
    out = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(blob)).Execute([x, np.float32(flag)])
    for o, e in zip(out, expected[flag]):
        np.testing.assert_array_equal(o.reshape(e.shape), e)


@pytest.mark.parametrize("flag", [1.0, 0.0])
def test_strided_reduce_spread_over_lanes_in_control_ranges(rt, flag):
    """The loader re-cuts both reductions by rows over the four lanes (inserting entries
    into FOR-body and IF-branch ranges); results equal the oracle's known answer."""
    vm = package()
    blob, (x, z0), expected = K.kat_strided_reduce_in_control_ranges()
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(blob))
    assert lp.stat("spread_reductions") == 2
    out = lp.Execute([x, np.float32(flag), z0])
    for o, e in zip(out, expected[flag]):
        np.testing.assert_array_equal(np.asarray(o).view(np.float32).reshape(e.shape), e)


def test_full_reductions_are_recut_over_all_lanes(rt):
    """RED_PART + RED_COMB pairs whose partials nothing else reads run as one phase:
    every lane reduces an equal share and the last lane to arrive stores the result."""
    vm = package()
    blob, args, expected = K.kat_full_reduce_recut()
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(blob))
    assert lp.stat("fused_full_reductions") == 3
    for _ in range(2):                     # twice: the arrival counter is back at rest after a run
        out = lp.Execute(args)
        np.testing.assert_array_equal(out[0], expected[0])
        np.testing.assert_array_equal(out[1], expected[1])
        np.testing.assert_array_equal(out[2], expected[2])
        args[3] = np.uint32(out[2])
        expected[2] = np.uint32((int(out[2]) + 3 * int(np.bitwise_xor.reduce(args[2]))) % 2 ** 32)


@pytest.mark.parametrize("name,build", [("c2_chain_f32_small", "stream"), ("c4_nbody_small", "shortrun"),
                                         ("dot_tc_bf16", "matmul"), ("flash_tc_bf16", "attn"),
                                         ("reduce_window_f32", "all")])
def test_program_runs_on_the_smallest_kernel_build_that_has_its_families(rt, name, build):
    vm = package()
    from conftest import Golden
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(Golden(name).blob))
    assert ["stream", "shortrun", "matmul", "attn", "all"][lp.stat("kernel_build")] == build


def test_config4_reductions_are_spread_over_lanes(rt):
    vm = package()
    from conftest import Golden
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(Golden("c4_nbody_mid").blob))
    assert lp.stat("spread_reductions") == 4      # one axis-1 sum per acceleration evaluation


def test_lanes_beyond_residency_are_refused_at_load(rt):
    vm = package()
    from blobs import Builder
    b = Builder(min(4096, rt.lanes + 1))
    x = b.buf(8)
    b.outputs, b.out_dims = [x], [[8]]
    t = b.task(0, x, x, x, 18, 8)
    b.ent(0, t, 0, 1)
    with pytest.raises(vm.FailedPrecondition, match="co-resident"):
        vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(b.serialize()))


def test_bounded_barrier_wait_reports_deadline_and_context_survives(rt):
    """A wait that nothing will ever satisfy runs out after its budget: the
    kernel returns normally with a status, the host reports DEADLINE_EXCEEDED,
    and the same runtime keeps working. (Lane 0's FOR body holds one more grid
    barrier than lane 1's, so lane 0 waits for an arrival that never comes.)"""
    vm = package()
    from blobs import BARRIER, FOR, NOP, Builder
    b = Builder(2)
    x = b.buf(8)
    b.outputs, b.out_dims = [x], [[8]]
    t = b.task(0, x, x, x, 18, 8, 0x3F800000)
    # both streams hold one BARRIER entry (the parser wants equal counts), but
    # lane 1's lies outside its FOR body and outside the root walk: never reached.
    b.ent(0, FOR, 1, 2, 1); b.ent(0, t, 0, 1); b.ent(0, BARRIER)
    b.ent(1, FOR, 1, 1, 1); b.ent(1, NOP); b.ent(1, BARRIER)
    b.root_lens = [1, 1]
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(b.serialize()))
    lp.set_wait_budget_ns(50_000_000)
    with pytest.raises(vm.DeadlineExceeded, match="grid barrier"):
        lp.Execute([])
    blob, args, expected = K.kat_a_two_level()
    out = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(blob)).Execute(args)
    np.testing.assert_array_equal(out[0], expected[0])
