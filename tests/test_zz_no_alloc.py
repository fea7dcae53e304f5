"""The allocation-free full sum (`b2_sum_f32_static`, include/b2vm.h).

Some hosts cannot allocate device memory when they call this library: a serving
process whose own allocator took all of HBM at start-up (a later cudaMalloc, and
with it a program load, fails there), or a latency path that must not take the
device-wide stall of cudaMalloc / cudaFree. For them the library carries the
reduction's scratch inside its own image. This test calls that entry point
through the C ABI twice in a row, on different sizes and data, and compares each
result with what the ordinary path (a RED_PART + RED_COMB program through
`b2_execute_device`) gives for the same input, at the f32 tolerance the other
parity tests use (rel 1e-5). The second call is the smaller one: stale partial
sums of the first call are still in the shared scratch then and must not leak
into the result.

This file sorts last on purpose, so a run that stops at the first failure has
already run every other test.
"""
import numpy as np
import pytest

from blobs import Builder
from conftest import package

pytestmark = pytest.mark.gpu

RED_PART, RED_COMB, SUM = 3, 4, 0
CHUNK = 131072


def _full_sum_program(n: int, lanes: int) -> bytes:
    """partials[t] = sum(x[t*CHUNK : (t+1)*CHUNK]); barrier; out = sum(partials)."""
    parts = -(-n // CHUNK)
    b = Builder(lanes)
    x, partial, out = b.buf(n), b.buf(parts), b.buf(1)
    b.inputs, b.outputs = [x], [out]
    b.in_dims, b.out_dims = [[n]], [[]]
    t_part = b.task(RED_PART, partial, x, x, n, CHUNK, SUM)
    t_comb = b.task(RED_COMB, out, partial, partial, parts, SUM)
    for lane in range(lanes):
        lo, hi = parts * lane // lanes, parts * (lane + 1) // lanes
        if hi > lo:
            b.ent(lane, t_part, lo, hi)
    b.barrier_all()
    b.ent(0, t_comb, 0, 1)
    return b.serialize()


def _both_ways(vm, rt, x: np.ndarray):
    n = x.size
    d_in = rt.AllocDevice(n * 4)
    d_out = rt.AllocDevice(4)
    try:
        rt.WriteToDevice(d_in, x)
        rt.WriteToDevice(d_out, np.array([np.nan], np.float32))
        rt.SumF32Static(d_in, n, d_out)
        got = rt.ReadFromDevice(d_out, 4).view(np.float32)[0]
        lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(_full_sum_program(n, 8)))
        (d_ref,) = lp.ExecuteDevice([d_in])
        want = rt.ReadFromDevice(d_ref, 4).view(np.float32)[0]
        rt.PoolFree(d_ref, 4)
        lp.close()
    finally:
        rt.PoolFree(d_in, n * 4)
        rt.PoolFree(d_out, 4)
    return got, want


def test_static_scratch_sum_matches_the_program_path_on_two_calls_in_a_row():
    vm = package()
    rt = vm.Runtime.Create(0)
    try:
        rng = np.random.default_rng(7)
        # 23 chunks with a ragged tail, then 3 chunks: the second call leaves 20 stale partials behind it
        for n, shift in ((22 * CHUNK + 70_001, 0.25), (2 * CHUNK + 5, -0.5)):
            x = (rng.standard_normal(n) + shift).astype(np.float32)
            got, want = _both_ways(vm, rt, x)
            exact = float(np.sum(x, dtype=np.float64))
            scale = float(np.sum(np.abs(x), dtype=np.float64))
            assert np.isfinite(got)
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5 * scale / n ** 0.5)
            np.testing.assert_allclose(got, exact, rtol=1e-5, atol=1e-5 * scale / n ** 0.5)
    finally:
        rt.close()


def test_static_scratch_sum_rejects_sizes_beyond_its_scratch():
    vm = package()
    rt = vm.Runtime.Create(0)
    try:
        limit = vm.lib().b2_sum_f32_static_max_elems()
        assert limit == 4096 * CHUNK
        d = rt.AllocDevice(16)
        with pytest.raises(vm.InvalidArgument, match="exceed"):
            rt.SumF32Static(d, limit + 1, d)      # refused before anything is read
        rt.PoolFree(d, 16)
    finally:
        rt.close()
