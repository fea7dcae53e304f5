"""Known-answer programs hand-encoded at the schedule level, mirroring the
reference's device test (pjrt_plugin/src/runtime_test.cc): A two-level
elementwise on 4 lanes (:136-170), B on-device WHILE on 2 lanes (:172-215), C a
GELU map-region (:217-267, descriptor in the layout of ops/region.py:19-23), the
hand-built WHILE known answer of tests/test_lowering.py:405-439 restated as a
schedule (counter -> 5, data -> iota * 32, using LTS and IOTA_FLAT), integer
division by zero -> 0 (ew.cl:410), FOR with trip count 0, and a nested IF.
Each returns (blob, inputs, expected outputs as numpy arrays).
"""
import struct

import numpy as np

from blobs import BARRIER, FOR, IF, NOP, WHILE, Builder

EW, REGION = 0, 13
EW_TS = 4096


def fbits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def kat_a_two_level():
    lanes, n = 4, 4 * EW_TS
    b = Builder(lanes)
    ba, bb, bt, bc = (b.buf(n) for _ in range(4))
    b.inputs, b.outputs = [ba, bb], [bc]
    b.in_dims, b.out_dims = [[n], [n]], [[n]]
    t0 = b.task(EW, bt, ba, bb, 0, n)
    t1 = b.task(EW, bc, bt, ba, 1, n)
    for l in range(lanes):
        b.ent(l, t0, l, l + 1)
    b.barrier_all()
    for l in range(lanes):
        b.ent(l, t1, l, l + 1)
    b.barrier_all()
    i = np.arange(n)
    a = (i % 251).astype(np.float32)
    bv = ((i % 83) + 1).astype(np.float32)
    return b.serialize(), [a, bv], [(a + bv) * a]


def kat_b_while():
    lanes, n = 2, 2 * EW_TS
    b = Builder(lanes)
    bx, bi, bk, bone, bcond = b.buf(n), b.buf(1), b.buf(1), b.buf(1), b.buf(1)
    b.inputs, b.outputs = [bx], [bx]
    b.in_dims, b.out_dims = [[n]], [[n]]
    b.consts = [(bi, struct.pack("<f", 0.0)), (bk, struct.pack("<f", 10.0)), (bone, struct.pack("<f", 1.0))]
    tdbl = b.task(EW, bx, bx, bx, 0, n)
    tinc = b.task(EW, bi, bi, bone, 0, 1)
    tlts = b.task(EW, bcond, bi, bk, 22, 1)
    for lane in range(2):
        b.ent(lane, WHILE, 1, 1, 2, 2, bcond)
    b.ent(0, tlts, 0, 1); b.ent(0, tdbl, 0, 1); b.ent(0, tinc, 0, 1)
    b.ent(1, NOP); b.ent(1, tdbl, 1, 2); b.ent(1, NOP)
    b.root_lens = [1, 1]
    x = ((np.arange(n) % 13) + 1).astype(np.float32)
    return b.serialize(), [x], [x * np.float32(1024.0)]


def kat_c_region_gelu():
    lanes, n = 8, 8 * EW_TS
    b = Builder(lanes)
    bx, by = b.buf(n), b.buf(n)
    b.inputs, b.outputs = [bx], [by]
    b.in_dims, b.out_dims = [[n]], [[n]]
    MUL, ADD, TANH, AFF = 1, 0, 13, 40
    micro = [
        (MUL, 1, 0, 0, 0, 0), (MUL, 1, 1, 0, 0, 0), (AFF, 1, 1, 0, fbits(0.044715), fbits(0.0)),
        (ADD, 1, 1, 0, 0, 0), (AFF, 1, 1, 0, fbits(0.7978845608), fbits(0.0)), (TANH, 1, 1, 0, 0, 0),
        (AFF, 1, 1, 0, fbits(0.5), fbits(0.5)), (MUL, 0, 0, 1, 0, 0)]
    b.aux = [1, 0, len(micro), 0] + [w for m in micro for w in m]
    t = b.task(REGION, by, bx, bx, 0, n, bx, bx, bx, bx, bx, bx)
    for l in range(lanes):
        b.ent(l, t, l, l + 1)
    x = (-4.0 + 8.0 * (np.arange(n) % 101) / 100.0).astype(np.float32)
    g = (0.5 * x.astype(np.float64) * (1.0 + np.tanh(0.7978845608 * (x + 0.044715 * x.astype(np.float64) ** 3))))
    return b.serialize(), [x], [g.astype(np.float32)]


def kat_while_counter():
    """counter = 0; data = iota(8); while (counter < 5) { counter += 1; data += data }"""
    b = Builder(2)
    bc, blim, bone, bcond, bdata = b.buf(1), b.buf(1), b.buf(1), b.buf(1), b.buf(8)
    b.outputs, b.out_dims = [bc, bdata], [[], [8]]
    b.consts = [(blim, struct.pack("<f", 5.0)), (bone, struct.pack("<f", 1.0))]
    tfill = b.task(EW, bc, bc, bc, 18, 1, fbits(0.0))
    tiota = b.task(EW, bdata, bdata, bdata, 19, 8)
    tlts = b.task(EW, bcond, bc, blim, 22, 1)
    tinc = b.task(EW, bc, bc, bone, 0, 1)
    tdbl = b.task(EW, bdata, bdata, bdata, 0, 8)
    # root: fill | iota, barrier, WHILE ; cond at [3,4), body at [4,5)
    b.ent(0, tfill, 0, 1); b.ent(1, tiota, 0, 1)
    b.barrier_all()
    for lane in range(2):
        b.ent(lane, WHILE, 3, 1, 4, 1, bcond)
    b.ent(0, tlts, 0, 1); b.ent(1, NOP)
    b.ent(0, tinc, 0, 1); b.ent(1, tdbl, 0, 1)
    b.root_lens = [3, 3]
    return b.serialize(), [], [np.float32(5.0), np.arange(8, dtype=np.float32) * np.float32(32.0)]


def kat_int_div_zero():
    n = 1000
    b = Builder(1)
    bx, by, bz = b.buf(n, 1), b.buf(n, 1), b.buf(n, 1)
    b.inputs, b.outputs = [bx, by], [bz]
    b.in_dims, b.out_dims = [[n], [n]], [[n]]
    t = b.task(EW, bz, bx, by, 3, n, dtype=1, adtype=1)
    b.ent(0, t, 0, 1)
    x = (np.arange(n, dtype=np.int32) - 500) * 7
    y = (np.arange(n, dtype=np.int32) % 5) - 2
    exp = np.where(y != 0, (x.astype(np.float64) / np.where(y == 0, 1, y)).astype(np.int64), 0).astype(np.int32)
    exp = np.where(y != 0, np.trunc(x / np.where(y == 0, 1, y)).astype(np.int32), 0).astype(np.int32)
    return b.serialize(), [x, y], [exp]


def kat_for_zero_trip_and_if():
    """x2 = x + x once (FOR trip 3 doubles x three times, FOR trip 0 is skipped);
    IF(flag) picks `y = x * x` else `y = x - x`; both branches scheduled."""
    n = 2 * EW_TS
    b = Builder(2)
    bx, by, bflag = b.buf(n), b.buf(n), b.buf(1)
    b.inputs, b.outputs = [bx, bflag], [bx, by]
    b.in_dims, b.out_dims = [[n], []], [[n], [n]]
    tdbl = b.task(EW, bx, bx, bx, 0, n)
    tmul = b.task(EW, by, bx, bx, 1, n)
    tsub = b.task(EW, by, bx, bx, 2, n)
    for lane in range(2):
        b.ent(lane, FOR, 4, 1, 3)           # body [4,5), trip 3
        b.ent(lane, FOR, 4, 1, 0)           # trip 0: skipped
        b.ent(lane, BARRIER)
        b.ent(lane, IF, 5, 1, 6, 1, bflag)  # then [5,6), else [6,7)
        b.ent(lane, tdbl, lane, lane + 1)
        b.ent(lane, tmul, lane, lane + 1)
        b.ent(lane, tsub, lane, lane + 1)
    b.root_lens = [4, 4]
    x = ((np.arange(n) % 7) + 1).astype(np.float32)
    out = {}
    for flag in (1.0, 0.0):
        x8 = x * np.float32(8.0)
        out[flag] = [x8, x8 * x8 if flag else x8 - x8]
    return b.serialize(), x, out


def kat_strided_reduce_in_control_ranges():
    """An interior-axis reduction owned by one lane inside a FOR body and inside an IF
    branch, with the other lanes' runs empty at a range start, empty at a range end, or
    holding NOPs: the layout a loader that re-cuts the reduction over all lanes has to
    re-index. z accumulates y = sum_r x[row, r, c] twice; w = y (summed again) if flag else y - y.
    Integer-valued inputs, so every summation order gives the same f32."""
    rows, red, inner = 8, 128, 3
    n_out = rows * inner
    b = Builder(4)
    bx, bflag, bz, by, bw = b.buf(rows * red * inner), b.buf(1), b.buf(n_out), b.buf(n_out), b.buf(n_out)
    b.inputs, b.outputs = [bx, bflag, bz], [bz, bw]
    b.in_dims, b.out_dims = [[rows, red, inner], [], [rows, inner]], [[rows, inner], [rows, inner]]
    RED_STRIDED = 15
    tsum = b.task(RED_STRIDED, by, bx, bx, n_out, red, inner, 0)
    tmax = b.task(RED_STRIDED, bw, bx, bx, n_out, red, inner, 0)       # the same sums again, into w
    tacc = b.task(EW, bz, bz, by, 0, n_out)
    tzero = b.task(EW, bw, by, by, 2, n_out)
    # lane 0: owner of both reductions
    b.ent(0, FOR, 3, 3, 2); b.ent(0, BARRIER); b.ent(0, IF, 6, 1, 7, 1, bflag)
    b.ent(0, tsum, 0, 1); b.ent(0, BARRIER); b.ent(0, NOP)
    b.ent(0, tmax, 0, 1)
    b.ent(0, tzero, 0, 1)
    # lane 1: the body starts with its barrier (an empty run at the range start), then accumulates
    b.ent(1, FOR, 3, 2, 2); b.ent(1, BARRIER); b.ent(1, IF, 5, 1, 6, 1, bflag)
    b.ent(1, BARRIER); b.ent(1, tacc, 0, 1)
    b.ent(1, NOP)
    b.ent(1, NOP)
    # lane 2: NOPs everywhere
    b.ent(2, FOR, 3, 3, 2); b.ent(2, BARRIER); b.ent(2, IF, 6, 1, 7, 1, bflag)
    b.ent(2, NOP); b.ent(2, BARRIER); b.ent(2, NOP)
    b.ent(2, NOP)
    b.ent(2, NOP)
    # lane 3: the body is the barrier alone (empty runs at both ends of the range)
    b.ent(3, FOR, 3, 1, 2); b.ent(3, BARRIER); b.ent(3, IF, 4, 1, 5, 1, bflag)
    b.ent(3, BARRIER)
    b.ent(3, NOP)
    b.ent(3, NOP)
    b.root_lens = [3, 3, 3, 3]
    rng = np.random.default_rng(7)
    x = rng.integers(-8, 9, size=(rows, red, inner)).astype(np.float32)
    z0 = rng.integers(-4, 5, size=(rows, inner)).astype(np.float32)
    y = x.sum(axis=1)
    out = {1.0: [z0 + 2 * y, y], 0.0: [z0 + 2 * y, np.zeros_like(y)]}
    return b.serialize(), [x, z0], out


def kat_full_reduce_recut():
    """Three full reductions (RED_PART + RED_COMB) a loader can re-cut over all lanes:
    an i32 sum with a ragged tail (70003 elements, wraps exactly), an f32 max, and a u32
    xor inside a FOR body of 3 trips whose result is accumulated each trip - the lanes'
    arrival counter must return to rest between the trips."""
    RED_PART, RED_COMB = 3, 4
    n, chunk, lanes = 70003, 16384, 4
    parts = -(-n // chunk)
    b = Builder(lanes)
    bi, bf, bu = b.buf(n, 1), b.buf(n, 0), b.buf(n, 2)
    pi, pf, pu = b.buf(parts, 1), b.buf(parts, 0), b.buf(parts, 2)
    oi, of, ou, acc = b.buf(1, 1), b.buf(1, 0), b.buf(1, 2), b.buf(1, 2)
    b.inputs, b.outputs = [bi, bf, bu, acc], [oi, of, acc]
    b.in_dims, b.out_dims = [[n], [n], [n], []], [[], [], []]
    t_pi = b.task(RED_PART, pi, bi, bi, n, chunk, 0, dtype=1, adtype=1)
    t_ci = b.task(RED_COMB, oi, pi, pi, parts, 0, dtype=1, adtype=1)
    t_pf = b.task(RED_PART, pf, bf, bf, n, chunk, 1)
    t_cf = b.task(RED_COMB, of, pf, pf, parts, 1)
    t_pu = b.task(RED_PART, pu, bu, bu, n, chunk, 6, dtype=2, adtype=2)
    t_cu = b.task(RED_COMB, ou, pu, pu, parts, 6, dtype=2, adtype=2)
    t_acc = b.task(EW, acc, acc, ou, 0, 1, dtype=2, adtype=2)          # acc += xor(bu)
    split = [(parts * l // lanes, parts * (l + 1) // lanes) for l in range(lanes)]
    # root: i32 parts | barrier | i32 comb + f32 parts | barrier | f32 comb | barrier | FOR 3 x {parts | comb | acc}
    for l, (lo, hi) in enumerate(split):
        b.ent(l, t_pi, lo, hi)
        b.ent(l, BARRIER)
        if l == 0:
            b.ent(l, t_ci, 0, 1)
        else:
            b.ent(l, NOP)
        b.ent(l, BARRIER)
        b.ent(l, t_pf, lo, hi)
        b.ent(l, BARRIER)
        b.ent(l, t_cf, 0, 1) if l == 1 else b.ent(l, NOP)
        b.ent(l, BARRIER)
        b.ent(l, FOR, 9, 5, 3)                      # entry 8: body [9, 14)
        b.ent(l, t_pu, lo, hi)                      # 9
        b.ent(l, BARRIER)                           # 10
        b.ent(l, t_cu, 0, 1) if l == 2 else b.ent(l, NOP)   # 11
        b.ent(l, BARRIER)                           # 12
        b.ent(l, t_acc, 0, 1) if l == 2 else b.ent(l, NOP)  # 13
    b.root_lens = [9] * lanes
    rng = np.random.default_rng(11)
    xi = rng.integers(-2 ** 31, 2 ** 31, size=n, dtype=np.int64).astype(np.int32)
    xf = rng.standard_normal(n).astype(np.float32)
    xu = rng.integers(0, 2 ** 32, size=n, dtype=np.int64).astype(np.uint32)
    a0 = np.uint32(12345)
    want_i = np.int32((int(np.sum(xi.astype(np.int64))) + 2 ** 31) % 2 ** 32 - 2 ** 31)   # two's-complement wrap
    want_u = np.uint32((int(a0) + 3 * int(np.bitwise_xor.reduce(xu))) % 2 ** 32)
    return b.serialize(), [xi, xf, xu, a0], [want_i, np.max(xf), want_u]


ALL = {
    "A_two_level": kat_a_two_level, "B_while": kat_b_while, "C_region_gelu": kat_c_region_gelu,
    "while_counter": kat_while_counter, "int_div_zero": kat_int_div_zero,
    "full_reduce_recut": kat_full_reduce_recut,
}
