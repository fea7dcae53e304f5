#!/usr/bin/env python
"""Generate the golden fixtures under tests/golden/*.npz.

Runs only where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 PYTHONPATH=<reference>/python \
        python tests/golden/make_golden.py [case-name-substring ...]

For every case it assembles a VMProgram v3 blob through the reference's own
lowering context, pass pipeline, scheduler and serializer (see
pjrt-ocl_b200/programs/vmasm.py), executes it with BOTH reference validators
(`vmreader.execute`, the tensor interpreter that is the semantic source of
truth, vmreader.py:389-470, and `vmreader.execute_schedule`, the lane
simulator, vmreader.py:529-652), requires them to agree bit-for-bit, and
stores: the blob, the seeded input description, and the validator outputs.

The tests then replay the blob on (a) the C oracle and (b) the CUDA backend
and compare against the stored outputs.
"""
from __future__ import annotations

import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "pjrt-ocl_b200", "programs"))

import numpy as np  # noqa: E402

import cases  # noqa: E402
import inputs as gen_inputs  # noqa: E402
from vmasm import (Asm, BF16, BOOL, F16, F32, I32, I64, MAX, MIN, PROD, SUM,  # noqa: E402
                   U32, L)
from pjrt_ocl import vmreader as R  # noqa: E402
from pjrt_ocl.ops import reduce as RED  # noqa: E402

DN = cases.DN
CASES = {}


def case(name, **meta):
    def deco(fn):
        CASES[name] = (fn, meta)
        return fn
    return deco


def N(shape, dt="f32", scale=1.0, shift=0.0):
    return ("normal", tuple(shape), dt, scale, shift)


def U(shape, lo, hi, dt="f32"):
    return ("uniform", tuple(shape), dt, lo, hi)


def I(shape, lo, hi, dt="i32"):
    return ("int", tuple(shape), dt, lo, hi)


RAG = 4096 * 2 + 77          # two full EW tiles + a ragged tail


# ---------------------------------------------------------------- elementwise
_BIN_F = [L.OP_ADD_F32, L.OP_MUL_F32, L.OP_SUB_F32, L.OP_DIV_F32, L.OP_MAX_F32,
          L.OP_MIN_F32, L.OP_ATAN2_F32, L.OP_REMAINDER_F32]
_UN_F = [L.OP_NEG_F32, L.OP_EXP_F32, L.OP_TANH_F32, L.OP_ABS_F32, L.OP_FLOOR_F32,
         L.OP_CEIL_F32, L.OP_SIGN_F32, L.OP_EXPM1_F32, L.OP_CBRT_F32,
         L.OP_SIN_F32, L.OP_COS_F32, L.OP_TAN_F32,
         L.OP_ROUND_NEAREST_EVEN_F32, L.OP_ROUND_NEAREST_AFZ_F32]
_UN_F_POS = [L.OP_LOG_F32, L.OP_SQRT_F32, L.OP_RSQRT_F32, L.OP_LOG1P_F32]


def _ew_float(dtype, lanes):
    a = Asm()
    x = a.input((RAG,), dtype)
    y = a.input((RAG,), dtype)
    p = a.input((RAG,), dtype)          # positive operand
    outs = [a.binop(op, x, y) for op in _BIN_F]
    outs.append(a.binop(L.OP_POW_F32, p, y))
    # round_nearest_afz is left out for 2-byte floats: the validator evaluates
    # floor(|x| + 0.5) in the storage precision (ops/elementwise.py:171-175),
    # which double-rounds just below .5; the device calls round() on the f32.
    outs += [a.unop(op, x) for op in _UN_F
             if dtype == F32 or op != L.OP_ROUND_NEAREST_AFZ_F32]
    outs += [a.unop(op, p) for op in _UN_F_POS]
    outs.append(a.gelu_fused(x))
    outs.append(a.copy(x))
    blob, prog = a.finish(outs, nlanes=lanes)
    d = DN[dtype]
    return blob, prog, (1, [N((RAG,), d, 1.5), N((RAG,), d, 1.5),
                            U((RAG,), 0.05, 4.0, d)])


@case("ew_f32_all", rtol=1e-5, atol=1e-6)
def _():
    return _ew_float(F32, 3)


@case("ew_bf16_all", rtol=2e-2, atol=1e-2)
def _():
    return _ew_float(BF16, 2)


@case("ew_f16_all", rtol=2e-2, atol=1e-2)
def _():
    return _ew_float(F16, 2)


def _ew_int(dtype, lanes):
    a = Asm()
    x = a.input((RAG,), dtype)
    y = a.input((RAG,), dtype)
    s = a.input((RAG,), dtype)          # shift counts 0..31
    outs = [a.binop(op, x, y) for op in
            (L.OP_ADD_F32, L.OP_MUL_F32, L.OP_SUB_F32, L.OP_DIV_F32,
             L.OP_MAX_F32, L.OP_MIN_F32, L.OP_AND, L.OP_OR, L.OP_XOR)]
    outs += [a.binop(op, x, s) for op in (L.OP_SHL, L.OP_SHR_L, L.OP_SHR_A)]
    outs += [a.unop(op, x) for op in (L.OP_NEG_F32, L.OP_ABS_F32, L.OP_SIGN_F32,
                                      L.OP_NOT)]
    outs.append(a.copy(x))
    blob, prog = a.finish(outs, nlanes=lanes)
    d = DN[dtype]
    # The divisor never is 0: the validators divide in float64 and cast inf to an
    # undefined integer, while the device defines x / 0 = 0 (ew.cl:410); that
    # device rule is covered by a known-answer test, not by a fixture.
    lo, hi = (-1000, 1000) if dtype != U32 else (0, 2000)
    return blob, prog, (2, [I((RAG,), lo * 1000, hi * 1000, d), I((RAG,), 1, 21, d),
                            I((RAG,), 0, 32, d)])


@case("ew_i32_all", exact=True)
def _():
    return _ew_int(I32, 3)


@case("ew_u32_high", exact=True)
def _():
    """u32 operands at and above 2^31, where signed and unsigned arithmetic part ways:
    division, maximum / minimum, right shifts, comparison and the conversion to f32."""
    a = Asm()
    x = a.input((RAG,), U32)
    y = a.input((RAG,), U32)
    s = a.input((RAG,), U32)
    outs = [a.binop(op, x, y) for op in (L.OP_ADD_F32, L.OP_SUB_F32, L.OP_DIV_F32, L.OP_MAX_F32, L.OP_MIN_F32,
                                         L.OP_AND, L.OP_OR, L.OP_XOR)]
    outs += [a.binop(op, x, s) for op in (L.OP_SHR_L, L.OP_SHL)]
    outs += [a.compare(x, y, d) for d in ("LT", "GE")]
    outs.append(a.convert(x, F32))
    blob, prog = a.finish(outs, nlanes=3)
    return blob, prog, (21, [I((RAG,), 2 ** 31 - 5000, 2 ** 32 - 1, "u32"), I((RAG,), 2 ** 31 - 100, 2 ** 32 - 7, "u32"),
                             I((RAG,), 0, 32, "u32")])


@case("ew_i64_all", exact=True)
def _():
    return _ew_int(I64, 2)


@case("ew_cmp_select_bool", exact=True)
def _():
    a = Asm()
    xf = a.input((RAG,), F32)
    yf = a.input((RAG,), F32)
    xi = a.input((RAG,), I32)
    yi = a.input((RAG,), I32)
    xb = a.input((RAG,), BF16)
    yb = a.input((RAG,), BF16)
    outs = []
    preds = []
    for d in ("EQ", "NE", "LT", "LE", "GT", "GE"):
        preds.append(a.compare(xf, yf, d))
        outs.append(preds[-1])
        outs.append(a.compare(xi, yi, d))
        outs.append(a.compare(xb, yb, d))
    p, q = preds[2], preds[4]
    outs += [a.and_(p, q), a.or_(p, q), a.xor(p, q), a.unop(L.OP_NOT, p)]
    outs += [a.select(p, xf, yf), a.select(q, xi, yi), a.select(p, xb, yb),
             a.select(p, q, preds[0])]
    fin = a.div(xf, a.maximum(yf, a.scalar(0.0, yf)))     # produces inf / nan
    outs += [a.unop(L.OP_IS_FINITE, fin)]
    for o in outs[-1:]:
        a.ctx.buffers[o.buf].dtype = BOOL
        a.ctx.buffers[o.buf].size_bytes = o.n
        o.dtype = BOOL
    blob, prog = a.finish(outs, nlanes=3)
    return blob, prog, (3, [("int", (RAG,), "f32", -3, 4), ("int", (RAG,), "f32", -3, 4),
                            I((RAG,), -3, 4), I((RAG,), -3, 4),
                            ("int", (RAG,), "bf16", -3, 4), ("int", (RAG,), "bf16", -3, 4)])


@case("ew_convert_bitcast", exact=True)
def _():
    a = Asm()
    xf = a.input((RAG,), F32)
    xi = a.input((RAG,), I32)
    xb = a.input((RAG,), BF16)
    xh = a.input((RAG,), F16)
    xl = a.input((RAG,), I64)
    xu = a.input((RAG,), U32)
    pb = a.compare(xi, a.unop(L.OP_NEG_F32, xi), "GT")
    outs = [a.convert(xf, I32), a.convert(xf, BF16), a.convert(xf, F16),
            a.convert(xf, I64), a.convert(xi, F32), a.convert(xi, BF16),
            a.convert(xi, I64), a.convert(xb, F32), a.convert(xb, F16),
            a.convert(xb, I32), a.convert(xh, F32), a.convert(xh, BF16),
            a.convert(xl, I32), a.convert(xl, F32), a.convert(xu, F32),
            a.convert(pb, F32), a.convert(pb, I32), a.convert(pb, BF16),
            a.bitcast(xf, I32), a.bitcast(xi, F32), a.bitcast(xb, F16),
            a.bitcast(xu, I32)]
    blob, prog = a.finish(outs, nlanes=2)
    return blob, prog, (4, [N((RAG,), "f32", 300.0), I((RAG,), -2**24, 2**24),
                            N((RAG,), "bf16", 100.0), N((RAG,), "f16", 100.0),
                            I((RAG,), -2**30, 2**30, "i64"),
                            I((RAG,), 0, 2**24, "u32")])


@case("ew_affine_fill", rtol=1e-6, atol=1e-6)
def _():
    a = Asm()
    x = a.input((RAG,), F32)
    y = a.add(a.mul(x, a.scalar(1.5, x)), a.scalar(-0.25, x))      # one affine
    z = a.sub(a.scalar(2.0, x), x)                                # c - x
    fill = T_new(a, (RAG,), F32)
    a.ctx.emit(L.Instr(L.OP_FILL_F32, dst=fill.buf, n=RAG, imm=L._f32_bits(3.25)))
    blob, prog = a.finish([y, z, fill], nlanes=3)
    return blob, prog, (5, [N((RAG,))])


def T_new(a, shape, dtype):
    return a._new(shape, dtype)


# ---------------------------------------------------------------- views / gather
@case("ew_views_f32", rtol=1e-6, atol=1e-6)
def _():
    a = Asm()
    R_, C = 37, 260
    x = a.input((R_, C), F32)
    row = a.input((R_,), F32)
    col = a.input((C,), F32)
    sc = a.input((), F32)
    xt = a.input((C, R_), F32)
    big = a.input((R_ + 3, C + 5), F32)
    o1 = a.sub(x, a.broadcast_in_dim(row, (R_, C), [0]))
    o2 = a.mul(a.broadcast_in_dim(col, (R_, C), [1]), x)
    o3 = a.add(x, a.broadcast_in_dim(sc, (R_, C), []))
    o4 = a.add(x, a.transpose(xt, [1, 0]))
    o5 = a.maximum(x, a.slice(big, [2, 3], [2 + R_, 3 + C]))
    o6 = a.exp(a.broadcast_in_dim(row, (R_, C), [0]))
    o7 = a.div(a.broadcast_in_dim(col, (R_, C), [1]),
               a.broadcast_in_dim(a.exp(row), (R_, C), [0]))
    blob, prog = a.finish([o1, o2, o3, o4, o5, o6, o7], nlanes=4)
    return blob, prog, (6, [N((R_, C)), N((R_,)), N((C,)), N(()), N((C, R_)),
                            N((R_ + 3, C + 5))])


@case("ew_views_aligned_f32_bf16", rtol=2e-2, atol=1e-2)
def _():
    """Row/column broadcasts with a last dim that is a multiple of the vector
    width (the vectorised view classes), f32 and bf16."""
    a = Asm()
    R_, C = 40, 512
    outs = []
    items = []
    for dt in (F32, BF16):
        x = a.input((R_, C), dt)
        row = a.input((R_,), dt)
        col = a.input((C,), dt)
        outs.append(a.add(a.mul(x, a.broadcast_in_dim(col, (R_, C), [1])),
                          a.broadcast_in_dim(row, (R_, C), [0])))
        items += [N((R_, C), DN[dt]), N((R_,), DN[dt]), N((C,), DN[dt])]
    blob, prog = a.finish(outs, nlanes=3)
    return blob, prog, (7, items)


@case("gather_shapes", exact=True)
def _():
    a = Asm()
    x = a.input((33, 70), F32)
    x3 = a.input((5, 12, 34), F32)
    xb = a.input((48, 64), BF16)
    xq = a.input((19, 23), BOOL)
    xl = a.input((9, 11), I64)
    v = a.input((70,), F32)
    outs = [a.transpose(x, [1, 0]), a.transpose(x3, [2, 0, 1]),
            a.transpose(x3, [0, 2, 1]), a.transpose(xb, [1, 0]),
            a.transpose(xq, [1, 0]), a.transpose(xl, [1, 0]),
            a.slice(x, [1, 2], [30, 68], [2, 3]),
            a.broadcast_in_dim(v, (50, 70), [1]),
            a.broadcast_in_dim(v, (70, 9), [0]),
            a.transpose(a.reshape(xb, (4, 12, 2, 32)), [0, 2, 1, 3])]
    # reverse along axis 1 (negative stride), as ops/shape.py:157-170
    outs.append(a._gather(x, (33, 70), [70, -1], 69))
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (8, [N((33, 70)), N((5, 12, 34)), N((48, 64), "bf16"),
                            I((19, 23), 0, 2, "bool"), I((9, 11), -99, 99, "i64"),
                            N((70,))])


@case("scatter_concat_pad", exact=True)
def _():
    a = Asm()
    x = a.input((6, 40), F32)
    y = a.input((6, 25), F32)
    z = a.input((3, 40), F32)
    c1 = a.concatenate([x, y], axis=1)
    c2 = a.concatenate([x, z, x], axis=0)
    xb = a.input((6, 40), BF16)
    c3 = a.concatenate([xb, xb], axis=0)
    blob, prog = a.finish([c1, c2, c3], nlanes=3)
    return blob, prog, (9, [N((6, 40)), N((6, 25)), N((3, 40)),
                            N((6, 40), "bf16")])


@case("iota_dims", exact=True)
def _():
    a = Asm()
    outs = [a.iota((7, 50, 3), 0, F32), a.iota((7, 50, 3), 1, I32),
            a.iota((7, 50, 3), 2, F32), a.iota((RAG,), 0, I32),
            a.iota((30, 30), 1, I64)]
    blob, prog = a.finish(outs, nlanes=2)
    return blob, prog, (0, [])


@case("dynslice", exact=True)
def _():
    a = Asm()
    x = a.input((20, 64), F32)
    upd = a.input((4, 16), F32)
    i0 = a.input((), I32)
    i1 = a.input((), I32)
    big = a.input((), I32)          # out of range -> clamped
    neg = a.input((), I32)
    outs = [a.dynamic_slice(x, [i0, i1], (5, 32)),
            a.dynamic_slice(x, [big, neg], (5, 32)),
            a.dynamic_update_slice(x, upd, [i0, i1]),
            a.dynamic_update_slice(x, upd, [big, big])]
    blob, prog = a.finish(outs, nlanes=3)
    return blob, prog, (10, [N((20, 64)), N((4, 16)), ("value", (), "i32", 7),
                             ("value", (), "i32", 13), ("value", (), "i32", 1000),
                             ("value", (), "i32", -5)])


# ---------------------------------------------------------------- reductions
@case("reduce_full", rtol=1e-5, atol=1e-5)
def _():
    a = Asm()
    x = a.input((5, 4096 * 3 + 11), F32)
    small = a.input((100,), F32)
    p = a.input((64,), F32)
    outs = [a.reduce(x, [0, 1], k) for k in (SUM, MAX, MIN)]
    outs += [a.reduce(small, [0], SUM), a.reduce(p, [0], PROD)]
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (11, [N((5, 4096 * 3 + 11)), N((100,)), U((64,), 0.8, 1.25)])


@case("reduce_full_16bit_source", rtol=1e-5, atol=1e-3)
def _():
    """Full f32 sums of the f32 copies of a bf16 and an f16 tensor (what an upcasting reduction lowers
    to): the backend may stream the 16-bit source instead of writing the copy. A third sum reads a copy
    that is also a program output, which therefore has to be written."""
    a = Asm()
    n = 65536 + 8 * 37
    xb = a.input((n,), BF16)
    xh = a.input((n,), F16)
    xk = a.input((n,), BF16)
    kept = a.convert(xk, F32)
    outs = [a.reduce(a.convert(xb, F32), [0], SUM), a.reduce(a.convert(xh, F32), [0], SUM),
            a.reduce(kept, [0], SUM), kept]
    blob, prog = a.finish(outs, nlanes=5)
    return blob, prog, (23, [N((n,), "bf16"), N((n,), "f16"), N((n,), "bf16")])


@case("rows_then_full_sum_f32", rtol=1e-5, atol=1e-4)
def _():
    """Softmax rows, then the sum of everything it wrote; the rows are a program output too. The backend may
    let the row op carry the sum instead of streaming the rows again."""
    a = Asm()
    x = a.input((72, 1024), F32)
    sm = a.softmax_fused(x)
    blob, prog = a.finish([sm, a.reduce(sm, [0, 1], SUM)], nlanes=5)
    return blob, prog, (29, [N((72, 1024), "f32", 2.0, 0.5)])


@case("rows_then_full_sum_bf16", rtol=0.3, atol=2e-2)
def _():
    """The same through 16-bit storage: layer norm and softmax in bf16, up-cast, full sum; neither the rows nor
    their f32 copy leave the program. The validators' numpy bodies add a bf16 row up in bf16 (reduce.py:464-475
    applied to bf16 arrays), so their softmax rows sum to about 1.25 where f32 accumulation gives 1: this fixture
    pins the total only that loosely, and the GPU tests compare the carried total with the streamed one."""
    a = Asm()
    x = a.input((72, 1024), BF16)
    g = a.input((72, 1024), BF16)
    ln = a.layernorm_fused(x, 1e-5)
    total = a.reduce(a.convert(a.softmax_fused(a.add(ln, g)), F32), [0, 1], SUM)
    blob, prog = a.finish([total], nlanes=5)
    return blob, prog, (31, [N((72, 1024), "bf16", 2.0, 0.5), N((72, 1024), "bf16")])


@case("rows_then_full_sum_ragged", rtol=1e-5, atol=1e-4)
def _():
    """Rows too short for the staged path (100 elements), summed afterwards."""
    a = Asm()
    x = a.input((700, 100), F32)
    blob, prog = a.finish([a.reduce(a.softmax_fused(x), [0, 1], SUM)], nlanes=5)
    return blob, prog, (37, [N((700, 100), "f32", 2.0, 0.5)])


@case("rmsnorm_rows_bf16", rtol=2e-2, atol=2e-2)
def _():
    """The decomposed RMS norm of the decoder block (cases._rmsnorm: f32 statistics, bf16 in and out) on rows of
    1024 and of 256 elements, the second one fed by an add the way the block's residual feeds its second norm.
    The backend may run each as one row op."""
    a = Asm()
    x = a.input((96, 1024), BF16)
    g = a.input((1024,), BF16)
    r = a.input((100, 256), BF16)
    s = a.input((100, 256), BF16)
    g2 = a.input((256,), BF16)
    x1 = a.add(r, s)
    blob, prog = a.finish([cases._rmsnorm(a, x, g, 1e-6), cases._rmsnorm(a, x1, g2, 1e-6), x1], nlanes=5)
    return blob, prog, (41, [N((96, 1024), "bf16", 1.5, 0.3), N((1024,), "bf16", 0.2, 1.0),
                             N((100, 256), "bf16"), N((100, 256), "bf16"), N((256,), "bf16", 0.2, 1.0)])


@case("reduce_full_int", exact=True)
def _():
    a = Asm()
    x = a.input((3, 4096 * 2 + 5), I32)
    u = a.input((4096 + 9,), U32)
    b = a.input((5000,), BOOL)
    outs = [a.reduce(x, [0, 1], k) for k in (SUM, MAX, MIN, RED.AND, RED.OR,
                                             RED.XOR)]
    outs += [a.reduce(u, [0], k) for k in (SUM, MAX, MIN)]
    outs += [a.reduce(b, [0], k) for k in (RED.AND, RED.OR, RED.XOR)]
    blob, prog = a.finish(outs, nlanes=3)
    return blob, prog, (12, [I((3, 4096 * 2 + 5), -50000, 50000),
                             I((4096 + 9,), 2**31 - 5000, 2**31 + 5000, "u32"),
                             I((5000,), 0, 2, "bool")])


@case("reduce_seg", rtol=1e-5, atol=1e-5)
def _():
    a = Asm()
    outs, items = [], []
    for rows, seg in ((300, 3), (70, 64), (33, 1000), (9, 4096), (5, 5003),
                      (1, 17)):
        x = a.input((rows, seg), F32)
        items.append(N((rows, seg)))
        for k in (SUM, MAX, MIN):
            outs.append(a.reduce(x, [1], k))
    xp = a.input((40, 12), F32)
    items.append(U((40, 12), 0.8, 1.25))
    outs.append(a.reduce(xp, [1], PROD))
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (13, items)


@case("reduce_seg_int", exact=True)
def _():
    a = Asm()
    x = a.input((50, 77), I32)
    u = a.input((20, 130), U32)
    outs = [a.reduce(x, [1], k) for k in (SUM, MAX, MIN, RED.XOR)]
    outs += [a.reduce(u, [1], k) for k in (MAX, MIN)]
    blob, prog = a.finish(outs, nlanes=2)
    return blob, prog, (14, [I((50, 77), -10**6, 10**6),
                             I((20, 130), 2**31 - 999, 2**31 + 999, "u32")])


@case("reduce_strided", rtol=1e-5, atol=1e-5)
def _():
    a = Asm()
    x = a.input((7, 50, 3), F32)            # nbody shape class: inner 3
    y = a.input((300, 1200), F32)           # axis-0 (prefix) reduce, wide inner
    z = a.input((4, 33, 5000), F32)         # interior, inner > tile
    outs = [a.reduce(x, [1], SUM), a.reduce(x, [1], MAX),
            a.reduce(y, [0], SUM), a.reduce(y, [0], MIN),
            a.reduce(z, [1], SUM), a.reduce(x, [0, 1], SUM)]
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (15, [N((7, 50, 3)), N((300, 1200)), N((4, 33, 5000))])


@case("gemv_dot_mode", rtol=1e-5, atol=1e-4)
def _():
    a = Asm()
    m = a.input((130, 515), F32)
    v = a.input((515, 1), F32)
    blob, prog = a.finish([a.matmul(m, v)], nlanes=3)
    return blob, prog, (16, [N((130, 515)), N((515, 1))])


@case("norms_fused", rtol=1e-5, atol=1e-5)
def _():
    a = Asm()
    outs, items = [], []
    for rows, seg in ((50, 8), (33, 100), (17, 1024), (6, 4096), (3, 5003)):
        x = a.input((rows, seg), F32)
        items.append(N((rows, seg), "f32", 2.0, 0.5))
        outs.append(a.softmax_fused(x))
        outs.append(a.layernorm_fused(x, 1e-5))
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (17, items)


@case("norms_recognized", rtol=1e-5, atol=1e-5)
def _():
    """Decomposed softmax / layernorm idioms at seg <= 1024, collapsed by the
    reference's own `_fuse_norm` recognizer (lowering.py:1561-1730)."""
    blob, prog, ins = cases.c2_chain(rows=24, cols=512, nlanes=4, fused=False)
    return blob, prog, ins


@case("map_region", rtol=1e-5, atol=1e-5)
def _():
    """Long pure-map f32 chains that `_fuse_region` (lowering.py:2071-2212)
    rewrites into OP_MAP_REGION micro-programs."""
    a = Asm()
    x = a.input((RAG,), F32)
    y = a.input((RAG,), F32)
    z = a.input((RAG,), F32)
    t = a.tanh(a.add(a.mul(x, y), z))
    u = a.exp(a.neg(a.mul(t, t)))
    v = a.div(a.sub(u, x), a.add(a.unop(L.OP_ABS_F32, y), a.scalar(1.0, y)))
    w = a.sqrt(a.add(a.mul(v, v), a.scalar(0.5, v)))
    o = a.maximum(a.minimum(w, a.add(z, a.scalar(3.0, z))), a.rsqrt(a.add(u, a.scalar(1.0, u))))
    o2 = a.log(a.add(a.mul(o, o), a.scalar(1.0, o)))
    blob, prog = a.finish([o2], nlanes=3)
    return blob, prog, (18, [N((RAG,)), N((RAG,)), N((RAG,))])


# ---------------------------------------------------------------- windows, indexed moves, convolution
@case("reduce_window_f32", rtol=1e-5, atol=1e-5)
def _():
    """Pooling shapes: channel-last 2x2/2 max and 3x3/2 padded sum (NHWC), a
    window over the innermost axes (NCHW) with padding, and a 1-D running min."""
    a = Asm()
    x = a.input((2, 17, 19, 8), F32)
    y = a.input((3, 4, 21, 22), F32)
    z = a.input((5003,), F32)
    outs = [a.reduce_window(x, (1, 2, 2, 1), (1, 2, 2, 1), kind=MAX),
            a.reduce_window(x, (1, 3, 3, 1), (1, 2, 2, 1), (0, 1, 1, 0), (0, 1, 1, 0), kind=SUM),
            a.reduce_window(y, (1, 1, 3, 3), (1, 1, 1, 2), (0, 0, 1, 2), (0, 0, 1, 0), kind=MAX),
            a.reduce_window(z, (7,), (3,), (2,), (4,), kind=MIN)]
    blob, prog = a.finish(outs, nlanes=5)
    return blob, prog, (40, [N((2, 17, 19, 8)), N((3, 4, 21, 22)), N((5003,))])


@case("reduce_window_int", exact=True)
def _():
    a = Asm()
    x = a.input((3, 33, 12), I32)
    u = a.input((40, 36), U32)
    outs = [a.reduce_window(x, (1, 4, 1), (1, 3, 1), (0, 2, 0), (0, 1, 0), kind=SUM),
            a.reduce_window(x, (2, 2, 2), (1, 1, 2), kind=MAX),
            a.reduce_window(u, (3, 3), (2, 1), (1, 1), (1, 1), kind=MAX),
            a.reduce_window(u, (2, 5), (2, 3), kind=MIN)]
    blob, prog = a.finish(outs, nlanes=3)
    return blob, prog, (41, [I((3, 33, 12), -2 ** 30, 2 ** 30), I((40, 36), 0, 2 ** 32, "u32")])


@case("gather_index", exact=True)
def _():
    """Embedding-style row lookups (f32 rows of 64, bf16 rows of 40, i64 rows of 3,
    i64 indices, out-of-range indices clamped) and a two-component point gather."""
    a = Asm()
    tab = a.input((300, 64), F32)
    tb = a.input((129, 40), BF16)
    tl = a.input((50, 3), I64)
    grid = a.input((37, 53), I32)
    i1 = a.input((1200,), I32)
    i2 = a.input((700,), I64)
    i3 = a.input((900, 2), I32)
    outs = [a.take_rows(tab, i1), a.take_rows(tb, i2), a.take_rows(tl, i2), a.take_points(grid, i3)]
    blob, prog = a.finish(outs, nlanes=6)
    return blob, prog, (42, [N((300, 64)), N((129, 40), "bf16"), I((50, 3), -2 ** 40, 2 ** 40, "i64"),
                             I((37, 53), -1000, 1000), I((1200,), -5, 305), I((700,), -3, 140, "i64"),
                             I((900, 2), -2, 56)])


@case("scatter_index_exact", exact=True)
def _():
    """Overwrite with unique indices (any order gives the same bytes) and the
    integer combiners with heavily duplicated indices (order-free, bit-exact)."""
    a = Asm()
    tab = a.input((400, 16), F32)
    ti = a.input((64, 8), I32)
    tu = a.input((64, 8), U32)
    uniq = a.input((250,), I32)
    dup = a.input((3000,), I32)
    uf = a.input((250, 16), F32)
    ui = a.input((3000, 8), I32)
    uu = a.input((3000, 8), U32)
    outs = [a.scatter_rows(tab, uniq, uf, 0), a.scatter_rows(ti, dup, ui, 1), a.scatter_rows(ti, dup, ui, 2),
            a.scatter_rows(ti, dup, ui, 3), a.scatter_rows(tu, dup, uu, 1), a.scatter_rows(tu, dup, uu, 2),
            a.scatter_rows(tu, dup, uu, 3)]
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (43, [N((400, 16)), I((64, 8), -10 ** 6, 10 ** 6), I((64, 8), 0, 2 ** 32, "u32"),
                             ("perm", (250,), "i32", 400), I((3000,), -4, 70),
                             N((250, 16)), I((3000, 8), -10 ** 6, 10 ** 6), I((3000, 8), 0, 2 ** 32, "u32")])


@case("scatter_index_f32", exact=True)
def _():
    """f32 combiners with duplicate indices. max / min are order-free; add sums ~47
    updates per row in whatever order the lanes reach them, so the values are small
    integers: every partial sum is exact and the result is the same in any order
    (the reference's lane simulator refuses a phase whose result depends on lane order)."""
    a = Asm()
    tab = a.input((64, 32), F32)
    dup = a.input((3000,), I32)
    upd = a.input((3000, 32), F32)
    outs = [a.scatter_rows(tab, dup, upd, 1), a.scatter_rows(tab, dup, upd, 2), a.scatter_rows(tab, dup, upd, 3)]
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (44, [I((64, 32), -50, 50, "f32"), I((3000,), -4, 70), I((3000, 32), -64, 64, "f32")])


@case("conv_f32", rtol=1e-5, atol=2e-5)
def _():
    """1-D, 2-D (stride, padding, dilation; Cout not a multiple of 4) and 3-D convolutions."""
    a = Asm()
    x1 = a.input((3, 50, 5), F32)
    w1 = a.input((4, 5, 7), F32)
    x2 = a.input((2, 15, 14, 6), F32)
    w2 = a.input((3, 3, 6, 16), F32)
    w2b = a.input((2, 3, 6, 5), F32)
    x3 = a.input((1, 6, 7, 5, 3), F32)
    w3 = a.input((2, 2, 2, 3, 8), F32)
    outs = [a.conv(x1, w1, (2,), (1,), (2,)),
            a.conv(x2, w2, (1, 1), (1, 1), (1, 1)),
            a.conv(x2, w2b, (2, 1), (0, 2), (1, 0), (2, 1)),
            a.conv(x3, w3, (1, 2, 1))]
    blob, prog = a.finish(outs, nlanes=4)
    return blob, prog, (45, [N((3, 50, 5)), N((4, 5, 7), "f32", 0.3), N((2, 15, 14, 6)),
                             N((3, 3, 6, 16), "f32", 0.2), N((2, 3, 6, 5), "f32", 0.2),
                             N((1, 6, 7, 5, 3)), N((2, 2, 2, 3, 8), "f32", 0.3)])


# ---------------------------------------------------------------- control flow
@case("golden_layout_kat", exact=True)
def _():
    """The reference's byte-layout golden program
    (tests/test_lowering.py:89-104): b3 = (b0 + b1) - [1,2,3]."""
    const = np.array([1.0, 2.0, 3.0], dtype=np.float32)
    prog = L.VMProgram(
        arena_bytes=256,
        buffers=[L.Buffer(0, 12), L.Buffer(64, 12), L.Buffer(128, 12),
                 L.Buffer(192, 12)],
        inputs=[0, 1], outputs=[3], input_shapes=[(3,), (3,)],
        output_shapes=[(3,)], consts=[(2, const.tobytes())],
        instrs=[L.Instr(L.OP_ADD_F32, dst=3, a=0, b=1, n=3),
                L.Instr(L.OP_SUB_F32, dst=3, a=3, b=2, n=3)],
        main_len=2)
    from pjrt_ocl import scheduler as S
    blob = prog.serialize(S.schedule_program(prog, S.DeviceConfig(nlanes=8)))
    return blob, prog, (19, [("int", (3,), "f32", -9, 9), ("int", (3,), "f32", -9, 9)])


@case("for_loop_carries", rtol=1e-5, atol=1e-5)
def _():
    a = Asm()
    x0 = a.input((RAG,), F32)
    v0 = a.input((RAG,), F32)

    def body(a, c):
        x, v = c
        acc = a.neg(x)                                 # harmonic oscillator
        v2 = a.add(v, a.mul(a.scalar(0.01, acc), acc))
        x2 = a.add(x, a.mul(a.scalar(0.01, v2), v2))
        return [x2, v2]
    x, v = a.fori_loop(25, [x0, v0], body)
    blob, prog = a.finish([x, v], nlanes=3)
    return blob, prog, (20, [N((RAG,)), N((RAG,))])


@case("for_loop_cross_lane", rtol=1e-4, atol=1e-4)
def _():
    """Loop body with a reduction + broadcast each iteration, so loop-carried
    data crosses lanes through the per-iteration barrier."""
    a = Asm()
    x0 = a.input((64, 300), F32)

    def body(a, c):
        (x,) = c
        m = a.reduce(x, [1], MAX)
        y = a.sub(x, a.broadcast_in_dim(m, (64, 300), [0]))
        return [a.add(a.mul(a.scalar(0.5, y), y), a.scalar(1.0, y))]
    (x,) = a.fori_loop(7, [x0], body)
    blob, prog = a.finish([x], nlanes=4)
    return blob, prog, (21, [N((64, 300))])


@case("while_loop_data_dependent", rtol=1e-6, atol=1e-6)
def _():
    a = Asm()
    x0 = a.input((5000,), F32)
    i0 = a.input((), F32)
    lim = a.input((), F32)

    def cond(a, c):
        x, i = c
        return a.compare(i, lim, "LT")

    def body(a, c):
        x, i = c
        return [a.add(x, x), a.add(i, a.scalar(1.0, i))]
    x, i = a.while_loop([x0, i0], cond, body)
    blob, prog = a.finish([x, i], nlanes=3)
    return blob, prog, (22, [("int", (5000,), "f32", 1, 14), ("value", (), "f32", 0.0),
                             ("value", (), "f32", 10.0)])


# ---------------------------------------------------------------- contractions
def _dot_case(dtype, out_dtype, shapes, lanes):
    a = Asm()
    outs, items = [], []
    for (M, K, N_) in shapes:
        x = a.input((M, K), dtype)
        y = a.input((K, N_), dtype)
        outs.append(a.matmul(x, y, out_dtype=out_dtype))
        items += [N((M, K), DN[dtype]), N((K, N_), DN[dtype])]
    blob, prog = a.finish(outs, nlanes=lanes)
    return blob, prog, (23, items)


_DOT_SHAPES = [(2, 2, 2), (96, 128, 64), (130, 70, 257), (1, 300, 5),
               (257, 33, 129), (256, 512, 384)]


@case("dot_f32", rtol=1e-5, atol=1e-4)
def _():
    return _dot_case(F32, F32, _DOT_SHAPES, 4)


@case("dot_bf16", rtol=2e-2, atol=2e-2)
def _():
    return _dot_case(BF16, BF16, _DOT_SHAPES, 4)


@case("dot_bf16_f32out", rtol=1e-5, atol=1e-3)
def _():
    return _dot_case(BF16, F32, _DOT_SHAPES, 4)


@case("dot_f16", rtol=2e-2, atol=2e-2)
def _():
    return _dot_case(F16, F16, _DOT_SHAPES, 4)


def _dot_tc_case(dtype, out_dtype, fold_views=False):
    """Shapes whose operands are 16-byte friendly (every leading dimension a multiple
    of 8 elements) but not multiples of the 128 tile or the 64-wide k block, in all
    four operand layouts: plain, q k^T (both k-contiguous), x^T y (both row-contiguous),
    batched, plus a bias + GELU + residual store epilogue."""
    a = Asm()
    dn = DN[dtype]
    q = a.input((3, 200, 72), dtype)
    k = a.input((3, 136, 72), dtype)
    x = a.input((264, 136), dtype)
    y = a.input((264, 152), dtype)
    w = a.input((136, 328), dtype)
    b = a.input((328,), dtype)
    r = a.input((264, 328), dtype)
    s = a.dot_general(q, k, lb=[0], lc=2, rb=[0], rc=2, out_dtype=out_dtype)       # [3,200,136]
    kk = a.input((3, 136, 88), dtype)
    sk = a.dot_general(a.convert(s, dtype) if out_dtype != dtype else s, kk, lb=[0], lc=2, rb=[0], rc=1,
                       out_dtype=out_dtype)                                       # [3,200,88]
    g = a.dot_general(x, y, lc=0, rc=0, out_dtype=out_dtype)                      # x^T y: [136,152]
    e = a.matmul(x, w, out_dtype=dtype)                                           # [264,328] + epilogue
    e = a.add(e, a.broadcast_in_dim(b, (264, 328), [1]))
    e = a.gelu_tanh(e)
    e = a.add(e, r)
    big = a.matmul(a.input((384, 520), dtype), a.input((520, 640), dtype), out_dtype=out_dtype)
    blob, prog = a.finish([s, sk, g, e, big], nlanes=6, fold_2byte_matmul_views=fold_views)
    return blob, prog, (29, [N((3, 200, 72), dn, 0.5), N((3, 136, 72), dn, 0.5), N((264, 136), dn, 0.5),
                             N((264, 152), dn, 0.5), N((136, 328), dn, 0.1), N((328,), dn), N((264, 328), dn),
                             N((3, 136, 88), dn, 0.2), N((384, 520), dn, 0.3), N((520, 640), dn, 0.1)])


@case("dot_tc_bf16", rtol=2e-2, atol=3e-2)
def _():
    return _dot_tc_case(BF16, BF16)


@case("dot_tc_bf16_f32out", rtol=2e-2, atol=3e-2)
def _():
    return _dot_tc_case(BF16, F32)


@case("dot_tc_f16", rtol=2e-2, atol=3e-2)
def _():
    return _dot_tc_case(F16, F16)


@case("dot_tc_views_bf16", rtol=2e-2, atol=3e-2)
def _():
    """The same graph with the transposes folded into the matmul tasks as operand
    views: k-contiguous B (q k^T) and row-contiguous A (x^T y) reach the matmul."""
    return _dot_tc_case(BF16, BF16, fold_views=True)


@case("dot_tc_broadcast_bf16", rtol=2e-2, atol=3e-2)
def _():
    """A batched 16-bit dot_general whose right operand is the broadcast of one program
    input over the batch: `_fuse_matmul_views` folds the broadcast into the matmul's operand
    view (batch stride 0), and the operand is an I/O port. Both results must come out the
    same whichever path (tensor maps or per-thread copies) the backend takes."""
    a = Asm()
    x = a.input((4, 200, 136), BF16)
    w = a.input((136, 152), BF16)
    wb = a.broadcast_in_dim(w, (4, 136, 152), [1, 2])
    o = a.dot_general(x, wb, lb=[0], lc=2, rb=[0], rc=1, out_dtype=BF16)           # [4,200,152]
    xb = a.broadcast_in_dim(a.input((200, 136), BF16), (4, 200, 136), [1, 2])
    o2 = a.dot_general(xb, a.input((4, 136, 88), BF16), lb=[0], lc=2, rb=[0], rc=1, out_dtype=F32)
    blob, prog = a.finish([o, o2], nlanes=6, fold_2byte_matmul_views=True)
    return blob, prog, (31, [N((4, 200, 136), "bf16", 0.5), N((136, 152), "bf16", 0.2),
                             N((200, 136), "bf16", 0.5), N((4, 136, 88), "bf16", 0.2)])


@case("dot_kat_2x2", exact=True)
def _():
    """tests/test_ops_dot.py:56-63 known answer: [[1,2],[3,4]] @ [[5,6],[7,8]]
    = [[19,22],[43,50]]; inputs are constants."""
    a = Asm()
    x = a.const(np.array([[1, 2], [3, 4]], np.float32))
    y = a.const(np.array([[5, 6], [7, 8]], np.float32))
    blob, prog = a.finish([a.matmul(x, y)], nlanes=2)
    return blob, prog, (0, [])


@case("dot_batched_views", rtol=1e-5, atol=1e-4)
def _():
    """Batched matmuls and transposed operands; `_fuse_matmul_views`
    (lowering.py:2381-2452) folds the transposes into operand views."""
    a = Asm()
    q = a.input((6, 40, 24), F32)
    k = a.input((6, 50, 24), F32)
    w = a.input((70, 24), F32)
    x = a.input((130, 70), F32)
    s = a.dot_general(q, k, lb=[0], lc=2, rb=[0], rc=2)      # q @ k^T batched
    o = a.dot_general(s, k, lb=[0], lc=2, rb=[0], rc=1)      # s @ k
    xt = a.dot_general(x, w, lc=1, rc=0)                     # x @ w
    g = a.dot_general(x, xt, lc=0, rc=0)                     # x^T @ (x w)
    blob, prog = a.finish([s, o, xt, g], nlanes=4)
    return blob, prog, (24, [N((6, 40, 24)), N((6, 50, 24)), N((70, 24)),
                             N((130, 70))])


@case("dot_epilogue", rtol=1e-5, atol=1e-4)
def _():
    """Bias + GELU + residual after a matmul; `_fuse_mma_epilogue`
    (lowering.py:2486-2601) folds what it can into the store epilogue."""
    a = Asm()
    x = a.input((150, 96), F32)
    w = a.input((96, 200), F32)
    b = a.input((200,), F32)
    r = a.input((150, 200), F32)
    y = a.matmul(x, w)
    y = a.add(y, a.broadcast_in_dim(b, (150, 200), [1]))
    y = a.gelu_tanh(y)
    y = a.add(y, r)
    z = a.mul(a.matmul(x, w), a.scalar(0.125, r))
    blob, prog = a.finish([y, z], nlanes=4)
    return blob, prog, (25, [N((150, 96)), N((96, 200), "f32", 0.1), N((200,)),
                             N((150, 200))])


_FLASH_SHAPES = ((3, 40, 40, 16, True), (2, 70, 70, 64, False), (4, 1, 130, 64, True), (2, 33, 97, 32, True),
                 (1, 200, 200, 64, True))
# head_dim 64 and key counts that are multiples of 8 (what the tensor-core path takes),
# query counts off the 128-row block, more keys than queries, causal and not
_FLASH_TC_SHAPES = ((3, 200, 200, 64, True), (2, 136, 264, 64, True), (2, 72, 328, 64, False),
                    (2, 300, 304, 64, False))


def _flash_case(dtype, lanes, shapes=_FLASH_SHAPES):
    a = Asm()
    outs, items = [], []
    for (H, T_, C, hd, causal) in shapes:
        q = a.input((H, T_, hd), dtype)
        kt = a.input((H, hd, C), dtype)
        v = a.input((H, C, hd), dtype)
        outs.append(a.flash_attn(q, kt, v, 1.0 / math.sqrt(hd), causal))
        items += [N((H, T_, hd), DN[dtype]), N((H, hd, C), DN[dtype]),
                  N((H, C, hd), DN[dtype])]
    blob, prog = a.finish(outs, nlanes=lanes)
    return blob, prog, (26, items)


@case("flash_f32", rtol=1e-5, atol=1e-5)
def _():
    return _flash_case(F32, 4)


@case("flash_bf16", rtol=2e-2, atol=2e-2, twin=lambda: _flash_case(F32, 4))
def _():
    return _flash_case(BF16, 4)


@case("flash_tc_bf16", rtol=2e-2, atol=2e-2, twin=lambda: _flash_case(F32, 5, _FLASH_TC_SHAPES))
def _():
    return _flash_case(BF16, 5, _FLASH_TC_SHAPES)


@case("flash_tc_f16", rtol=2e-2, atol=2e-2, twin=lambda: _flash_case(F32, 5, _FLASH_TC_SHAPES))
def _():
    return _flash_case(F16, 5, _FLASH_TC_SHAPES)


# ---------------------------------------------------------------- configs
@case("c1_relu_matmul", rtol=1e-5, atol=1e-4)
def _():
    return cases.c1_relu_matmul(nlanes=8)


@case("c2_chain_f32_small", rtol=1e-5, atol=1e-5)
def _():
    return cases.c2_chain(rows=48, cols=4096, nlanes=8)


@case("c2_chain_decomposed_small", rtol=1e-5, atol=1e-5)
def _():
    return cases.c2_chain(rows=48, cols=4096, nlanes=8, fused=False)


@case("c2_int_chain_small", exact=True)
def _():
    return cases.c2_int_chain(rows=40, cols=4096, nlanes=8)


@case("c3_mlp_f32_small", rtol=1e-4, atol=1e-5)
def _():
    return cases.c3_mlp_step(batch=160, widths=(96, 256, 192, 64), nlanes=8,
                             dtype=F32)


@case("c3_dp2_grads_f32_small", rtol=1e-4, atol=1e-5)
def _():
    """Config 3's per-rank program at 2 ranks: gradients of half the batch, scaled for the global batch."""
    blob, prog, (seed, items) = cases.c3_mlp_step(batch=80, global_batch=160, widths=(96, 256, 192, 64), nlanes=8,
                                                  dtype=F32, apply_sgd=False)
    # the case lists x, y at the global batch (callers slice); this fixture feeds one shard
    items = [(k, (80,) + tuple(shp[1:]), *rest) if i < 2 else (k, shp, *rest) for i, (k, shp, *rest) in enumerate(items)]
    return blob, prog, (seed, items)


@case("c3_dp2_apply_f32_small", rtol=1e-5, atol=1e-6)
def _():
    """Config 3's post-all-reduce program: w <- w - lr g."""
    blob, prog, _ = cases.sgd_apply([(96, 256), (256, 192), (192, 64)], nlanes=8, dtype=F32)
    return blob, prog, (31, [N((96, 256)), N((256, 192)), N((192, 64)), N((96, 256), "f32", 0.01),
                             N((256, 192), "f32", 0.01), N((192, 64), "f32", 0.01)])


@case("c3_mlp_bf16_small", rtol=2e-2, atol=2e-2)
def _():
    return cases.c3_mlp_step(batch=160, widths=(96, 256, 192, 64), nlanes=8,
                             dtype=BF16)


@case("c4_nbody_small", rtol=1e-4, atol=1e-5)
def _():
    return cases.c4_nbody(n=96, steps=3, nlanes=8)


# 256 bodies on 8 lanes: the axis-1 force sum is one output tile, so the loader spreads it
# over the lanes by rows (two full 96-load steps per 768-element row); the trailing-axis
# sum has 65536 segments of 3
@case("c4_nbody_mid", rtol=1e-4, atol=1e-5)
def _():
    return cases.c4_nbody(n=256, steps=2, nlanes=8)


@case("c5_block_f32_small", rtol=1e-4, atol=1e-4)
def _():
    return cases.c5_block(batch=2, seq=48, d_model=128, heads=4, d_ff=256,
                          nlanes=8, dtype=F32)


@case("c5_block_bf16_small", rtol=2e-2, atol=3e-2,
      twin=lambda: cases.c5_block(batch=2, seq=48, d_model=128, heads=4,
                                  d_ff=256, nlanes=8, dtype=F32))
def _():
    return cases.c5_block(batch=2, seq=48, d_model=128, heads=4, d_ff=256,
                          nlanes=8, dtype=BF16)


@case("c5_decode_bf16_small", rtol=2e-2, atol=3e-2,
      twin=lambda: cases.c5_decode(batch=3, cache=70, d_model=128, heads=4,
                                   d_ff=256, nlanes=8, dtype=F32))
def _():
    return cases.c5_decode(batch=3, cache=70, d_model=128, heads=4, d_ff=256,
                           nlanes=8, dtype=BF16)


@case("c5_decode_in_place_f32_small", rtol=1e-4, atol=1e-4)
def _():
    return cases.c5_decode_in_place(batch=3, cache=70, d_model=128, heads=2, d_ff=256,
                                    nlanes=8, dtype=F32)


@case("c5_decode_in_place_bf16_small", rtol=2e-2, atol=3e-2,
      twin=lambda: cases.c5_decode_in_place(batch=3, cache=70, d_model=128, heads=2,
                                            d_ff=256, nlanes=8, dtype=F32))
def _():
    return cases.c5_decode_in_place(batch=3, cache=70, d_model=128, heads=2, d_ff=256,
                                    nlanes=8, dtype=BF16)


# ---------------------------------------------------------------- driver
def build(name):
    fn, meta = CASES[name]
    meta = dict(meta)
    twin = meta.pop("twin", None)
    blob, prog, (seed, items) = fn()
    args = gen_inputs.gen_all(seed, items)
    parsed = R.parse(blob)
    if twin is not None:
        # The validators cannot evaluate this program in its storage dtype
        # (numpy has no bf16 einsum; ml_dtypes reductions accumulate in bf16).
        # Expected values come from the validators run on the SAME graph built
        # in f32, fed the storage-rounded inputs, rounded once to the storage
        # dtype at the outputs.
        meta["oracle"] = "validators on the f32 twin program, outputs rounded"
        tblob, _tprog, _ = twin()
        tparsed = R.parse(tblob)
        targs = [a.astype(np.float32) if a.dtype.kind == "f" or a.dtype.itemsize == 2
                 and a.dtype.kind == "V" else a for a in args]
        targs = [np.asarray(a, dtype=np.float32)
                 if gen_inputs.ENUM_NAME[parsed.buffers[b].dtype] in ("bf16", "f16")
                 else a for a, b in zip(args, parsed.inputs)]
        sem32 = R.execute(tparsed, targs)
        sch32 = R.execute_schedule(tparsed, targs)
        odt = [L.DTYPE_NUMPY[parsed.buffers[b].dtype] for b in parsed.outputs]
        sem = [np.asarray(u).astype(d) for u, d in zip(sem32, odt)]
        sch = [np.asarray(u).astype(d) for u, d in zip(sch32, odt)]
    else:
        sem = R.execute(parsed, args)
        sch = R.execute_schedule(parsed, args)
    for i, (u, v) in enumerate(zip(sem, sch)):
        uu = np.atleast_1d(np.asarray(u))
        vv = np.atleast_1d(np.asarray(v))
        if meta.get("exact") or uu.dtype.kind in "iub":
            np.testing.assert_array_equal(uu.view(np.uint8), vv.view(np.uint8),
                                          err_msg=f"{name} out {i}")
        else:
            # the two validators may associate float reductions differently
            # (per-tile matmul blocks vs whole-matrix); both must be within
            # the case's own tolerance of each other.
            np.testing.assert_allclose(
                uu.astype(np.float64), vv.astype(np.float64),
                rtol=meta.get("rtol", 1e-5), atol=meta.get("atol", 1e-5),
                err_msg=f"{name} out {i}")
    out = {
        "blob": np.frombuffer(blob, np.uint8),
        "meta": np.frombuffer(json.dumps({
            "name": name, "seed": seed, "items": items, "numpy": np.__version__,
            "ew_ts": 4096, "mma_t": 128,
            "out_dtypes": [gen_inputs.ENUM_NAME[parsed.buffers[b].dtype]
                           for b in parsed.outputs],
            "out_shapes": [list(s) for s in parsed.output_shapes],
            **meta}).encode(), np.uint8),
    }
    for i, u in enumerate(sem):
        out[f"out{i}"] = np.ascontiguousarray(np.atleast_1d(u)).view(np.uint8).reshape(-1)
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    return os.path.getsize(path), len(blob)


def main():
    sel = sys.argv[1:]
    total = 0
    for name in CASES:
        if sel and not any(s in name for s in sel):
            continue
        try:
            size, nblob = build(name)
        except Exception as e:                       # noqa: BLE001
            print(f"FAIL {name}: {type(e).__name__}: {e}")
            raise
        total += size
        print(f"{name:32s} blob {nblob:8d} B  fixture {size:9d} B")
    print(f"total {total / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
