"""Program builders for the five benchmark configurations and for the op-family
parity cases.  Build-time only (needs the reference's Python package through
`vmasm`); the run-time side only ever sees the serialized blobs.

Each builder returns `(blob, prog, (seed, items))`; `inputs.gen_all(seed, items)`
yields the seeded numpy arguments in PJRT argument order.  Shapes, distributions and seeds
of the `c1..c5` builders are the benchmark's; every builder takes size
parameters so the parity tests can run reduced-size twins of the same graph.
"""
from __future__ import annotations

import math

import ml_dtypes
import numpy as np

from vmasm import (Asm, BF16, BOOL, F16, F32, I32, I64, MAX, MIN, PROD, SUM, U32,
                   L)

NP = {F32: np.float32, I32: np.int32, U32: np.uint32, BOOL: np.uint8,
      I64: np.int64, F16: np.float16, BF16: ml_dtypes.bfloat16}
DN = {F32: "f32", I32: "i32", U32: "u32", BOOL: "bool", I64: "i64",
      F16: "f16", BF16: "bf16"}
NLANES = 148
# The scheduler's per-tile cost table (scheduler.py:116-156; the reference's runtime
# supplies a calibrated one through PJRT_OCL_COST_TABLE) for this backend: microseconds
# one lane spends on a 4096-element elementwise / gather / reduce tile and on a
# 128 x 128 matmul tile of typical depth. With the all-ones default a matmul sharing a
# phase with an elementwise op would be given a fifth of the lanes.
B200_COSTS = {"ew_tile_us": 1.0, "gather_tile_us": 1.5, "reduce_tile_us": 1.0, "mma_tile_us": 20.0}


# --------------------------------------------------------------------------
# config 1: relu(a @ w)
# --------------------------------------------------------------------------
def c1_relu_matmul(M=256, K=128, N=64, nlanes=NLANES, dtype=F32):
    a_ = Asm()
    a = a_.input((M, K), dtype)
    w = a_.input((K, N), dtype)
    y = a_.matmul(a, w, out_dtype=dtype)
    zero = a_.scalar(0.0, y)
    out = a_.maximum(y, zero)
    blob, prog = a_.finish([out], nlanes=nlanes)

    return blob, prog, (0, [("normal", (M, K), DN[dtype]),
                            ("normal", (K, N), DN[dtype])])


def dot_general_square(n=8192, nlanes=NLANES, dtype=BF16, transpose_b=False):
    """One dot_general, n x n x n, for the matmul tile-op family on its own.
    `transpose_b`: y = x . w^T with w stored [n_out, n_in] (both operands k-contiguous)."""
    a_ = Asm()
    x = a_.input((n, n), dtype)
    w = a_.input((n, n), dtype)
    y = (a_.dot_general(x, w, lc=1, rc=1, out_dtype=dtype) if transpose_b
         else a_.matmul(x, w, out_dtype=dtype))
    blob, prog = a_.finish([y], nlanes=nlanes, fold_2byte_views=True)
    return blob, prog, (3, [("normal", (n, n), DN[dtype]), ("normal", (n, n), DN[dtype], 1.0 / n ** 0.5)])


def flash_only(H=128, T=2048, hd=64, causal=True, nlanes=NLANES, dtype=BF16):
    """Config 5's attention on its own: H = batch x heads, q [H,T,hd], k^T [H,hd,T], v [H,T,hd]."""
    a_ = Asm()
    q = a_.input((H, T, hd), dtype)
    kt = a_.input((H, hd, T), dtype)
    v = a_.input((H, T, hd), dtype)
    o = a_.flash_attn(q, kt, v, 1.0 / math.sqrt(hd), causal)
    blob, prog = a_.finish([o], nlanes=nlanes, costs=B200_COSTS)
    return blob, prog, (5, [("normal", (H, T, hd), DN[dtype]), ("normal", (H, hd, T), DN[dtype]),
                            ("normal", (H, T, hd), DN[dtype])])


def region_only(n=8192 * 4096, nlanes=NLANES):
    """One MAP_REGION over n f32 elements: the GELU derivative of config 3's backward pass
    (14 micro-ops, one input), for per-family numbers."""
    a_ = Asm()
    zf = a_.input((n,), F32)
    c, k = 0.7978845608, 0.044715
    z2 = a_.mul(zf, zf)
    u = a_.mul(a_.scalar(c, zf), a_.add(zf, a_.mul(a_.scalar(k, zf), a_.mul(z2, zf))))
    t = a_.tanh(u)
    sech2 = a_.sub(a_.scalar(1.0, t), a_.mul(t, t))
    du = a_.mul(a_.scalar(c, zf), a_.add(a_.scalar(1.0, zf), a_.mul(a_.scalar(3 * k, zf), z2)))
    g = a_.add(a_.mul(a_.scalar(0.5, t), a_.add(a_.scalar(1.0, t), t)),
               a_.mul(a_.mul(a_.scalar(0.5, zf), zf), a_.mul(sech2, du)))
    blob, prog = a_.finish([g], nlanes=nlanes, costs=B200_COSTS)
    return blob, prog, (7, [("normal", (n,), "f32")])


def flash_decode_only(H=512, C=2049, hd=64, nlanes=NLANES, dtype=BF16):
    """The attention of config 5's decode step on its own: one query row per head against
    a cache of C positions, K [H,C,hd] read through its transposed view, V [H,C,hd]."""
    a_ = Asm()
    q = a_.input((H, 1, hd), dtype)
    kc = a_.input((H, C, hd), dtype)
    vc = a_.input((H, C, hd), dtype)
    o = a_.flash_attn(q, a_.transpose_view(kc, [0, 2, 1]), vc, 1.0 / math.sqrt(hd), True)
    blob, prog = a_.finish([o], nlanes=nlanes, costs=B200_COSTS)
    return blob, prog, (6, [("normal", (H, 1, hd), DN[dtype]), ("normal", (H, C, hd), DN[dtype]),
                            ("normal", (H, C, hd), DN[dtype])])


# --------------------------------------------------------------------------
# config 2: LayerNorm -> tanh-GELU -> softmax -> full sum ; i32 add/xor/max
# --------------------------------------------------------------------------
def c2_chain(rows=8192, cols=4096, nlanes=NLANES, dtype=F32, fused=True,
             eps=1e-5):
    """f32 / bf16-storage chain.  `fused=True` uses the fused row ops
    (LAYERNORM_SEG / SOFTMAX_SEG / GELU) at this segment length; `fused=False`
    is the decomposed reduce+viewed-elementwise form jax's own lowering takes
    when the segment exceeds the reference's 1024 limit."""
    a_ = Asm()
    x = a_.input((rows, cols), dtype)
    gamma = a_.input((cols,), dtype)
    beta = a_.input((cols,), dtype)
    g2 = a_.broadcast_in_dim(gamma, (rows, cols), [1])
    b2 = a_.broadcast_in_dim(beta, (rows, cols), [1])
    if fused:
        core = a_.layernorm_fused(x, eps)
        y = a_.add(a_.mul(core, g2), b2)
        y = a_.gelu_tanh(y)
        sm = a_.softmax_fused(y)
    else:
        assert dtype == F32
        inv_n = a_.const(np.float32(1.0 / cols), F32, shape=())
        mean = a_.mul(a_.reduce(x, [1], SUM),
                      a_.broadcast_in_dim(inv_n, (rows,), []))
        xc = a_.sub(x, a_.broadcast_in_dim(mean, (rows, cols), [0]))
        var = a_.mul(a_.reduce(a_.mul(xc, xc), [1], SUM),
                     a_.broadcast_in_dim(inv_n, (rows,), []))
        rstd = a_.rsqrt(a_.add(var, a_.scalar(eps, var)))
        core = a_.mul(xc, a_.broadcast_in_dim(rstd, (rows, cols), [0]))
        y = a_.add(a_.mul(core, g2), b2)
        y = a_.gelu_tanh(y)
        mx = a_.reduce(y, [1], MAX)
        e = a_.exp(a_.sub(y, a_.broadcast_in_dim(mx, (rows, cols), [0])))
        den = a_.reduce(e, [1], SUM)
        sm = a_.div(e, a_.broadcast_in_dim(den, (rows, cols), [0]))
    if dtype == F32:
        total = a_.reduce(sm, [0, 1], SUM)
    else:
        # jax up-casts a 2-byte-float sum to f32 before reducing
        total = a_.reduce(a_.convert(sm, F32), [0, 1], SUM)
    blob, prog = a_.finish([sm, total], nlanes=nlanes)

    return blob, prog, (0, [("normal", (rows, cols), DN[dtype]),
                            ("normal", (cols,), DN[dtype], 0.1, 1.0),
                            ("normal", (cols,), DN[dtype], 0.1, 0.0)])


def c2_stage(stage, rows=8192, cols=4096, nlanes=NLANES, dtype=F32, eps=1e-5):
    """One stage of the config-2 chain as a program of its own."""
    a_ = Asm()
    x = a_.input((rows, cols), dtype)
    items = [("normal", (rows, cols), DN[dtype])]
    if stage == "layernorm":
        out = a_.layernorm_fused(x, eps)
    elif stage == "affine_gelu":
        gamma = a_.input((cols,), dtype)
        beta = a_.input((cols,), dtype)
        items += [("normal", (cols,), DN[dtype], 0.1, 1.0), ("normal", (cols,), DN[dtype], 0.1, 0.0)]
        y = a_.add(a_.mul(x, a_.broadcast_in_dim(gamma, (rows, cols), [1])),
                   a_.broadcast_in_dim(beta, (rows, cols), [1]))
        out = a_.gelu_tanh(y)
    elif stage == "softmax":
        out = a_.softmax_fused(x)
    elif stage == "sum":
        out = a_.reduce(x, [0, 1], SUM)
    else:
        raise ValueError(stage)
    blob, prog = a_.finish([out], nlanes=nlanes)
    return blob, prog, (0, items)


def c2_int_chain(rows=8192, cols=4096, nlanes=NLANES):
    """max((a + b) ^ c, d) on i32, bit-exact."""
    a_ = Asm()
    ins = [a_.input((rows, cols), I32) for _ in range(4)]
    out = a_.maximum(a_.xor(a_.add(ins[0], ins[1]), ins[2]), ins[3])
    blob, prog = a_.finish([out], nlanes=nlanes)

    return blob, prog, (0, [("int", (rows, cols), "i32", -2**20, 2**20)] * 4)


# --------------------------------------------------------------------------
# config 3: 3-layer MLP forward + grad of MSE + one SGD step
# --------------------------------------------------------------------------
def c3_mlp_step(batch=8192, widths=(1024, 4096, 4096, 1024), nlanes=NLANES,
                dtype=BF16, lr=1e-3, global_batch=None, apply_sgd=True, fold_transposes=True):
    """Storage `dtype`, f32 accumulate in every contraction.  Outputs: loss
    (f32 scalar) and either the three updated weights (`apply_sgd`) or the three
    weight gradients (for the data-parallel path, where the all-reduce sits
    between this program and the SGD program).  The MSE mean divides by
    `global_batch * widths[-1]` so shards sum to the global gradient."""
    d0, d1, d2, d3 = widths
    gb = batch if global_batch is None else global_batch
    a_ = Asm()
    x = a_.input((batch, d0), dtype)
    y = a_.input((batch, d3), dtype)
    w1 = a_.input((d0, d1), dtype)
    w2 = a_.input((d1, d2), dtype)
    w3 = a_.input((d2, d3), dtype)

    def gelu_fwd(z):
        return a_.gelu_tanh(z)

    def gelu_grad(z, dy):
        # d/dz [0.5 z (1 + tanh(u))],  u = c (z + k z^3)
        c, k = 0.7978845608, 0.044715
        zf = a_.convert(z, F32)
        z2 = a_.mul(zf, zf)
        u = a_.mul(a_.scalar(c, zf),
                   a_.add(zf, a_.mul(a_.scalar(k, zf), a_.mul(z2, zf))))
        t = a_.tanh(u)
        sech2 = a_.sub(a_.scalar(1.0, t), a_.mul(t, t))
        du = a_.mul(a_.scalar(c, zf),
                    a_.add(a_.scalar(1.0, zf), a_.mul(a_.scalar(3 * k, zf), z2)))
        g = a_.add(a_.mul(a_.scalar(0.5, t), a_.add(a_.scalar(1.0, t), t)),
                   a_.mul(a_.mul(a_.scalar(0.5, zf), zf), a_.mul(sech2, du)))
        return a_.convert(a_.mul(g, a_.convert(dy, F32)), dtype)

    z1 = a_.matmul(x, w1, out_dtype=dtype)
    h1 = gelu_fwd(z1)
    z2_ = a_.matmul(h1, w2, out_dtype=dtype)
    h2 = gelu_fwd(z2_)
    p = a_.matmul(h2, w3, out_dtype=dtype)
    diff = a_.sub(a_.convert(p, F32), a_.convert(y, F32))
    loss = a_.mul(a_.reduce(a_.mul(diff, diff), [0, 1], SUM),
                  a_.const(np.float32(1.0 / (gb * d3)), F32, shape=()))
    dp = a_.convert(a_.mul(diff, a_.scalar(2.0 / (gb * d3), diff)), dtype)
    # backward: dW = h^T @ dz (contract over batch), dX = dz @ W^T
    dw3 = a_.dot_general(h2, dp, lc=0, rc=0, out_dtype=F32)
    dh2 = a_.dot_general(dp, w3, lc=1, rc=1, out_dtype=dtype)
    dz2 = gelu_grad(z2_, dh2)
    dw2 = a_.dot_general(h1, dz2, lc=0, rc=0, out_dtype=F32)
    dh1 = a_.dot_general(dz2, w2, lc=1, rc=1, out_dtype=dtype)
    dz1 = gelu_grad(z1, dh1)
    dw1 = a_.dot_general(x, dz1, lc=0, rc=0, out_dtype=F32)
    if apply_sgd:
        outs = [loss]
        for w, dw in ((w1, dw1), (w2, dw2), (w3, dw3)):
            upd = a_.sub(a_.convert(w, F32), a_.mul(a_.scalar(lr, dw), dw))
            outs.append(a_.convert(upd, dtype))
    else:
        outs = [loss, dw1, dw2, dw3]
    # `fold_transposes`: the transposed operands of the backward contractions reach the matmul
    # tasks as operand views (what the reference's _fuse_matmul_views does for f32,
    # lowering.py:2381-2452) instead of materialised 2-byte transposes
    blob, prog = a_.finish(outs, nlanes=nlanes, costs=B200_COSTS, fold_2byte_matmul_views=fold_transposes)

    # x, y are drawn at the GLOBAL batch size; a data-parallel shard takes its
    # rows of them (the caller slices), weights are replicated.
    items = [("normal", (gb, d0), DN[dtype]), ("normal", (gb, d3), DN[dtype])]
    items += [("normal", (i, o), DN[dtype], 1.0 / math.sqrt(i))
              for i, o in ((d0, d1), (d1, d2), (d2, d3))]
    return blob, prog, (0, items)


def sgd_apply(shapes, nlanes=NLANES, dtype=BF16, lr=1e-3):
    """w <- w - lr * g for each (w, g) pair: the post-all-reduce half of the
    data-parallel config-3 step."""
    a_ = Asm()
    outs = []
    ws = [a_.input(s, dtype) for s in shapes]
    gs = [a_.input(s, F32) for s in shapes]
    for w, g in zip(ws, gs):
        upd = a_.sub(a_.convert(w, F32), a_.mul(a_.scalar(lr, g), g))
        outs.append(a_.convert(upd, dtype))
    blob, prog = a_.finish(outs, nlanes=nlanes, costs=B200_COSTS)
    return blob, prog, None


# --------------------------------------------------------------------------
# config 4: N-body, RK4, fori_loop
# --------------------------------------------------------------------------
def c4_nbody(n=4096, steps=200, nlanes=NLANES, dt=1e-3, soft=1e-2, seed=0):
    a_ = Asm()
    pos0 = a_.input((n, 3), F32)
    vel0 = a_.input((n, 3), F32)
    mass = a_.input((n,), F32)

    def accel(a, pos):
        # d[i,j,:] = pos[j] - pos[i]
        pj = a.broadcast_in_dim(pos, (n, n, 3), [1, 2])
        pi = a.broadcast_in_dim(pos, (n, n, 3), [0, 2])
        d = a.sub(pj, pi)
        r2 = a.reduce(a.mul(d, d), [2], SUM)                  # (n, n) seg 3
        r2 = a.add(r2, a.scalar(soft * soft, r2))
        inv3 = a.power(r2, a.scalar(-1.5, r2))
        w = a.mul(inv3, a.broadcast_in_dim(mass, (n, n), [1]))
        f = a.mul(d, a.broadcast_in_dim(w, (n, n, 3), [0, 1]))
        return a.reduce(f, [1], SUM)                          # (n, 3) strided

    def body(a, carry):
        pos, vel = carry
        h = a.scalar(dt, pos)
        h2 = a.scalar(dt / 2, pos)
        k1v = accel(a, pos)
        k1x = vel
        k2v = accel(a, a.add(pos, a.mul(h2, k1x)))
        k2x = a.add(vel, a.mul(h2, k1v))
        k3v = accel(a, a.add(pos, a.mul(h2, k2x)))
        k3x = a.add(vel, a.mul(h2, k2v))
        k4v = accel(a, a.add(pos, a.mul(h, k3x)))
        k4x = a.add(vel, a.mul(h, k3v))
        h6 = a.scalar(dt / 6, pos)
        two = a.scalar(2.0, pos)
        sx = a.add(a.add(k1x, a.mul(two, k2x)), a.add(a.mul(two, k3x), k4x))
        sv = a.add(a.add(k1v, a.mul(two, k2v)), a.add(a.mul(two, k3v), k4v))
        return [a.add(pos, a.mul(h6, sx)), a.add(vel, a.mul(h6, sv))]

    pos, vel = a_.fori_loop(steps, [pos0, vel0], body)
    blob, prog = a_.finish([pos, vel], nlanes=nlanes)

    return blob, prog, (seed, [("uniform", (n, 3), "f32", -1.0, 1.0),
                               ("normal", (n, 3), "f32", 0.1),
                               ("uniform", (n,), "f32", 0.5, 1.5)])


# --------------------------------------------------------------------------
# config 5: pre-norm decoder block (prefill) and a decode step
# --------------------------------------------------------------------------
def _rmsnorm(a, x, gain, eps):
    """RMSNorm over the last axis, f32 statistics, storage dtype in/out."""
    rows, d = x.shape
    xf = a.convert(x, F32)
    ms = a.mul(a.reduce(a.mul(xf, xf), [1], SUM),
               a.broadcast_in_dim(a.const(np.float32(1.0 / d), F32, shape=()),
                                  (rows,), []))
    r = a.rsqrt(a.add(ms, a.scalar(eps, ms)))
    y = a.mul(a.mul(xf, a.broadcast_in_dim(r, (rows, d), [0])),
              a.broadcast_in_dim(a.convert(gain, F32), (rows, d), [1]))
    return a.convert(y, x.dtype)


def c5_block(batch=8, seq=2048, d_model=1024, heads=16, d_ff=4096,
             nlanes=NLANES, dtype=BF16, eps=1e-6, attend_in_place=True):
    """Prefill: x (batch*seq, d_model) -> decoder block output, causal fused
    flash-attention over (batch*heads) heads. `attend_in_place`: the head split of the
    q / k / v projections reaches the attention op as operand views (the way the
    reference folds reshapes and transposes into matmul operands, lowering.py:2381-2452)
    instead of three materialised transposes."""
    hd = d_model // heads
    n = batch * seq
    a = Asm()
    # g1 is argument 0 on purpose: the reference's epilogue validator treats a
    # residual operand with buffer id 0 as "no residual" (ops/dot.py:262), and
    # x is folded into the output projection's epilogue as the residual.
    g1 = a.input((d_model,), dtype)
    x = a.input((n, d_model), dtype)
    wq = a.input((d_model, d_model), dtype)
    wk = a.input((d_model, d_model), dtype)
    wv = a.input((d_model, d_model), dtype)
    wo = a.input((d_model, d_model), dtype)
    g2 = a.input((d_model,), dtype)
    w1 = a.input((d_model, d_ff), dtype)
    w2 = a.input((d_ff, d_model), dtype)

    h = _rmsnorm(a, x, g1, eps)
    q = a.matmul(h, wq, out_dtype=dtype)
    k = a.matmul(h, wk, out_dtype=dtype)
    v = a.matmul(h, wv, out_dtype=dtype)
    # (b, s, H, hd) -> (b*H, s, hd) / K as (b*H, hd, s)
    q4 = a.reshape(q, (batch, seq, heads, hd))
    k4 = a.reshape(k, (batch, seq, heads, hd))
    v4 = a.reshape(v, (batch, seq, heads, hd))
    if attend_in_place:
        qh = a.transpose_view(q4, [0, 2, 1, 3], (batch * heads, seq, hd))
        kt = a.transpose_view(k4, [0, 2, 3, 1], (batch * heads, hd, seq))
        vh = a.transpose_view(v4, [0, 2, 1, 3], (batch * heads, seq, hd))
    else:
        qh = a.reshape(a.transpose(q4, [0, 2, 1, 3]), (batch * heads, seq, hd))
        kt = a.reshape(a.transpose(k4, [0, 2, 3, 1]), (batch * heads, hd, seq))
        vh = a.reshape(a.transpose(v4, [0, 2, 1, 3]), (batch * heads, seq, hd))
    o = a.flash_attn(qh, kt, vh, 1.0 / math.sqrt(hd), causal=True)
    o2 = a.reshape(a.transpose(a.reshape(o, (batch, heads, seq, hd)),
                               [0, 2, 1, 3]), (n, d_model))
    attn = a.matmul(o2, wo, out_dtype=dtype)
    x1 = a.add(x, attn)
    h2 = _rmsnorm(a, x1, g2, eps)
    f = a.gelu_tanh(a.matmul(h2, w1, out_dtype=dtype))
    y = a.add(x1, a.matmul(f, w2, out_dtype=dtype))
    blob, prog = a.finish([y], nlanes=nlanes, costs=B200_COSTS)

    d = DN[dtype]
    items = [("ones", (d_model,), d), ("normal", (n, d_model), d)]
    items += [("normal", (d_model, d_model), d, 0.02)] * 4
    items += [("ones", (d_model,), d), ("normal", (d_model, d_ff), d, 0.02),
              ("normal", (d_ff, d_model), d, 0.02)]
    return blob, prog, (0, items)


def c5_decode(batch=32, cache=2048, d_model=1024, heads=16, d_ff=4096,
              nlanes=NLANES, dtype=BF16, eps=1e-6):
    """One decode step: new token activations (batch, d_model), K/V caches
    (batch*heads, cache, hd) with the new position appended at the end
    (attention window = cache + 1 keys)."""
    hd = d_model // heads
    H = batch * heads
    C = cache + 1
    a = Asm()
    g1 = a.input((d_model,), dtype)     # argument 0: see c5_block
    x = a.input((batch, d_model), dtype)
    kc = a.input((H, cache, hd), dtype)
    vc = a.input((H, cache, hd), dtype)
    wq = a.input((d_model, d_model), dtype)
    wk = a.input((d_model, d_model), dtype)
    wv = a.input((d_model, d_model), dtype)
    wo = a.input((d_model, d_model), dtype)
    g2 = a.input((d_model,), dtype)
    w1 = a.input((d_model, d_ff), dtype)
    w2 = a.input((d_ff, d_model), dtype)

    h = _rmsnorm(a, x, g1, eps)
    q = a.reshape(a.matmul(h, wq, out_dtype=dtype), (H, 1, hd))
    k = a.reshape(a.matmul(h, wk, out_dtype=dtype), (H, 1, hd))
    v = a.reshape(a.matmul(h, wv, out_dtype=dtype), (H, 1, hd))
    kfull = a.concatenate([kc, k], axis=1)            # (H, C, hd)
    vfull = a.concatenate([vc, v], axis=1)
    kt = a.transpose(kfull, [0, 2, 1])                # (H, hd, C)
    o = a.flash_attn(q, kt, vfull, 1.0 / math.sqrt(hd), causal=True)
    o2 = a.reshape(o, (batch, d_model))
    x1 = a.add(x, a.matmul(o2, wo, out_dtype=dtype))
    h2 = _rmsnorm(a, x1, g2, eps)
    f = a.gelu_tanh(a.matmul(h2, w1, out_dtype=dtype))
    y = a.add(x1, a.matmul(f, w2, out_dtype=dtype))
    blob, prog = a.finish([y, kfull, vfull], nlanes=nlanes, costs=B200_COSTS)

    d = DN[dtype]
    items = [("ones", (d_model,), d), ("normal", (batch, d_model), d),
             ("normal", (H, cache, hd), d), ("normal", (H, cache, hd), d)]
    items += [("normal", (d_model, d_model), d, 0.02)] * 4
    items += [("ones", (d_model,), d), ("normal", (d_model, d_ff), d, 0.02),
              ("normal", (d_ff, d_model), d, 0.02)]
    return blob, prog, (0, items)


def c5_decode_in_place(batch=32, cache=2048, d_model=1024, heads=16, d_ff=4096,
                       nlanes=NLANES, dtype=BF16, eps=1e-6):
    """The decode step of `c5_decode` with the caches as in/out buffers of
    `cache + 1` positions: the new K/V rows are written at position `pos` by the
    scatter half of dynamic_update_slice alone (the reference's in-place DUS into a
    loop carry), K is read through a transposed view instead of being transposed,
    and the caches come back as results 1 and 2 (the same buffers)."""
    hd = d_model // heads
    H = batch * heads
    C = cache + 1
    a = Asm()
    g1 = a.input((d_model,), dtype)
    x = a.input((batch, d_model), dtype)
    kc = a.input((H, C, hd), dtype)
    vc = a.input((H, C, hd), dtype)
    pos = a.input((), I32)
    wq = a.input((d_model, d_model), dtype)
    wk = a.input((d_model, d_model), dtype)
    wv = a.input((d_model, d_model), dtype)
    wo = a.input((d_model, d_model), dtype)
    g2 = a.input((d_model,), dtype)
    w1 = a.input((d_model, d_ff), dtype)
    w2 = a.input((d_ff, d_model), dtype)
    zero = a.const(0, I32)

    h = _rmsnorm(a, x, g1, eps)
    q = a.reshape(a.matmul(h, wq, out_dtype=dtype), (H, 1, hd))
    k = a.reshape(a.matmul(h, wk, out_dtype=dtype), (H, 1, hd))
    v = a.reshape(a.matmul(h, wv, out_dtype=dtype), (H, 1, hd))
    kc = a.dynamic_update_in_place(kc, k, [zero, pos, zero])
    vc = a.dynamic_update_in_place(vc, v, [zero, pos, zero])
    kt = a.transpose_view(kc, [0, 2, 1])              # (H, hd, C) read in place
    o = a.flash_attn(q, kt, vc, 1.0 / math.sqrt(hd), causal=True)
    o2 = a.reshape(o, (batch, d_model))
    x1 = a.add(x, a.matmul(o2, wo, out_dtype=dtype))
    h2 = _rmsnorm(a, x1, g2, eps)
    f = a.gelu_tanh(a.matmul(h2, w1, out_dtype=dtype))
    y = a.add(x1, a.matmul(f, w2, out_dtype=dtype))
    blob, prog = a.finish([y, kc, vc], nlanes=nlanes, costs=B200_COSTS)

    d = DN[dtype]
    items = [("ones", (d_model,), d), ("normal", (batch, d_model), d),
             ("normal", (H, C, hd), d), ("normal", (H, C, hd), d),
             ("value", (), "i32", cache)]
    items += [("normal", (d_model, d_model), d, 0.02)] * 4
    items += [("ones", (d_model,), d), ("normal", (d_model, d_ff), d, 0.02),
              ("normal", (d_ff, d_model), d, 0.02)]
    return blob, prog, (0, items)
