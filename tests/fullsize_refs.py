"""Independent numpy restatements of the benchmark configurations' math, used to
check the device results at the sizes the benchmark times (where the C oracle, a
scalar interpreter, would take minutes per program).

They restate what the program builders in pjrt-ocl_b200/programs/cases.py
assemble - not the bytecode - with values rounded to the storage dtype where the
program stores them, f32 arithmetic in between (numpy float32 matmuls accumulate
in f32 like the device), so they also catch a wrongly assembled program. bf16
results are compared at rel 2e-2, measured against max(|want|, rms(want)): an
element close to zero in a tensor of O(1) values has no meaningful relative error
of its own (and see assert_close for the ten-per-million tail allowance on large
tensors). f32 results at rel 1e-5 on the same scale rule.
"""
from __future__ import annotations

import math

import ml_dtypes
import numpy as np

BF16 = ml_dtypes.bfloat16


def bf(x):
    """Round to bf16 storage, keep computing in f32."""
    return np.asarray(x, np.float32).astype(BF16).astype(np.float32)


def f32(x):
    return np.asarray(x).astype(np.float32)


def assert_close(got, want, rel, what, tail=1e-5):
    """|got - want| <= rel * max(|want|, rms(want)) element by element. On tensors of millions
    of elements that went through a dozen bf16 roundings a handful of elements land three
    bf16 steps (2.3 %) away from any restatement that rounds at slightly different points, so
    up to `tail` of the elements (10 per million) may exceed the bound, none by more than 2 x."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    scale = math.sqrt(float(np.mean(want * want))) if want.size else 0.0
    tol = rel * np.maximum(np.abs(want), scale)
    err = np.abs(got - want)
    bad = err > tol
    if bad.sum() <= tail * bad.size and not (err > 2.0 * tol).any():
        return
    if bad.any():
        i = np.unravel_index(np.argmax(np.abs(got - want) / np.maximum(tol, 1e-300)), got.shape)
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} elements beyond rel {rel} "
                             f"(worst at {i}: got {got[i]!r}, want {want[i]!r}, scale {scale:.3g})")


def gelu_tanh(x):
    x = f32(x)
    return (0.5 * x * (1.0 + np.tanh(np.float32(0.7978845608) * (x + np.float32(0.044715) * x * x * x)))).astype(np.float32)


def gelu_tanh_grad(z):
    z = f32(z)
    c, k = np.float32(0.7978845608), np.float32(0.044715)
    z2 = z * z
    t = np.tanh(c * (z + k * z2 * z))
    return (0.5 * (1.0 + t) + 0.5 * z * (1.0 - t * t) * (c * (1.0 + 3.0 * k * z2))).astype(np.float32)


def rmsnorm(x, gain, eps):
    xf = f32(x)
    ms = np.mean(xf.astype(np.float64) ** 2, axis=1, keepdims=True)
    return bf(xf * (1.0 / np.sqrt(ms + eps)).astype(np.float32) * f32(gain)[None, :])


# ---- config 3 -----------------------------------------------------------------------
def c3_forward_backward(x, y, w1, w2, w3, global_batch, cols):
    """Loss and the weight-gradient columns `cols` = (c1, c2, c3) index arrays of a
    (local) batch, MSE normalised by the global batch (cases.c3_mlp_step)."""
    X, Y, W1, W2, W3 = f32(x), f32(y), f32(w1), f32(w2), f32(w3)
    d3 = W3.shape[1]
    z1 = bf(X @ W1)
    h1 = bf(gelu_tanh(z1))
    z2 = bf(h1 @ W2)
    h2 = bf(gelu_tanh(z2))
    p = bf(h2 @ W3)
    diff = p - Y
    loss = float(np.sum(diff.astype(np.float64) ** 2) / (global_batch * d3))
    dp = bf(diff * np.float32(2.0 / (global_batch * d3)))
    c1, c2, c3 = cols
    dw3 = h2.T @ dp[:, c3]
    dh2 = bf(dp @ W3.T)
    dz2 = bf(gelu_tanh_grad(z2) * dh2)
    dw2 = h1.T @ dz2[:, c2]
    dh1 = bf(dz2 @ W2.T)
    dz1 = bf(gelu_tanh_grad(z1) * dh1)
    dw1 = X.T @ dz1[:, c1]
    return loss, dw1, dw2, dw3


# ---- config 5 -----------------------------------------------------------------------
def c5_block_sequence(x, g1, wq, wk, wv, wo, g2, w1, w2, heads, eps=1e-6):
    """One sequence (seq, d_model) through the pre-norm decoder block (cases.c5_block)."""
    seq, d = x.shape
    hd = d // heads
    h = rmsnorm(x, g1, eps)
    q, k, v = bf(h @ f32(wq)), bf(h @ f32(wk)), bf(h @ f32(wv))
    o = np.empty((seq, d), np.float32)
    mask = np.tril(np.ones((seq, seq), bool))
    for hh in range(heads):
        sl = slice(hh * hd, (hh + 1) * hd)
        s = (q[:, sl].astype(np.float64) @ k[:, sl].astype(np.float64).T) / math.sqrt(hd)
        s = np.where(mask, s, -np.inf)
        pm = np.exp(s - s.max(axis=1, keepdims=True))
        o[:, sl] = (pm / pm.sum(axis=1, keepdims=True)) @ v[:, sl].astype(np.float64)
    o = bf(o)
    x1 = bf(f32(x) + o @ f32(wo))
    h2 = rmsnorm(x1, g2, eps)
    f = bf(gelu_tanh(h2 @ f32(w1)))
    return bf(x1 + f @ f32(w2))


def c5_decode_step(x, kc, vc, g1, wq, wk, wv, wo, g2, w1, w2, heads, eps=1e-6):
    """One decode step (cases.c5_decode): returns y (batch, d), the new K and V rows
    (batch*heads, hd)."""
    batch, d = x.shape
    hd = d // heads
    H = batch * heads
    h = rmsnorm(x, g1, eps)
    q = bf(h @ f32(wq)).reshape(H, hd)
    k = bf(h @ f32(wk)).reshape(H, hd)
    v = bf(h @ f32(wv)).reshape(H, hd)
    kf = np.concatenate([f32(kc), k[:, None, :]], axis=1).astype(np.float64)     # (H, C, hd)
    vf = np.concatenate([f32(vc), v[:, None, :]], axis=1).astype(np.float64)
    s = np.einsum("hd,hcd->hc", q.astype(np.float64), kf) / math.sqrt(hd)
    pm = np.exp(s - s.max(axis=1, keepdims=True))
    o = bf(np.einsum("hc,hcd->hd", pm / pm.sum(axis=1, keepdims=True), vf)).reshape(batch, d)
    x1 = bf(f32(x) + o @ f32(wo))
    h2 = rmsnorm(x1, g2, eps)
    f = bf(gelu_tanh(h2 @ f32(w1)))
    return bf(x1 + f @ f32(w2)), k, v


# ---- one-call checks of a benchmark workload's outputs (bench.py's "verified" field) ------
def _as(raw, dtype, shape):
    return np.frombuffer(np.ascontiguousarray(raw).tobytes(), dtype=dtype).reshape(shape)


def verify_workload(program: str, args, outs, oracle_rows=None) -> str:
    """Check the host copies `outs` (raw byte arrays) of one step of `program` run on
    `args`. Returns a short description of what was compared; raises AssertionError on a
    mismatch. `oracle_rows(sample_program, x_rows, gamma, beta)` runs the C oracle on a row
    sample (config 2)."""
    if program.startswith("c2_int_chain"):
        a, b, c, d = args
        assert np.array_equal(_as(outs[0], np.int32, a.shape), np.maximum((a + b) ^ c, d))
        return "all elements bit-exact against numpy"
    if program.startswith("c2_chain"):
        x, gamma, beta = args
        two_byte = x.dtype.itemsize == 2
        dt = BF16 if two_byte else np.float32
        sm = _as(outs[0], dt, x.shape).astype(np.float32)
        rows = np.sort(np.random.default_rng(3).choice(x.shape[0], size=min(512, x.shape[0]), replace=False))
        if oracle_rows is not None and x.shape[0] >= 512:
            sample = "c2_chain_bf16_cpu_sample" if two_byte else "c2_chain_f32_cpu_sample"
            want = _as(oracle_rows(sample, x[rows], gamma, beta)[0], dt, (len(rows), x.shape[1])).astype(np.float32)
            rel = 2e-2 if two_byte else 1e-5
            assert np.all(np.abs(sm[rows] - want) <= rel * np.abs(want) + (1e-7 if two_byte else 1e-9))
        total = float(_as(outs[1], np.float32, (1,))[0])
        assert abs(total - sm.astype(np.float64).sum()) <= 1e-5 * x.shape[0]
        return f"{len(rows)} sampled rows against the oracle, scalar against the float64 sum"
    if program.startswith("c5_block"):
        g1, x, wq, wk, wv, wo, g2, w1, w2 = args
        seq, d = 2048, x.shape[1]
        nseq = x.shape[0] // seq
        got = _as(outs[0], BF16, (nseq, seq, d)).astype(np.float32)
        b = nseq - 1
        want = c5_block_sequence(x.reshape(nseq, seq, d)[b], g1, wq, wk, wv, wo, g2, w1, w2, heads=16)
        assert_close(got[b], want, 2e-2, f"sequence {b}")
        return f"sequence {b} of {nseq} against the numpy restatement (rel 2e-2)"
    if program.startswith("c5_decode_in_place"):
        g1, x, kc, vc, pos, wq, wk, wv, wo, g2, w1, w2 = args
        p_ = int(np.asarray(pos).reshape(-1)[0])
        assert p_ == kc.shape[1] - 1, "the restatement appends at the last position"
        want_y, k, v = c5_decode_step(x, kc[:, :p_], vc[:, :p_], g1, wq, wk, wv, wo, g2, w1, w2, heads=16)
        assert_close(_as(outs[0], BF16, x.shape).astype(np.float32), want_y, 2e-2, "decode y")
        for o, cache, row, what in ((outs[1], kc, k, "K"), (outs[2], vc, v, "V")):
            got = _as(o, BF16, cache.shape)
            assert np.array_equal(got[:, :p_].view(np.uint16), cache[:, :p_].view(np.uint16)), f"{what} cache rows below pos changed"
            assert_close(got[:, p_].astype(np.float32), row, 2e-2, f"{what} row written at pos")
        return "y, the K and V rows written in place at pos, and the untouched cache rows against the numpy restatement"
    if program.startswith("c5_decode"):
        g1, x, kc, vc, wq, wk, wv, wo, g2, w1, w2 = args
        want_y, k, v = c5_decode_step(x, kc, vc, g1, wq, wk, wv, wo, g2, w1, w2, heads=16)
        assert_close(_as(outs[0], BF16, x.shape).astype(np.float32), want_y, 2e-2, "decode y")
        kf = _as(outs[1], BF16, (kc.shape[0], kc.shape[1] + 1, kc.shape[2]))
        assert np.array_equal(kf[:, :-1].view(np.uint16), kc.view(np.uint16))
        assert_close(kf[:, -1].astype(np.float32), k, 2e-2, "appended K row")
        return "y, the appended K row and the moved cache against the numpy restatement"
    if program.startswith("c3_mlp_step"):
        x, y, w1, w2, w3 = args
        rng = np.random.default_rng(5)
        cols = (np.sort(rng.choice(w1.shape[1], 32, replace=False)), np.sort(rng.choice(w2.shape[1], 32, replace=False)),
                np.sort(rng.choice(w3.shape[1], 32, replace=False)))
        loss, dw1, dw2, dw3 = c3_forward_backward(x, y, w1, w2, w3, x.shape[0], cols)
        got_loss = float(_as(outs[0], np.float32, (1,))[0])
        assert abs(got_loss - loss) <= 2e-2 * abs(loss), (got_loss, loss)
        for o, w, dw, c in ((outs[1], w1, dw1, cols[0]), (outs[2], w2, dw2, cols[1]), (outs[3], w3, dw3, cols[2])):
            assert_close(_as(o, BF16, w.shape).astype(np.float32)[:, c], bf(f32(w)[:, c] - np.float32(1e-3) * dw), 2e-2, "updated weights")
        return "loss and 32 sampled columns of each updated weight against the numpy restatement"
    if program.startswith("dot_bf16"):
        x, w = args
        n = x.shape[0]
        got = _as(outs[0], BF16, (n, n)).astype(np.float64)
        rows = np.random.default_rng(7).choice(n, size=16, replace=False)
        want = x[rows].astype(np.float64) @ w.astype(np.float64)
        assert_close(got[rows], want, 2e-2, "sampled rows")
        return "16 sampled rows against a float64 dot"
    if program.startswith("flash_decode_bf16"):
        q, kc, vc = args
        H, C, hd = kc.shape
        got = _as(outs[0], BF16, (H, hd)).astype(np.float32)
        heads = np.sort(np.random.default_rng(9).choice(H, 32, replace=False))
        s = np.einsum("hd,hcd->hc", f32(q)[heads, 0].astype(np.float64), f32(kc)[heads].astype(np.float64)) / math.sqrt(hd)
        pm = np.exp(s - s.max(axis=1, keepdims=True))
        want = np.einsum("hc,hcd->hd", pm / pm.sum(axis=1, keepdims=True), f32(vc)[heads].astype(np.float64))
        assert_close(got[heads], want.astype(np.float32), 2e-2, "decode attention")
        return "32 sampled heads against float64 softmax(qK^T)V"
    if program.startswith("flash_bf16"):
        q, kt, v = args
        H, T, hd = q.shape
        got = _as(outs[0], BF16, (H, T, hd)).astype(np.float64)
        rng = np.random.default_rng(11)
        for h, m in zip(rng.integers(0, H, 12), list(rng.integers(0, T, 10)) + [0, T - 1]):
            s = (q[h, m].astype(np.float64) @ kt[h].astype(np.float64))[: m + 1] / np.sqrt(hd)
            pm = np.exp(s - s.max())
            want = (pm / pm.sum()) @ v[h, : m + 1].astype(np.float64)
            assert np.max(np.abs(got[h, m] - want) / (np.abs(want) + 2e-2)) < 2e-2, (h, m)
        return "12 sampled query rows against float64 softmax(QK^T)V"
    if program.startswith("c4_nbody"):
        pos0, vel0, mass = args
        pos = _as(outs[0], np.float32, pos0.shape).astype(np.float64)
        vel = _as(outs[1], np.float32, vel0.shape).astype(np.float64)
        assert np.isfinite(pos).all() and np.isfinite(vel).all()
        m = mass.astype(np.float64).reshape(-1, 1)
        p0, p1 = (m * vel0).sum(axis=0), (m * vel).sum(axis=0)
        assert np.all(np.abs(p1 - p0) <= 1e-3 * np.abs(m * vel).sum(axis=0)), "total momentum drifted"
        assert np.abs(pos - pos0).max() > 1e-3, "the system did not move"
        return "finite state, total momentum conserved over the 200 steps (1e-3 of the summed magnitudes), bodies moved"
    return ""
