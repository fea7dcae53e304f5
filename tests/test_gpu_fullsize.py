"""Full-size configurations on the GPU, checked by value on samples - the C oracle on
sampled rows where rows are independent, numpy restatements of the program builders
(tests/fullsize_refs.py) elsewhere - and through size-independent properties:
  * config 2 f32 / bf16 chains: 512 sampled rows against the oracle; the scalar against
    the float64 sum of the softmax;
  * config 3: loss, updated weights and (through the shard program) the weight gradients
    on sampled columns;
  * config 5: two whole sequences of the decoder block, and the decode step with its
    cache append;
  * config 2 i32 chain: bit-exact against numpy on all 33.5 M elements;
  * config 2 f32 chain: softmax rows are non-negative and sum to 1, the scalar equals
    their sum (= the row count);
  * dot_general bf16 4096^3: sampled rows against a float64 dot of the same bf16 inputs;
  * config 5's attention (128 heads x 2048 x 2048, causal, bf16): sampled query rows
    against a float64 softmax(QK^T)V;
  * config 4 (4096 bodies): two RK4 steps against a float64 recomputation; 200 steps
    conserve total momentum (pair forces are antisymmetric) and stay finite.
Tolerances: integer exact; f32 rel 1e-5 class; bf16 rel 2e-2."""
import gzip
import json
import os
import sys

import ml_dtypes
import numpy as np
import pytest

from conftest import package

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROG = os.path.join(ROOT, "pjrt-ocl_b200", "programs")
sys.path.insert(0, PROG)
import inputs as gen_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    vm = package()
    r = vm.Runtime.Create(0)
    yield r
    r.close()


def _run(rt, name):
    vm = package()
    man = json.load(open(os.path.join(PROG, "manifest.json")))[name]
    with gzip.open(os.path.join(PROG, name + ".vmprog.gz"), "rb") as f:
        blob = f.read()
    args = gen_inputs.gen_all(man["seed"], man["items"])
    lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(blob))
    outs = lp.Execute(args)
    st = lp.Status()
    lp.close()
    assert st["code"] == 0
    return args, outs


def test_config2_int_chain_is_bit_exact_at_full_size(rt):
    (a, b, c, d), (out,) = _run(rt, "c2_int_chain")
    want = np.maximum((a + b) ^ c, d)
    got = np.asarray(out).view(np.int32).reshape(want.shape)
    assert np.array_equal(got, want)


def _oracle_rows(sample_program, x_rows, gamma, beta):
    """The config-2 chain on a 512-row slice through the C oracle (rows are independent)."""
    import vmoracle
    with gzip.open(os.path.join(PROG, sample_program + ".vmprog.gz"), "rb") as f:
        blob = f.read()
    return vmoracle.Program(blob).execute([np.ascontiguousarray(x_rows), gamma, beta])


def test_config2_f32_chain_values_at_full_size(rt):
    """512 rows spread over the whole matrix against the oracle at rel 1e-5; the scalar
    against the float64 sum of the device's own softmax."""
    (x, gamma, beta), outs = _run(rt, "c2_chain_f32")
    sm = np.asarray(outs[0]).view(np.float32).reshape(8192, 4096)
    rows = np.sort(np.random.default_rng(3).choice(8192, size=512, replace=False))
    want = np.frombuffer(_oracle_rows("c2_chain_f32_cpu_sample", x[rows], gamma, beta)[0].tobytes(), np.float32).reshape(512, 4096)
    np.testing.assert_allclose(sm[rows], want, rtol=1e-5, atol=1e-9)
    total = float(np.asarray(outs[1]).view(np.float32).reshape(-1)[0])
    assert abs(total - sm.astype(np.float64).sum()) <= 1e-5 * 8192


def test_config2_bf16_chain_values_at_full_size(rt):
    (x, gamma, beta), outs = _run(rt, "c2_chain_bf16")
    sm = np.asarray(outs[0]).view(ml_dtypes.bfloat16).reshape(8192, 4096).astype(np.float32)
    rows = np.sort(np.random.default_rng(4).choice(8192, size=512, replace=False))
    raw = _oracle_rows("c2_chain_bf16_cpu_sample", x[rows], gamma, beta)[0]
    want = np.frombuffer(raw.tobytes(), ml_dtypes.bfloat16).reshape(512, 4096).astype(np.float32)
    # softmax values span many decades: relative to each value, with a floor far below the row's largest
    assert np.all(np.abs(sm[rows] - want) <= 2e-2 * np.abs(want) + 1e-7)
    total = float(np.asarray(outs[1]).view(np.float32).reshape(-1)[0])
    assert abs(total - sm.astype(np.float64).sum()) <= 1e-5 * 8192


def test_config3_step_and_gradients_at_full_size(rt):
    """The benchmarked step program (loss + updated weights) and, for the gradients it
    consumes internally, the data-parallel gradient program on a 4096-row shard: both
    against a numpy restatement on sampled weight columns."""
    import fullsize_refs as F
    rng = np.random.default_rng(5)
    cols = (np.sort(rng.choice(4096, 48, replace=False)), np.sort(rng.choice(4096, 48, replace=False)),
            np.sort(rng.choice(1024, 48, replace=False)))
    (x, y, w1, w2, w3), outs = _run(rt, "c3_mlp_step_bf16")
    loss, dw1, dw2, dw3 = F.c3_forward_backward(x, y, w1, w2, w3, 8192, cols)
    got_loss = float(np.asarray(outs[0]).view(np.float32).reshape(-1)[0])
    assert abs(got_loss - loss) <= 2e-2 * abs(loss), (got_loss, loss)
    for o, w, dw, c, what in ((outs[1], w1, dw1, cols[0], "W1"), (outs[2], w2, dw2, cols[1], "W2"), (outs[3], w3, dw3, cols[2], "W3")):
        got = np.asarray(o).view(ml_dtypes.bfloat16).reshape(w.shape).astype(np.float32)[:, c]
        F.assert_close(got, F.bf(F.f32(w)[:, c] - np.float32(1e-3) * dw), 2e-2, f"updated {what}")
    # gradients themselves: the shard program of the 2-GPU plan on rows 0..4095 (MSE over the global batch)
    vm = package()
    with gzip.open(os.path.join(PROG, "c3_mlp_grads_bf16_dp2.vmprog.gz"), "rb") as f:
        lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(f.read()))
    g = lp.Execute([np.ascontiguousarray(x[:4096]), np.ascontiguousarray(y[:4096]), w1, w2, w3])
    lp.close()
    loss, dw1, dw2, dw3 = F.c3_forward_backward(x[:4096], y[:4096], w1, w2, w3, 8192, cols)
    assert abs(float(np.asarray(g[0]).view(np.float32).reshape(-1)[0]) - loss) <= 2e-2 * abs(loss)
    for o, w, dw, c, what in ((g[1], w1, dw1, cols[0], "dW1"), (g[2], w2, dw2, cols[1], "dW2"), (g[3], w3, dw3, cols[2], "dW3")):
        F.assert_close(np.asarray(o).view(np.float32).reshape(w.shape)[:, c], dw, 2e-2, what)


def test_config5_block_values_at_full_size(rt):
    """Two of the eight sequences (2048 tokens each) against the numpy restatement of the block."""
    import fullsize_refs as F
    (g1, x, wq, wk, wv, wo, g2, w1, w2), (y,) = _run(rt, "c5_block_bf16")
    got = np.asarray(y).view(ml_dtypes.bfloat16).reshape(8, 2048, 1024).astype(np.float32)
    xs = x.reshape(8, 2048, 1024)
    for b in (0, 5):
        want = F.c5_block_sequence(xs[b], g1, wq, wk, wv, wo, g2, w1, w2, heads=16)
        F.assert_close(got[b], want, 2e-2, f"sequence {b}")


def test_config5_decode_values_at_full_size(rt):
    import fullsize_refs as F
    (g1, x, kc, vc, wq, wk, wv, wo, g2, w1, w2), (y, kfull, vfull) = _run(rt, "c5_decode_bf16")
    want_y, k, v = F.c5_decode_step(x, kc, vc, g1, wq, wk, wv, wo, g2, w1, w2, heads=16)
    kf = np.asarray(kfull).view(ml_dtypes.bfloat16).reshape(512, 2049, 64)
    vf = np.asarray(vfull).view(ml_dtypes.bfloat16).reshape(512, 2049, 64)
    assert np.array_equal(kf[:, :2048].view(np.uint16), kc.view(np.uint16))      # the cache is moved bit for bit
    assert np.array_equal(vf[:, :2048].view(np.uint16), vc.view(np.uint16))
    F.assert_close(kf[:, 2048].astype(np.float32), k, 2e-2, "appended K row")
    F.assert_close(vf[:, 2048].astype(np.float32), v, 2e-2, "appended V row")
    F.assert_close(np.asarray(y).view(ml_dtypes.bfloat16).reshape(32, 1024).astype(np.float32), want_y, 2e-2, "decode y")


def test_config5_decode_in_place_values_at_full_size(rt):
    """The in-place decode step through the allocating entry point (argument and result
    differ: the caches are copied into the results, then updated there)."""
    import fullsize_refs as F
    args, outs = _run(rt, "c5_decode_in_place_bf16")
    what = F.verify_workload("c5_decode_in_place_bf16", args, [np.asarray(o).view(np.uint8).reshape(-1) for o in outs])
    assert "in place" in what


def test_config2_f32_chain_properties_at_full_size(rt):
    _, outs = _run(rt, "c2_chain_f32")
    sm = np.asarray(outs[0]).view(np.float32).reshape(8192, 4096)
    total = float(np.asarray(outs[1]).view(np.float32).reshape(-1)[0])
    assert np.isfinite(sm).all() and (sm >= 0).all()
    rows = sm.astype(np.float64).sum(axis=1)
    assert np.max(np.abs(rows - 1.0)) < 1e-4          # every softmax row sums to 1
    assert abs(total - rows.sum()) / 8192.0 < 1e-5     # the full sum is the sum of the rows (~8192)


def test_dot_bf16_4096_sampled_rows(rt):
    (x, w), (y,) = _run(rt, "dot_bf16_4096")
    got = np.asarray(y).view(ml_dtypes.bfloat16).reshape(4096, 4096).astype(np.float64)
    rows = np.random.default_rng(7).choice(4096, size=16, replace=False)
    want = x[rows].astype(np.float64) @ w.astype(np.float64)
    err = np.abs(got[rows] - want)
    assert np.max(err / (np.abs(want) + 2e-2)) < 2e-2


def test_flash_attention_c5_sampled_rows(rt):
    (q, kt, v), (o,) = _run(rt, "flash_bf16_c5")
    H, T, hd = q.shape
    got = np.asarray(o).view(ml_dtypes.bfloat16).reshape(H, T, hd).astype(np.float64)
    rng = np.random.default_rng(11)
    for h, m in zip(rng.integers(0, H, 12), list(rng.integers(0, T, 10)) + [0, T - 1]):
        s = (q[h, m].astype(np.float64) @ kt[h].astype(np.float64))[: m + 1] / np.sqrt(hd)   # causal: keys 0..m
        p = np.exp(s - s.max())
        want = (p / p.sum()) @ v[h, : m + 1].astype(np.float64)
        assert np.max(np.abs(got[h, m] - want) / (np.abs(want) + 2e-2)) < 2e-2, (h, m)


def _nbody_accel64(pos, mass, soft=1e-2, block=512):
    acc = np.empty_like(pos)
    for i0 in range(0, pos.shape[0], block):
        d = pos[None, :, :] - pos[i0:i0 + block, None, :]              # d[i, j] = pos[j] - pos[i]
        r2 = (d * d).sum(axis=2) + soft * soft
        w = r2 ** -1.5 * mass[None, :]
        acc[i0:i0 + block] = (d * w[:, :, None]).sum(axis=1)
    return acc


def _nbody_rk4_64(pos, vel, mass, steps, dt=1e-3):
    for _ in range(steps):
        k1v, k1x = _nbody_accel64(pos, mass), vel
        k2v, k2x = _nbody_accel64(pos + dt / 2 * k1x, mass), vel + dt / 2 * k1v
        k3v, k3x = _nbody_accel64(pos + dt / 2 * k2x, mass), vel + dt / 2 * k2v
        k4v, k4x = _nbody_accel64(pos + dt * k3x, mass), vel + dt * k3v
        pos = pos + dt / 6 * (k1x + 2 * k2x + 2 * k3x + k4x)
        vel = vel + dt / 6 * (k1v + 2 * k2v + 2 * k3v + k4v)
    return pos, vel


def test_config4_two_steps_match_float64_at_full_size(rt):
    (pos0, vel0, mass), outs = _run(rt, "c4_nbody_2steps")
    pos = np.asarray(outs[0]).view(np.float32).reshape(4096, 3)
    vel = np.asarray(outs[1]).view(np.float32).reshape(4096, 3)
    want_p, want_v = _nbody_rk4_64(pos0.astype(np.float64), vel0.astype(np.float64), mass.astype(np.float64), 2)
    # f32 sums of 4096 pair terms per body: rel 1e-5 class on the accelerations, which enter
    # the velocities scaled by dt = 1e-3
    np.testing.assert_allclose(pos, want_p, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(vel, want_v, rtol=1e-4, atol=1e-5 * np.abs(want_v).max())


def test_config4_200_steps_conserve_momentum(rt):
    (pos0, vel0, mass), outs = _run(rt, "c4_nbody")
    pos = np.asarray(outs[0]).view(np.float32).reshape(4096, 3).astype(np.float64)
    vel = np.asarray(outs[1]).view(np.float32).reshape(4096, 3).astype(np.float64)
    assert np.isfinite(pos).all() and np.isfinite(vel).all()
    m = mass.astype(np.float64)[:, None]
    p0, p1 = (m * vel0).sum(axis=0), (m * vel).sum(axis=0)
    scale = np.abs(m * vel).sum(axis=0)
    assert np.all(np.abs(p1 - p0) <= 1e-3 * scale), (p0, p1, scale)
    assert np.abs(pos - pos0).max() > 1e-3          # the system moved
