"""The numpy restatements used by the full-size GPU checks (tests/fullsize_refs.py),
pinned on CPU against the reduced-size fixtures of the same graphs: they must
agree with what the reference validators produced there before they are trusted
at sizes the validators cannot reach."""
import numpy as np

import fullsize_refs as F
from conftest import Golden


def test_decoder_block_restatement_matches_the_small_fixture():
    g = Golden("c5_block_bf16_small")
    g1, x, wq, wk, wv, wo, g2, w1, w2 = g.args
    want = g.expected[0].astype(np.float32).reshape(2, 48, 128)
    for b in range(2):
        got = F.c5_block_sequence(x.reshape(2, 48, 128)[b], g1, wq, wk, wv, wo, g2, w1, w2, heads=4)
        F.assert_close(got, want[b], 2e-2, f"block sequence {b}")


def test_decode_restatement_matches_the_small_fixture():
    g = Golden("c5_decode_bf16_small")
    g1, x, kc, vc, wq, wk, wv, wo, g2, w1, w2 = g.args
    y, k, v = F.c5_decode_step(x, kc, vc, g1, wq, wk, wv, wo, g2, w1, w2, heads=4)
    F.assert_close(y, g.expected[0].astype(np.float32), 2e-2, "decode y")
    kfull = g.expected[1].astype(np.float32)
    vfull = g.expected[2].astype(np.float32)
    assert np.array_equal(kfull[:, :-1], kc.astype(np.float32)) and np.array_equal(vfull[:, :-1], vc.astype(np.float32))
    F.assert_close(k, kfull[:, -1], 2e-2, "new K row")
    F.assert_close(v, vfull[:, -1], 2e-2, "new V row")


def test_mlp_gradient_restatement_matches_the_small_fixture():
    g = Golden("c3_dp2_grads_f32_small")        # outputs: loss, dW1, dW2, dW3 of a 80-row shard of a 160-row batch
    x, y, w1, w2, w3 = g.args
    cols = (np.arange(256), np.arange(192), np.arange(64))
    # the fixture is f32 end to end; the restatement rounds activations to bf16, so compare at the bf16 class
    loss, dw1, dw2, dw3 = F.c3_forward_backward(x[:80], y[:80], w1, w2, w3, 160, cols)
    assert abs(loss - float(g.expected[0])) <= 2e-2 * abs(float(g.expected[0]))
    for got, want, what in ((dw1, g.expected[1], "dW1"), (dw2, g.expected[2], "dW2"), (dw3, g.expected[3], "dW3")):
        F.assert_close(got, want, 3e-2, what)
