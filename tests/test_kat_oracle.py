"""The hand-encoded known-answer programs on the CPU oracle."""
import numpy as np
import pytest

import kat_programs as K
import vmoracle


def _check(out_raw, expected, rtol=0.0, atol=0.0):
    for raw, exp in zip(out_raw, expected):
        exp = np.asarray(exp)
        got = np.frombuffer(raw.tobytes(), exp.dtype).reshape(exp.shape)
        if rtol == 0.0 and atol == 0.0:
            np.testing.assert_array_equal(got, exp)
        else:
            np.testing.assert_allclose(got, exp, rtol=rtol, atol=atol)


@pytest.mark.parametrize("name", sorted(K.ALL))
def test_kat_on_oracle(name):
    blob, args, expected = K.ALL[name]()
    tol = dict(rtol=1e-5, atol=1e-5) if name == "C_region_gelu" else {}
    _check(vmoracle.Program(blob).execute(args), expected, **tol)


@pytest.mark.parametrize("flag", [1.0, 0.0])
def test_for_zero_trip_and_if_on_oracle(flag):
    blob, x, expected = K.kat_for_zero_trip_and_if()
    _check(vmoracle.Program(blob).execute([x, np.float32(flag)]), expected[flag])


@pytest.mark.parametrize("flag", [1.0, 0.0])
def test_strided_reduce_in_control_ranges_on_oracle(flag):
    blob, (x, z0), expected = K.kat_strided_reduce_in_control_ranges()
    _check(vmoracle.Program(blob).execute([x, np.float32(flag), z0]), expected[flag])
