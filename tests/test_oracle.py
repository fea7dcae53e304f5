"""Pins the C oracle (oracle/vmoracle.c) against the golden fixtures, i.e.
against the outputs of the reference's two numpy validators on blobs assembled
by the reference's own lowering + scheduler."""
import numpy as np
import pytest

from conftest import Golden, check_outputs, golden_names

import vmoracle


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_validators(name):
    g = Golden(name)
    prog = vmoracle.Program(g.blob, g.meta["ew_ts"], g.meta["mma_t"])
    out = prog.execute(g.args)
    check_outputs(g, out, "oracle")


def test_oracle_rejects_malformed_blobs():
    g = Golden("golden_layout_kat")
    bad_magic = b"XXXX" + g.blob[4:]
    with pytest.raises(vmoracle.OracleError, match="bad magic"):
        vmoracle.Program(bad_magic)
    bad_version = g.blob[:4] + (9).to_bytes(4, "little") + g.blob[8:]
    with pytest.raises(vmoracle.OracleError, match="unsupported version"):
        vmoracle.Program(bad_version)
    with pytest.raises(vmoracle.OracleError, match="trailing"):
        vmoracle.Program(g.blob + b"\0" * 8)
    with pytest.raises(vmoracle.OracleError):
        vmoracle.Program(g.blob[:100])


def test_oracle_threads_do_not_change_integer_results():
    g = Golden("c2_int_chain_small")
    prog = vmoracle.Program(g.blob)
    a = prog.execute(g.args, threads=1)
    b = prog.execute(g.args, threads=4)
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x, y)
