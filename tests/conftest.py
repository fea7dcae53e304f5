"""Shared test plumbing: marker registration, fixture loading, comparison."""
from __future__ import annotations

import glob
import importlib
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
for p in (ROOT, os.path.join(ROOT, "pjrt-ocl_b200", "programs"), os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

import inputs as gen_inputs  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def package():
    """The backend package (its directory name is not a Python identifier)."""
    return importlib.import_module("pjrt-ocl_b200")


def golden_names():
    return sorted(os.path.basename(f)[:-4] for f in glob.glob(os.path.join(GOLDEN, "*.npz")))


class Golden:
    def __init__(self, name):
        z = np.load(os.path.join(GOLDEN, name + ".npz"))
        self.name = name
        self.meta = json.loads(bytes(z["meta"]))
        self.blob = bytes(z["blob"])
        self.args = gen_inputs.gen_all(self.meta["seed"], self.meta["items"])
        self.expected = []
        for i, (dt, shape) in enumerate(zip(self.meta["out_dtypes"], self.meta["out_shapes"])):
            self.expected.append(z[f"out{i}"].view(gen_inputs.DTYPES[dt]).reshape(shape))


def check_outputs(g: Golden, raw_outputs, what: str):
    """Compare raw uint8 output buffers against the fixture: integer, bool and
    index outputs (and every output of an `exact` case) bit-for-bit, float
    outputs within the fixture's tolerance (f32 rel 1e-5 class, bf16/f16 rel
    2e-2 class; the exact numbers are stored per case)."""
    assert len(raw_outputs) == len(g.expected)
    for i, (raw, exp) in enumerate(zip(raw_outputs, g.expected)):
        got = np.frombuffer(np.ascontiguousarray(raw).tobytes(), dtype=exp.dtype)
        got = got.reshape(exp.shape)
        label = f"{what}: {g.name} output {i} ({g.meta['out_dtypes'][i]}{list(exp.shape)})"
        if g.meta.get("exact") or g.meta["out_dtypes"][i] in ("i32", "u32", "i64", "bool"):
            np.testing.assert_array_equal(
                np.atleast_1d(got).view(np.uint8), np.atleast_1d(exp).view(np.uint8), err_msg=label)
        else:
            e = exp.astype(np.float64)
            gt = got.astype(np.float64)
            np.testing.assert_allclose(gt, e, rtol=g.meta.get("rtol", 1e-5),
                                       atol=g.meta.get("atol", 1e-5), err_msg=label)
