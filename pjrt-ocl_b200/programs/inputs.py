"""Seeded input generation shared by the fixture generator, the tests and the
benchmark.

A program's arguments are described by `(seed, items)`: one
`numpy.random.default_rng(seed)` stream from which the items are drawn in
argument order.  Each item is `(kind, shape, dtype_name, *params)`.  The
generator streams are stable across machines for a given numpy version.
"""
from __future__ import annotations

import ml_dtypes
import numpy as np

DTYPES = {
    "f32": np.float32, "i32": np.int32, "u32": np.uint32, "bool": np.uint8,
    "i64": np.int64, "f64": np.float64, "f16": np.float16,
    "bf16": ml_dtypes.bfloat16,
}
# VMProgram dtype enum -> name (f32 0, i32 1, u32 2, bool 3, i64 4, f64 5,
# f16 6, bf16 7)
ENUM_NAME = ["f32", "i32", "u32", "bool", "i64", "f64", "f16", "bf16"]


def gen_item(rng, item):
    kind, shape, dt = item[0], tuple(item[1]), item[2]
    p = list(item[3:])
    npdt = DTYPES[dt]
    if kind == "normal":          # params: scale, shift
        scale = p[0] if len(p) > 0 else 1.0
        shift = p[1] if len(p) > 1 else 0.0
        v = rng.standard_normal(shape).astype(np.float32)
        v = v * np.float32(scale) + np.float32(shift)
        return v.astype(np.float32).astype(npdt)
    if kind == "uniform":         # params: lo, hi
        return rng.uniform(p[0], p[1], shape).astype(np.float32).astype(npdt)
    if kind == "int":             # params: lo, hi (hi exclusive)
        return rng.integers(int(p[0]), int(p[1]), size=shape,
                            dtype=np.int64).astype(npdt)
    if kind == "perm":            # params: n; the first prod(shape) entries of a permutation of range(n)
        count = int(np.prod(shape)) if shape else 1
        return rng.permutation(int(p[0]))[:count].reshape(shape).astype(npdt)
    if kind == "ones":
        return np.ones(shape, np.float32).astype(npdt)
    if kind == "value":           # params: the scalar value
        return np.full(shape, p[0]).astype(npdt)
    raise ValueError(f"unknown input item kind {kind!r}")


def gen_all(seed, items):
    rng = np.random.default_rng(int(seed))
    return [gen_item(rng, tuple(it)) for it in items]
