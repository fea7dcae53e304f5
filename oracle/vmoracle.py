"""ctypes binding of the CPU oracle (oracle/vmoracle.c).

Test infrastructure: imported only by tests/, by `__graft_entry__.smoke()` and by
the benchmark's CPU-baseline legs, as the checker or the timed CPU arm - never
by the CUDA backend.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "libvmoracle.so")
    src = os.path.join(_HERE, "vmoracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libvmoracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        L.vmo_parse.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_uint32,
                                ctypes.c_uint32, ctypes.POINTER(ctypes.c_void_p),
                                ctypes.c_char_p, ctypes.c_size_t]
        L.vmo_execute.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                  ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                  ctypes.c_char_p, ctypes.c_size_t]
        L.vmo_free.argtypes = [ctypes.c_void_p]
        for f in ("vmo_n_inputs", "vmo_n_outputs", "vmo_n_lanes"):
            getattr(L, f).argtypes = [ctypes.c_void_p]
            getattr(L, f).restype = ctypes.c_uint32
        for f in ("vmo_input_bytes", "vmo_output_bytes"):
            getattr(L, f).argtypes = [ctypes.c_void_p, ctypes.c_uint32]
            getattr(L, f).restype = ctypes.c_uint64
        for f in ("vmo_input_dtype", "vmo_output_dtype"):
            getattr(L, f).argtypes = [ctypes.c_void_p, ctypes.c_uint32]
            getattr(L, f).restype = ctypes.c_uint32
        L.vmo_arena_bytes.argtypes = [ctypes.c_void_p]
        L.vmo_arena_bytes.restype = ctypes.c_uint64
        _LIB = L
    return _LIB


class OracleError(RuntimeError):
    pass


class Program:
    """A parsed + loaded VMProgram on the CPU oracle."""

    def __init__(self, blob: bytes, ew_ts: int = 4096, mma_t: int = 128):
        L = lib()
        err = ctypes.create_string_buffer(512)
        h = ctypes.c_void_p()
        if L.vmo_parse(blob, len(blob), ew_ts, mma_t, ctypes.byref(h), err, 512):
            raise OracleError(err.value.decode())
        self._h = h
        self.n_inputs = L.vmo_n_inputs(h)
        self.n_outputs = L.vmo_n_outputs(h)
        self.n_lanes = L.vmo_n_lanes(h)
        self.input_bytes = [L.vmo_input_bytes(h, i) for i in range(self.n_inputs)]
        self.output_bytes = [L.vmo_output_bytes(h, i) for i in range(self.n_outputs)]
        self.output_dtypes = [L.vmo_output_dtype(h, i) for i in range(self.n_outputs)]

    def execute(self, args, threads: int = 0):
        """args: arrays in argument order -> list of raw uint8 output arrays."""
        L = lib()
        if len(args) != self.n_inputs:
            raise OracleError(f"got {len(args)} args, want {self.n_inputs}")
        keep = [np.ascontiguousarray(a) for a in args]
        for a, nb in zip(keep, self.input_bytes):
            if a.nbytes != nb:
                raise OracleError(f"argument has {a.nbytes} bytes, buffer is {nb}")
        ins = (ctypes.c_void_p * max(1, self.n_inputs))(*[a.ctypes.data for a in keep])
        outs_np = [np.empty(max(1, nb), np.uint8) for nb in self.output_bytes]
        outs = (ctypes.c_void_p * max(1, self.n_outputs))(*[o.ctypes.data for o in outs_np])
        err = ctypes.create_string_buffer(512)
        if L.vmo_execute(self._h, ins, outs, threads, err, 512):
            raise OracleError(err.value.decode())
        return [o[:nb] for o, nb in zip(outs_np, self.output_bytes)]

    def close(self):
        if self._h:
            lib().vmo_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:      # noqa: BLE001
            pass
