"""Python mirror of the reference's runtime interface over the C ABI (ctypes).

The class and method names follow the reference's C++ runtime
(pjrt_plugin/src/runtime.h): `VmProgram.Parse`, `OclRuntime.Create` (here
`Runtime.Create`), `LoadedProgram.Load / Execute / ExecuteDevice`, with the same
argument meaning and the same error behaviour (a failure raises `RuntimeError`
subclasses carrying the message the C++ side would have put in `*err`).

All computation happens in the native library (`libb2vm.so`: C++ host runtime +
the sm_100a megakernel).  There is no Python or CPU execution path: when the
library is missing, or no B200 is present, construction fails.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

# VMProgram dtype enum -> numpy dtype
def _np_dtypes():
    import ml_dtypes
    return {0: np.dtype("<f4"), 1: np.dtype("<i4"), 2: np.dtype("<u4"), 3: np.dtype("u1"),
            4: np.dtype("<i8"), 5: np.dtype("<f8"), 6: np.dtype("<f2"),
            7: np.dtype(ml_dtypes.bfloat16)}


class B2Error(RuntimeError):
    """Base of the errors the C ABI reports; `.code` is the b2_status value."""
    code = 13


class InvalidArgument(B2Error):
    code = 3


class DeadlineExceeded(B2Error):
    code = 4


class ResourceExhausted(B2Error):
    code = 8


class FailedPrecondition(B2Error):
    code = 9


class Unimplemented(B2Error):
    code = 12


class Internal(B2Error):
    code = 13


_BY_CODE = {c.code: c for c in (InvalidArgument, DeadlineExceeded, ResourceExhausted,
                                FailedPrecondition, Unimplemented, Internal)}


def find_library() -> str:
    """Search order mirrors the reference's `find_plugin_library`
    (python/pjrt_ocl/__init__.py:50-76): an explicit path in the environment
    (`B2VM_LIBRARY`), then the in-tree build next to this file."""
    env = os.environ.get("B2VM_LIBRARY")
    if env:
        return env
    return os.path.join(_HERE, "libb2vm.so")


class _DeviceInfo(ctypes.Structure):
    _fields_ = [("device_name", ctypes.c_char * 128), ("device_ordinal", ctypes.c_int),
                ("sm_count", ctypes.c_int), ("cc_major", ctypes.c_int), ("cc_minor", ctypes.c_int),
                ("total_mem_bytes", ctypes.c_uint64), ("lanes", ctypes.c_uint32),
                ("ew_ts", ctypes.c_uint32), ("mma_t", ctypes.c_uint32),
                ("threads_per_lane", ctypes.c_uint32)]


class _ExecStatus(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint32), ("lane", ctypes.c_uint32), ("where", ctypes.c_uint32),
                ("detail", ctypes.c_uint32), ("barriers", ctypes.c_uint64),
                ("device_ns", ctypes.c_uint64)]


_LIB = None
_ERRCAP = 512

# every entry point include/b2vm.h declares
EXPORTS = [
    "b2_runtime_create", "b2_runtime_destroy", "b2_runtime_info", "b2_alloc", "b2_free",
    "b2_h2d", "b2_d2h", "b2_program_parse", "b2_program_destroy", "b2_program_num_inputs",
    "b2_program_num_outputs", "b2_program_num_lanes", "b2_program_num_tasks",
    "b2_program_arena_bytes", "b2_program_io_bytes", "b2_program_io_dtype",
    "b2_program_io_rank", "b2_program_io_dim", "b2_program_load", "b2_loaded_destroy",
    "b2_loaded_program", "b2_execute_host", "b2_execute_device", "b2_execute_device_async",
    "b2_loaded_status", "b2_loaded_launch_count", "b2_loaded_set_wait_budget_ns",
    "b2_loaded_phase_ns", "b2_loaded_stat", "b2_sum_f32_static", "b2_sum_f32_static_max_elems",
    "b2_loaded_lane_timing", "b2_loaded_lane_times", "b2_loaded_in_out_result",
]


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = find_library()
    if not os.path.exists(path):
        raise FailedPrecondition(
            f"native library {path} not found: build it with "
            f"`python -c 'import __graft_entry__ as g; g.build()'` (there is no fallback path)")
    L = ctypes.CDLL(path)
    vp, cp, sz = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t
    pvp = ctypes.POINTER(ctypes.c_void_p)
    sig = {
        "b2_runtime_create": (ctypes.c_int, [ctypes.c_int, pvp, cp, sz]),
        "b2_runtime_destroy": (None, [vp]),
        "b2_runtime_info": (ctypes.c_int, [vp, ctypes.POINTER(_DeviceInfo)]),
        "b2_alloc": (ctypes.c_int, [vp, sz, pvp, cp, sz]),
        "b2_free": (ctypes.c_int, [vp, vp, sz]),
        "b2_h2d": (ctypes.c_int, [vp, vp, vp, sz, cp, sz]),
        "b2_d2h": (ctypes.c_int, [vp, vp, vp, sz, cp, sz]),
        "b2_program_parse": (ctypes.c_int, [cp, sz, pvp, cp, sz]),
        "b2_program_destroy": (None, [vp]),
        "b2_program_num_inputs": (ctypes.c_uint32, [vp]),
        "b2_program_num_outputs": (ctypes.c_uint32, [vp]),
        "b2_program_num_lanes": (ctypes.c_uint32, [vp]),
        "b2_program_num_tasks": (ctypes.c_uint32, [vp]),
        "b2_program_arena_bytes": (ctypes.c_uint64, [vp]),
        "b2_program_io_bytes": (ctypes.c_uint64, [vp, ctypes.c_int, ctypes.c_uint32]),
        "b2_program_io_dtype": (ctypes.c_uint32, [vp, ctypes.c_int, ctypes.c_uint32]),
        "b2_program_io_rank": (ctypes.c_uint32, [vp, ctypes.c_int, ctypes.c_uint32]),
        "b2_program_io_dim": (ctypes.c_int64, [vp, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32]),
        "b2_program_load": (ctypes.c_int, [vp, vp, pvp, cp, sz]),
        "b2_loaded_destroy": (None, [vp]),
        "b2_loaded_program": (vp, [vp]),
        "b2_execute_host": (ctypes.c_int, [vp, pvp, sz, pvp, sz, cp, sz]),
        "b2_execute_device": (ctypes.c_int, [vp, pvp, sz, pvp, sz, cp, sz]),
        "b2_execute_device_async": (ctypes.c_int, [vp, pvp, sz, pvp, sz, vp, cp, sz]),
        "b2_loaded_status": (ctypes.c_int, [vp, ctypes.POINTER(_ExecStatus), cp, sz]),
        "b2_loaded_launch_count": (ctypes.c_uint64, [vp]),
        "b2_loaded_set_wait_budget_ns": (None, [vp, ctypes.c_uint64]),
        "b2_loaded_phase_ns": (sz, [vp, ctypes.POINTER(ctypes.c_uint64), sz]),
        "b2_loaded_stat": (ctypes.c_uint64, [vp, ctypes.c_int]),
        "b2_loaded_lane_timing": (ctypes.c_int, [vp, ctypes.c_int, cp, sz]),
        "b2_loaded_lane_times": (sz, [vp, ctypes.POINTER(ctypes.c_uint64), sz]),
        "b2_loaded_in_out_result": (ctypes.c_int, [vp, ctypes.c_uint32]),
        "b2_sum_f32_static": (ctypes.c_int, [ctypes.c_int, vp, ctypes.c_uint64, vp, vp, cp, sz]),
        "b2_sum_f32_static_max_elems": (ctypes.c_uint64, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = L
    return L


def _check(status: int, err) -> None:
    if status != 0:
        raise _BY_CODE.get(status, Internal)(err.value.decode(errors="replace"))


def _errbuf():
    return ctypes.create_string_buffer(_ERRCAP)


class VmProgram:
    """A parsed VMProgram v3 (runtime.h:77-104). Host-only: needs no GPU."""

    def __init__(self, handle):
        self._h = handle
        L = lib()
        self.n_inputs = L.b2_program_num_inputs(handle)
        self.n_outputs = L.b2_program_num_outputs(handle)
        self.n_lanes = L.b2_program_num_lanes(handle)
        self.n_tasks = L.b2_program_num_tasks(handle)
        self.arena_bytes = L.b2_program_arena_bytes(handle)
        dts = _np_dtypes()

        def io(is_out, n):
            out = []
            for i in range(n):
                rank = L.b2_program_io_rank(handle, is_out, i)
                out.append({
                    "bytes": L.b2_program_io_bytes(handle, is_out, i),
                    "dtype": dts[L.b2_program_io_dtype(handle, is_out, i)],
                    "shape": tuple(L.b2_program_io_dim(handle, is_out, i, d) for d in range(rank)),
                })
            return out
        self.inputs = io(0, self.n_inputs)
        self.outputs = io(1, self.n_outputs)

    @staticmethod
    def Parse(blob: bytes) -> "VmProgram":
        """VmProgram::Parse (runtime.cc:90-251): raises InvalidArgument with the
        parser's message on a malformed blob."""
        L = lib()
        h = ctypes.c_void_p()
        err = _errbuf()
        _check(L.b2_program_parse(bytes(blob), len(blob), ctypes.byref(h), err, _ERRCAP), err)
        return VmProgram(h)

    def _release(self):
        h, self._h = self._h, None
        return h

    def __del__(self):
        if getattr(self, "_h", None):
            lib().b2_program_destroy(self._h)
            self._h = None


class Runtime:
    """One CUDA device + stream + buffer pool (OclRuntime, runtime.h:120-305)."""

    def __init__(self, handle):
        self._h = handle
        info = _DeviceInfo()
        lib().b2_runtime_info(handle, ctypes.byref(info))
        self.device_name = info.device_name.decode()
        self.device_ordinal = info.device_ordinal
        self.sm_count = info.sm_count
        self.compute_capability = (info.cc_major, info.cc_minor)
        self.total_mem_bytes = info.total_mem_bytes
        self.lanes = info.lanes                 # ngroups(): what PJRT_OCL_NLANES advertises
        self.ew_ts = info.ew_ts                 # ew_ts()
        self.mma_t = info.mma_t                 # mma_t()
        self.threads_per_lane = info.threads_per_lane

    @staticmethod
    def Create(device_ordinal: int = 0) -> "Runtime":
        L = lib()
        h = ctypes.c_void_p()
        err = _errbuf()
        _check(L.b2_runtime_create(device_ordinal, ctypes.byref(h), err, _ERRCAP), err)
        return Runtime(h)

    def AllocDevice(self, nbytes: int) -> int:
        p = ctypes.c_void_p()
        err = _errbuf()
        _check(lib().b2_alloc(self._h, nbytes, ctypes.byref(p), err, _ERRCAP), err)
        return p.value

    def PoolFree(self, dev_ptr: int, nbytes: int) -> None:
        lib().b2_free(self._h, ctypes.c_void_p(dev_ptr), nbytes)

    def WriteToDevice(self, dev_ptr: int, host: np.ndarray) -> None:
        a = np.ascontiguousarray(host)
        err = _errbuf()
        _check(lib().b2_h2d(self._h, ctypes.c_void_p(dev_ptr), ctypes.c_void_p(a.ctypes.data),
                            a.nbytes, err, _ERRCAP), err)

    def ReadFromDevice(self, dev_ptr: int, nbytes: int) -> np.ndarray:
        out = np.empty(max(1, nbytes), np.uint8)
        err = _errbuf()
        _check(lib().b2_d2h(self._h, ctypes.c_void_p(out.ctypes.data), ctypes.c_void_p(dev_ptr),
                            nbytes, err, _ERRCAP), err)
        return out[:nbytes]

    def SumF32Static(self, dev_in: int, n_elems: int, dev_out: int, stream: int = 0) -> None:
        """out[0] = sum of n_elems f32 at dev_in, through the entry point that
        allocates nothing (its scratch is an array built into the library; see
        include/b2vm.h for who needs that and for the size limit). Returns once
        the result is in dev_out."""
        err = _errbuf()
        _check(lib().b2_sum_f32_static(self.device_ordinal, ctypes.c_void_p(dev_in), n_elems,
                                       ctypes.c_void_p(dev_out), ctypes.c_void_p(stream), err, _ERRCAP), err)

    def close(self):
        if self._h:
            lib().b2_runtime_destroy(self._h)
            self._h = None


class LoadedProgram:
    """A program resident on the device (LoadedProgram, runtime.h:309-435)."""

    def __init__(self, rt: Runtime, handle, prog_view: VmProgram):
        self._rt = rt          # the runtime must outlive the loaded program (runtime.h:365)
        self._h = handle
        self.prog = prog_view

    @staticmethod
    def Load(rt: Runtime, prog: VmProgram) -> "LoadedProgram":
        """LoadedProgram::Load (runtime.cc:735-1074). Consumes `prog`."""
        L = lib()
        h = ctypes.c_void_p()
        err = _errbuf()
        _check(L.b2_program_load(rt._h, prog._h, ctypes.byref(h), err, _ERRCAP), err)
        prog._release()
        view = VmProgram(ctypes.c_void_p(L.b2_loaded_program(h)))
        view._h = None  # borrowed: owned by the loaded program
        return LoadedProgram(rt, h, view)

    def Execute(self, inputs, out=None) -> list:
        """Host arrays in, host arrays out (LoadedProgram::Execute,
        runtime.cc:1103-1177); synchronous. `out` may supply the result arrays
        (e.g. views of pinned memory) instead of fresh pageable ones."""
        p = self.prog
        if out is not None:
            return self._execute_into(inputs, out)
        if len(inputs) != p.n_inputs:
            raise InvalidArgument(f"Execute: got {len(inputs)} args, want {p.n_inputs}")
        keep = []
        for a, spec in zip(inputs, p.inputs):
            a = np.ascontiguousarray(a)
            if a.nbytes != spec["bytes"]:
                raise InvalidArgument(f"Execute: argument has {a.nbytes} bytes, buffer is {spec['bytes']}")
            keep.append(a)
        ins = (ctypes.c_void_p * max(1, p.n_inputs))(*[a.ctypes.data for a in keep])
        outs_np = [np.empty(max(1, s["bytes"]), np.uint8) for s in p.outputs]
        outs = (ctypes.c_void_p * max(1, p.n_outputs))(*[o.ctypes.data for o in outs_np])
        err = _errbuf()
        _check(lib().b2_execute_host(self._h, ins, p.n_inputs, outs, p.n_outputs, err, _ERRCAP), err)
        return [o[:s["bytes"]].view(s["dtype"]).reshape(s["shape"]) for o, s in zip(outs_np, p.outputs)]

    def _execute_into(self, inputs, out) -> list:
        p = self.prog
        if len(inputs) != p.n_inputs or len(out) != p.n_outputs:
            raise InvalidArgument(f"Execute: got {len(inputs)} args / {len(out)} results, "
                                  f"want {p.n_inputs} / {p.n_outputs}")
        for a, spec in zip(list(inputs) + list(out), p.inputs + p.outputs):
            if not a.flags["C_CONTIGUOUS"] or a.nbytes != spec["bytes"]:
                raise InvalidArgument("Execute: host buffers must be contiguous and of the buffer's size")
        ins = (ctypes.c_void_p * max(1, p.n_inputs))(*[a.ctypes.data for a in inputs])
        outs = (ctypes.c_void_p * max(1, p.n_outputs))(*[o.ctypes.data for o in out])
        err = _errbuf()
        _check(lib().b2_execute_host(self._h, ins, p.n_inputs, outs, p.n_outputs, err, _ERRCAP), err)
        return list(out)

    def ExecuteDevice(self, dev_inputs) -> list:
        """Device pointers in, freshly pooled device pointers out (caller owns;
        `Runtime.PoolFree`) - LoadedProgram::ExecuteDevice, runtime.cc:2107-2242."""
        p = self.prog
        ins = (ctypes.c_void_p * max(1, p.n_inputs))(*[int(x) for x in dev_inputs])
        outs = (ctypes.c_void_p * max(1, p.n_outputs))()
        err = _errbuf()
        _check(lib().b2_execute_device(self._h, ins, len(dev_inputs), outs, p.n_outputs, err, _ERRCAP), err)
        return [outs[i] for i in range(p.n_outputs)]

    def ExecuteDeviceAsync(self, dev_inputs, dev_outputs, stream: int = 0) -> None:
        """Enqueue on a CUDA stream into caller-provided result buffers, without
        waiting (see include/b2vm.h). Call `Status()` after synchronising."""
        p = self.prog
        ins = (ctypes.c_void_p * max(1, p.n_inputs))(*[int(x) for x in dev_inputs])
        outs = (ctypes.c_void_p * max(1, p.n_outputs))(*[int(x) for x in dev_outputs])
        err = _errbuf()
        _check(lib().b2_execute_device_async(self._h, ins, len(dev_inputs), outs, len(dev_outputs),
                                             ctypes.c_void_p(stream), err, _ERRCAP), err)

    def InOutResults(self) -> dict:
        """{argument index: result index} of the program's in/out buffers: pass the
        same device address for both and the buffer is updated in place."""
        pairs = {}
        for i in range(self.prog.n_inputs):
            o = lib().b2_loaded_in_out_result(self._h, i)
            if o >= 0:
                pairs[i] = int(o)
        return pairs

    def Status(self) -> dict:
        st = _ExecStatus()
        err = _errbuf()
        _check(lib().b2_loaded_status(self._h, ctypes.byref(st), err, _ERRCAP), err)
        return {"code": st.code, "lane": st.lane, "where": st.where, "detail": st.detail,
                "barriers": st.barriers, "device_ns": st.device_ns}

    def PhaseTimes(self) -> list:
        """ns since kernel entry at which each grid barrier of the last execute
        released (first 64 barriers): the end of each phase for every lane."""
        buf = (ctypes.c_uint64 * 64)()
        n = lib().b2_loaded_phase_ns(self._h, buf, 64)
        return [int(buf[i]) for i in range(n)]

    def LaneTiming(self, on: bool = True) -> None:
        """Switch per-lane timestamps on or off for the next executes."""
        err = _errbuf()
        _check(lib().b2_loaded_lane_timing(self._h, 1 if on else 0, err, _ERRCAP), err)

    def LaneReport(self) -> dict:
        """Per-phase wall time, arrival skew and mean idle of the last execute, and
        the mean lane utilisation over the launch - the figures the reference prints
        under PJRT_OCL_PHASE_TS (runtime.cc:2196-2240), from every lane's arrival
        time at every grid barrier. Empty when lane timing is off."""
        slots = 66
        n = self.prog.n_lanes * slots
        buf = (ctypes.c_uint64 * n)()
        got = lib().b2_loaded_lane_times(self._h, buf, n)
        if got != n:
            return {}
        t = np.frombuffer(buf, dtype=np.uint64).reshape(self.prog.n_lanes, slots).astype(np.int64)
        start = int(t[:, 0].min())
        phases, prev = [], start
        for b in range(64):
            arr = t[:, 2 + b]
            if not arr.all():
                break
            release = int(arr.max())
            phases.append({"wall_ns": release - prev, "skew_ns": release - int(arr.min()),
                           "idle_ns": float(release - arr.mean())})
            prev = release
        end = int(t[:, 1].max())
        tail = {"wall_ns": end - prev, "skew_ns": end - int(t[:, 1].min()), "idle_ns": float(end - t[:, 1].mean())}
        wall = sum(p["wall_ns"] for p in phases) + tail["wall_ns"]
        idle = sum(p["idle_ns"] for p in phases) + tail["idle_ns"]
        return {"phases": phases, "tail": tail, "total_ns": end - start,
                "mean_lane_util": 1.0 - idle / wall if wall else 0.0}

    _STATS = {"chains": 0, "forwarded": 0 + 1, "dead_stores": 2, "matmuls": 3, "tensor_core_matmuls": 4,
              "matmul_flops": 5, "flash": 6, "tensor_core_flash": 7, "spread_reductions": 8,
              "kernel_build": 9, "families": 10, "fused_full_reductions": 11, "decode_flash": 12,
              "in_out_ports": 13, "rebalanced_phases": 14, "row_pipelines": 15, "folded_converts": 16, "carried_sums": 17, "carried_barriers_removed": 18, "rms_rows": 19,
              "empty_phases_dropped": 20}

    def stat(self, name: str) -> int:
        """Load-time mapping facts, by name (see `_STATS`)."""
        return int(lib().b2_loaded_stat(self._h, self._STATS[name]))

    @property
    def launch_count(self) -> int:
        return lib().b2_loaded_launch_count(self._h)

    def set_wait_budget_ns(self, ns: int) -> None:
        lib().b2_loaded_set_wait_budget_ns(self._h, ns)

    def close(self):
        if self._h:
            lib().b2_loaded_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:      # noqa: BLE001
            pass
