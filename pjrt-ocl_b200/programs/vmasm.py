"""Tensor-level assembler for VMProgram v3 blobs, driving the reference's own
lowering context, fusion passes, scheduler and serializer.

This is build-time tooling, not part of the execution path: it needs the
reference's Python package (``pjrt_ocl``) on ``PYTHONPATH`` and is used to
produce (a) the committed ``*.vmprog`` blobs the benchmark executes and (b) the
golden fixtures of the parity tests.  Nothing here is imported at run time by
the CUDA backend.

Every method emits exactly the instruction pattern the reference's StableHLO
handler for the same op emits (cited per method, paths relative to the
reference's ``python/pjrt_ocl``), so that after the reference pass pipeline
(lowering.py:3039-3090) and ``schedule_program`` (scheduler.py:671-715) the
bytes are what its ``lower_service`` would hand the plugin for the equivalent
``jax.jit`` program.  The StableHLO front end itself (``lower_artifact``)
cannot be used because it needs ``jaxlib.mlir``.

Environment contract (scheduler.py:36-45): ``PJRT_OCL_EW_TS`` and
``PJRT_OCL_MMA_T`` are read when ``pjrt_ocl.scheduler`` is first imported and
must match the tile geometry the device backend advertises (4096 / 128).
"""
from __future__ import annotations

import dataclasses
import math
import os

os.environ.setdefault("PJRT_OCL_EW_TS", "4096")
os.environ.setdefault("PJRT_OCL_MMA_T", "128")

import numpy as np

import pjrt_ocl.ops  # noqa: F401  (registers TO_TASK / INTERP tables)
from pjrt_ocl import lowering as L
from pjrt_ocl import scheduler as S
from pjrt_ocl.ops import reduce as R

assert S.TILE_SIZE == 4096 and S.MMA_T == 128, (
    "pjrt_ocl.scheduler was imported before PJRT_OCL_EW_TS/MMA_T were set")

F32, I32, U32, BOOL, I64, F64, F16, BF16 = (
    L.DT_F32, L.DT_I32, L.DT_U32, L.DT_BOOL, L.DT_I64, L.DT_F64, L.DT_F16,
    L.DT_BF16)
SUM, MAX, MIN, PROD = R.SUM, R.MAX, R.MIN, R.PROD


def _strides(shape):
    out, acc = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        out[i] = acc
        acc *= shape[i]
    return out


@dataclasses.dataclass(eq=False)
class T:
    """An SSA tensor value: arena buffer id + static shape + dtype enum."""
    buf: int
    shape: tuple
    dtype: int

    @property
    def n(self) -> int:
        return math.prod(self.shape) if self.shape else 1


@dataclasses.dataclass(eq=False)
class ViewT(T):
    """A strided view of another tensor's buffer that has not been materialised:
    `buf` is the SOURCE buffer, `view` the descriptor [rank, dims, strides, offset]
    mapping the flat index of `shape` into it (the GATHER aux layout, ops/shape.py:
    57-84). Only ops that take operand views accept one (flash_attn)."""
    view: tuple = ()


class Asm:
    def __init__(self):
        self.ctx = L._Ctx()
        self._scalar_const: dict[int, float] = {}   # id(T) -> value
        self._scalar_bcast: dict[int, float] = {}
        self._keep: list = []                       # keep T objects alive (ids)
        self._in_region = False

    # -- values ---------------------------------------------------------
    def _new(self, shape, dtype) -> T:
        shape = tuple(int(d) for d in shape)
        t = T(self.ctx.new_buffer(math.prod(shape) if shape else 1, dtype),
              shape, dtype)
        self._keep.append(t)
        return t

    def input(self, shape, dtype=F32) -> T:
        """Program argument (lowering.py:2995-3000)."""
        t = self._new(shape, dtype)
        self.ctx.inputs.append(t.buf)
        self.ctx.input_shapes.append(t.shape)
        return t

    def const(self, value, dtype=F32, shape=None) -> T:
        """stablehlo.constant (lowering.py:552-585): const-pool entry; rank-0
        f32 constants are recorded for the affine fold."""
        arr = np.asarray(value, dtype=L.DTYPE_NUMPY[dtype])
        if shape is not None:
            arr = np.broadcast_to(arr, shape).copy()
        t = self._new(arr.shape, dtype)
        self.ctx.consts.append((t.buf, arr.reshape(-1).tobytes()))
        if t.n == 1 and dtype == F32:
            self._scalar_const[id(t)] = float(arr.reshape(-1)[0])
        return t

    def alias(self, x: T, shape) -> T:
        """stablehlo.reshape: same buffer, new shape (ops/shape.py:115-122)."""
        shape = tuple(int(d) for d in shape)
        assert math.prod(shape) == x.n, (shape, x.shape)
        t = T(x.buf, shape, x.dtype)
        self._keep.append(t)
        return t

    reshape = alias

    # -- shape ops (OP_GATHER_STRIDED) ------------------------------------
    def _gather(self, x: T, out_shape, out_strides, src_off=0) -> T:
        """ops/shape.py:57-84 `_emit_gather` incl. the identity-map alias."""
        from pjrt_ocl.ops.shape import _emit_gather
        buf = _emit_gather(self.ctx, tuple(out_shape), x.buf, list(out_strides),
                           src_off, dtype=x.dtype, in_n=x.n)
        t = T(buf, tuple(int(d) for d in out_shape), x.dtype)
        self._keep.append(t)
        return t

    def broadcast_in_dim(self, x: T, out_shape, dims) -> T:
        """ops/shape.py:87-112."""
        ins = _strides(x.shape)
        out_strides = [0] * len(out_shape)
        for in_axis, out_axis in enumerate(dims):
            if x.shape[in_axis] != 1:
                assert out_shape[out_axis] == x.shape[in_axis]
                out_strides[out_axis] = ins[in_axis]
        t = self._gather(x, out_shape, out_strides)
        if id(x) in self._scalar_const and all(s == 0 for s in out_strides):
            self._scalar_bcast[id(t)] = self._scalar_const[id(x)]
        return t

    def scalar(self, value, like: T) -> T:
        """A scalar constant broadcast to `like`'s shape (what jax emits for
        python scalars in arithmetic)."""
        c = self.const(value, like.dtype, shape=())
        return self.broadcast_in_dim(c, like.shape, [])

    def transpose(self, x: T, perm) -> T:
        """ops/shape.py:173-186."""
        ins = _strides(x.shape)
        out_shape = [x.shape[p] for p in perm]
        return self._gather(x, out_shape, [ins[p] for p in perm])

    def transpose_view(self, x: T, perm, reshape_to=None) -> ViewT:
        """The transpose as an operand view instead of a gather: nothing is emitted;
        the consumer reads `x`'s buffer through the strides. `reshape_to` regroups the
        transposed axes (same element order)."""
        ins = _strides(x.shape)
        dims = [x.shape[p] for p in perm]
        strides = [ins[p] for p in perm]
        shape = tuple(reshape_to) if reshape_to is not None else tuple(dims)
        assert math.prod(shape) == x.n
        t = ViewT(x.buf, shape, x.dtype, tuple([len(dims)] + dims + strides + [0]))
        self._keep.append(t)
        return t

    def slice(self, x: T, starts, limits, strides=None) -> T:
        """ops/shape.py:131-153."""
        strides = strides or [1] * len(x.shape)
        ins = _strides(x.shape)
        out_shape = [-(-(limits[d] - starts[d]) // strides[d])
                     for d in range(len(x.shape))]
        return self._gather(x, out_shape,
                            [ins[d] * strides[d] for d in range(len(x.shape))],
                            sum(starts[d] * ins[d] for d in range(len(x.shape))))

    def iota(self, shape, dim, dtype=F32) -> T:
        """ops/making.py:68-77."""
        from pjrt_ocl.ops.making import _emit_iota
        t = T(_emit_iota(self.ctx, tuple(shape), dim, dtype), tuple(shape), dtype)
        self._keep.append(t)
        return t

    # -- elementwise ------------------------------------------------------
    def binop(self, opcode, x: T, y: T) -> T:
        """lowering.py:512-544 (add/mul/sub with scalar-affine fold) and
        ops/elementwise.py:98-110 (all other binary ops)."""
        assert x.shape == y.shape and x.dtype == y.dtype, (x, y)
        if opcode in (L.OP_ADD_F32, L.OP_MUL_F32, L.OP_SUB_F32) and x.dtype == F32:
            r_s = self._scalar_bcast.get(id(y))
            l_s = self._scalar_bcast.get(id(x))
            if r_s is not None and l_s is None:
                s, t = L._affine_st(opcode, True, r_s)
                d = self._new(x.shape, F32)
                L.emit_affine(self.ctx, d.buf, x.buf, s, t, x.n)
                return d
            if l_s is not None and r_s is None:
                s, t = L._affine_st(opcode, False, l_s)
                d = self._new(x.shape, F32)
                L.emit_affine(self.ctx, d.buf, y.buf, s, t, x.n)
                return d
        d = self._new(x.shape, x.dtype)
        self.ctx.emit(L.Instr(opcode, dst=d.buf, a=x.buf, b=y.buf, n=x.n))
        return d

    def add(self, x, y): return self.binop(L.OP_ADD_F32, x, y)
    def sub(self, x, y): return self.binop(L.OP_SUB_F32, x, y)
    def mul(self, x, y): return self.binop(L.OP_MUL_F32, x, y)
    def div(self, x, y): return self.binop(L.OP_DIV_F32, x, y)
    def maximum(self, x, y): return self.binop(L.OP_MAX_F32, x, y)
    def minimum(self, x, y): return self.binop(L.OP_MIN_F32, x, y)
    def power(self, x, y): return self.binop(L.OP_POW_F32, x, y)
    def xor(self, x, y): return self.binop(L.OP_XOR, x, y)
    def and_(self, x, y): return self.binop(L.OP_AND, x, y)
    def or_(self, x, y): return self.binop(L.OP_OR, x, y)

    def unop(self, opcode, x: T) -> T:
        """ops/elementwise.py:113-122."""
        d = self._new(x.shape, x.dtype)
        self.ctx.emit(L.Instr(opcode, dst=d.buf, a=x.buf, b=0, n=x.n))
        return d

    def neg(self, x): return self.unop(L.OP_NEG_F32, x)
    def exp(self, x): return self.unop(L.OP_EXP_F32, x)
    def log(self, x): return self.unop(L.OP_LOG_F32, x)
    def sqrt(self, x): return self.unop(L.OP_SQRT_F32, x)
    def rsqrt(self, x): return self.unop(L.OP_RSQRT_F32, x)
    def tanh(self, x): return self.unop(L.OP_TANH_F32, x)

    def compare(self, x: T, y: T, direction: str) -> T:
        """ops/elementwise.py:349-365."""
        pred = {"EQ": 0, "NE": 1, "LT": 2, "LE": 3, "GT": 4, "GE": 5}[direction]
        d = self._new(x.shape, BOOL)
        self.ctx.emit(L.Instr(L.OP_CMP_F32, dst=d.buf, a=x.buf, b=y.buf, n=x.n,
                              imm=pred))
        return d

    def select(self, pred: T, on_true: T, on_false: T) -> T:
        """ops/elementwise.py:391-403."""
        d = self._new(on_true.shape, on_true.dtype)
        self.ctx.emit(L.Instr(L.OP_SELECT_F32, dst=d.buf, a=on_true.buf,
                              b=on_false.buf, n=on_true.n, imm=pred.buf))
        return d

    def convert(self, x: T, dtype) -> T:
        """ops/making.py:131-143."""
        if dtype == x.dtype:
            return x
        d = self._new(x.shape, dtype)
        self.ctx.emit(L.Instr(L.OP_CONVERT, dst=d.buf, a=x.buf, n=x.n))
        return d

    def bitcast(self, x: T, dtype) -> T:
        """ops/bitcast.py:25-39."""
        d = self._new(x.shape, dtype)
        self.ctx.emit(L.Instr(L.OP_BITCAST, dst=d.buf, a=x.buf, n=x.n))
        return d

    def copy(self, x: T) -> T:
        d = self._new(x.shape, x.dtype)
        self.ctx.emit(L.Instr(L.OP_COPY_F32, dst=d.buf, a=x.buf, n=x.n))
        return d

    def gelu_tanh(self, x: T) -> T:
        """jax.nn.gelu(approximate=True) as jax lowers it: the mul/affine/tanh
        chain `_fuse_gelu` (lowering.py:1737-1916) recognises for f32.  For
        2-byte floats the recognizer does not fire, so the fused OP_GELU is
        emitted directly."""
        if x.dtype != F32:
            d = self._new(x.shape, x.dtype)
            self.ctx.emit(L.Instr(L.OP_GELU, dst=d.buf, a=x.buf, b=x.buf, n=x.n))
            return d
        x3 = self.mul(self.mul(x, x), x)
        inner = self.add(x, self.mul(self.scalar(0.044715, x), x3))
        th = self.tanh(self.mul(self.scalar(0.7978845608, x), inner))
        return self.mul(self.mul(self.scalar(0.5, x), x),
                        self.add(self.scalar(1.0, x), th))

    def gelu_fused(self, x: T) -> T:
        """OP_GELU directly (what `_fuse_gelu` rewrites the chain above to)."""
        d = self._new(x.shape, x.dtype)
        self.ctx.emit(L.Instr(L.OP_GELU, dst=d.buf, a=x.buf, b=x.buf, n=x.n))
        return d

    # -- reductions -------------------------------------------------------
    def reduce(self, x: T, dims, kind=SUM) -> T:
        """ops/reduce.py:162-247: full reduce -> PART+COMB; innermost suffix ->
        OP_REDUCE_SEG; interior/prefix block -> OP_REDUCE_STRIDED."""
        dims = sorted(dims)
        rank = len(x.shape)
        if dims == list(range(rank)):
            n_parts = R._n_parts(x.n)
            part = self._new((n_parts,), x.dtype)
            self.ctx.emit(L.Instr(L.OP_REDUCE, dst=part.buf, a=x.buf, b=x.buf,
                                  n=x.n, imm=R._encode_imm(R.PHASE_PART, kind)))
            out = self._new((), x.dtype)
            self.ctx.emit(L.Instr(L.OP_REDUCE, dst=out.buf, a=part.buf,
                                  b=part.buf, n=n_parts,
                                  imm=R._encode_imm(R.PHASE_COMB, kind)))
            return out
        k, m = dims[0], len(dims)
        assert dims == list(range(k, k + m)), "contiguous axis block only"
        red = math.prod(x.shape[d] for d in dims)
        inner = math.prod(x.shape[k + m:]) if k + m < rank else 1
        out_shape = tuple(s for d, s in enumerate(x.shape) if d not in dims)
        out = self._new(out_shape, x.dtype)
        if inner == 1:
            self.ctx.emit(L.Instr(L.OP_REDUCE_SEG, dst=out.buf, a=x.buf, b=x.buf,
                                  n=out.n, imm=(kind << 28) | red))
        else:
            self.ctx.emit(L.Instr(L.OP_REDUCE_STRIDED, dst=out.buf, a=x.buf,
                                  b=x.buf, n=out.n, imm=(kind << 28) | red,
                                  imm2=inner))
        return out

    def reduce_window(self, x: T, window, strides=None, pad_low=None, pad_high=None, kind=SUM) -> T:
        """stablehlo.reduce_window without dilations (ops/reduce_window.py:104-145):
        OP_REDUCE_WINDOW with aux [kind, rank, out, win, stride, pad_low, in dims,
        in strides]; padding elements are the reduction's identity."""
        rank = len(x.shape)
        strides = list(strides or [1] * rank)
        pad_low = list(pad_low or [0] * rank)
        pad_high = list(pad_high or [0] * rank)
        out_shape = [(x.shape[d] + pad_low[d] + pad_high[d] - window[d]) // strides[d] + 1
                     for d in range(rank)]
        aux = ([kind, rank] + out_shape + list(window) + strides + pad_low
               + list(x.shape) + _strides(x.shape))
        d = self._new(out_shape, x.dtype)
        self.ctx.emit(L.Instr(L.OP_REDUCE_WINDOW, dst=d.buf, a=x.buf, n=d.n,
                              aux=self.ctx.add_aux(aux)))
        return d

    def gather_index(self, operand: T, indices: T, out_shape, op_stride, si_stride,
                     idx_op_stride, clamp_max, si_vec_stride=0) -> T:
        """stablehlo.gather as the reference plans it (ops/gather_index.py:128-143):
        OP_GATHER_INDEX with aux [out_rank, nidx, si_vec_stride, is64, 0, idx buffer,
        out dims, operand stride per out dim, indices stride per out dim, operand
        stride per index component, clamp per component]."""
        is64 = 1 if indices.dtype == I64 else 0
        aux = ([len(out_shape), len(idx_op_stride), si_vec_stride, is64, 0, indices.buf]
               + list(out_shape) + list(op_stride) + list(si_stride)
               + list(idx_op_stride) + list(clamp_max))
        d = self._new(out_shape, operand.dtype)
        self.ctx.emit(L.Instr(L.OP_GATHER_INDEX, dst=d.buf, a=operand.buf, n=d.n,
                              aux=self.ctx.add_aux(aux), reads_hint=(indices.buf,)))
        return d

    def take_rows(self, table: T, idx: T) -> T:
        """table[idx] for a 2-D table and a 1-D index vector (an embedding lookup):
        offset dim 1 walks a row, index component 0 picks it."""
        v, dcols = table.shape
        return self.gather_index(table, idx, (idx.shape[0], dcols), [0, 1], [1, 0],
                                 [dcols], [v - 1])

    def take_points(self, x: T, idx: T) -> T:
        """x[idx[:, 0], idx[:, 1]] for a 2-D x and an (n, 2) index matrix."""
        r, c = x.shape
        return self.gather_index(x, idx, (idx.shape[0],), [0], [2], [c, 1],
                                 [r - 1, c - 1], si_vec_stride=1)

    def scatter_index(self, operand: T, indices: T, updates: T, kind: int, op_stride,
                      si_stride, idx_op_stride, clamp_max, si_vec_stride=0) -> T:
        """stablehlo.scatter (ops/scatter_index.py:196-216): an identity-gather copy
        of the operand, then OP_SCATTER_INDEX combining the updates into it.
        kind: 0 set, 1 add, 2 max, 3 min."""
        is64 = 1 if indices.dtype == I64 else 0
        out = self._new(operand.shape, operand.dtype)
        caux = self.ctx.add_aux([len(operand.shape)] + list(operand.shape)
                                + _strides(operand.shape) + [0])
        self.ctx.emit(L.Instr(L.OP_GATHER_STRIDED, dst=out.buf, a=operand.buf,
                              n=operand.n, aux=caux))
        aux = ([len(updates.shape), len(idx_op_stride), si_vec_stride, is64, 0, indices.buf, kind]
               + list(updates.shape) + list(op_stride) + list(si_stride)
               + list(idx_op_stride) + list(clamp_max))
        self.ctx.emit(L.Instr(L.OP_SCATTER_INDEX, dst=out.buf, a=updates.buf,
                              n=updates.n, aux=self.ctx.add_aux(aux),
                              reads_hint=(indices.buf,)))
        return out

    def scatter_rows(self, table: T, idx: T, upd: T, kind: int) -> T:
        """table.at[idx].{set,add,max,min}(upd): 2-D table, 1-D indices, (n, cols) updates."""
        v, dcols = table.shape
        return self.scatter_index(table, idx, upd, kind, [0, 1], [1, 0], [dcols], [v - 1])

    def conv(self, x: T, w: T, strides=None, pad_low=None, pad_high=None, dilation=None) -> T:
        """stablehlo.convolution in the canonical layout (ops/conv.py:131-143):
        x [B, S..., Cin], w [W..., Cin, Cout] -> [B, O..., Cout], f32."""
        sdim = len(x.shape) - 2
        strides = list(strides or [1] * sdim)
        pad_low = list(pad_low or [0] * sdim)
        pad_high = list(pad_high or [0] * sdim)
        dilation = list(dilation or [1] * sdim)
        spatial, win = list(x.shape[1:1 + sdim]), list(w.shape[:sdim])
        cin, cout = x.shape[-1], w.shape[-1]
        assert w.shape[sdim] == cin
        out_sp = [(spatial[d] + pad_low[d] + pad_high[d] - (win[d] - 1) * dilation[d] - 1)
                  // strides[d] + 1 for d in range(sdim)]
        aux = [sdim, cin, cout] + out_sp + win + strides + pad_low + dilation + spatial
        d = self._new([x.shape[0]] + out_sp + [cout], F32)
        self.ctx.emit(L.Instr(L.OP_CONV, dst=d.buf, a=x.buf, b=w.buf, n=d.n,
                              aux=self.ctx.add_aux(aux)))
        return d

    def softmax_fused(self, x: T) -> T:
        """OP_SOFTMAX over the last axis (ops/reduce.py:478-491; emitted by
        `_fuse_norm`, lowering.py:1561-1730, for seg <= 1024 - here for any seg)."""
        seg = x.shape[-1]
        d = self._new(x.shape, x.dtype)
        self.ctx.emit(L.Instr(L.OP_SOFTMAX, dst=d.buf, a=x.buf, b=x.buf,
                              n=x.n // seg, imm=seg))
        return d

    def layernorm_fused(self, x: T, eps: float) -> T:
        """OP_LAYERNORM core over the last axis (ops/reduce.py:483-498)."""
        seg = x.shape[-1]
        d = self._new(x.shape, x.dtype)
        self.ctx.emit(L.Instr(L.OP_LAYERNORM, dst=d.buf, a=x.buf, b=x.buf,
                              n=x.n // seg, imm=seg, imm2=L._f32_bits(eps)))
        return d

    # -- contractions -----------------------------------------------------
    def dot_general(self, x: T, y: T, lb=(), lc=None, rb=(), rc=None,
                    out_dtype=F32) -> T:
        """ops/dot.py:94-162.  `out_dtype` other than f32 is an extension the
        bytecode already carries (task word0 dtype byte): the result buffer is
        typed `out_dtype` and both validators round on store."""
        from pjrt_ocl.ops.dot import _canonicalize
        lb, rb = list(lb), list(rb)
        lc = len(x.shape) - 1 if lc is None else lc
        rc = len(rb) if rc is None else rc
        nb = len(lb)
        assert len(rb) == nb
        xb, xs = _canonicalize(self.ctx, x.buf, x.shape, lb, lc, False)
        yb, ys = _canonicalize(self.ctx, y.buf, y.shape, rb, rc, True)
        if x.dtype != F32:
            # _canonicalize allocates f32 gather outputs; retype them.
            for b in (xb, yb):
                if b not in (x.buf, y.buf):
                    self._retype(b, x.dtype)
        G = math.prod(xs[:nb]) if nb else 1
        K = xs[-1]
        assert ys[nb] == K
        M = math.prod(xs[nb:-1]) if len(xs) - 1 > nb else 1
        N = math.prod(ys[nb + 1:]) if len(ys) > nb + 1 else 1
        assert N <= 0xFFFF and K <= 0xFFFF
        out_shape = tuple(xs[:nb]) + tuple(xs[nb:-1]) + tuple(ys[nb + 1:])
        d = self._new(out_shape, out_dtype)
        self.ctx.emit(L.Instr(L.OP_DOT, dst=d.buf, a=xb, b=yb, n=M,
                              imm=(N << 16) | K, imm2=G))
        return d

    def _retype(self, buf: int, dtype: int) -> None:
        b = self.ctx.buffers[buf]
        n = b.size_bytes // L.DTYPE_NUMPY[b.dtype].itemsize
        b.dtype = dtype
        b.size_bytes = n * L.DTYPE_NUMPY[dtype].itemsize

    def matmul(self, x: T, y: T, out_dtype=F32) -> T:
        return self.dot_general(x, y, out_dtype=out_dtype)

    def flash_attn(self, q: T, kT: T, v: T, scale: float, causal: bool,
                   out_dtype=None) -> T:
        """OP_FLASH_ATTN (ops/attention.py:1-25): q [H,T,hd], kT [H,hd,C]
        (the QK^T matmul's B operand), v [H,C,hd]; descriptor
        [H,T,C,hd,scale_bits,causal,qv,kv,vv] with contiguous operands."""
        H, Tq, hd = q.shape
        C = kT.shape[2]
        assert kT.shape == (H, hd, C) and v.shape == (H, C, hd)
        # operands given as views are read in place: descriptor words 6..8 hold 1 + the
        # aux offset of each operand's view (0 = contiguous), ops/attention.py:16-19
        views = [self.ctx.add_aux(list(o.view)) + 1 if isinstance(o, ViewT) else 0 for o in (q, kT, v)]
        aux = self.ctx.add_aux([H, Tq, C, hd, L._f32_bits(scale),
                                1 if causal else 0] + views)
        d = self._new((H, Tq, hd), q.dtype if out_dtype is None else out_dtype)
        self.ctx.emit(L.Instr(L.OP_FLASH_ATTN, dst=d.buf, a=q.buf, b=kT.buf,
                              n=H, imm=Tq, aux=aux, imm2=v.buf))
        return d

    # -- dynamic slicing / concatenation -------------------------------------
    def dynamic_slice(self, x: T, starts: list, sizes) -> T:
        """ops/dynslice.py:89-104."""
        from pjrt_ocl.ops.dynslice import _emit_dyn
        rank = len(x.shape)
        ins = _strides(x.shape)
        cmax = [x.shape[d] - sizes[d] for d in range(rank)]
        is64 = 1 if starts[0].dtype == I64 else 0
        d = self._new(sizes, x.dtype)
        _emit_dyn(self.ctx, L.OP_DYNAMIC_SLICE, list(sizes), ins, cmax,
                  [s.buf for s in starts], [0] * rank, is64, d.buf, x.buf, d.n)
        return d

    def dynamic_update_slice(self, x: T, upd: T, starts: list) -> T:
        """ops/dynslice.py:107-129 (identity-gather copy, then the scatter)."""
        from pjrt_ocl.ops.dynslice import _emit_dyn
        rank = len(x.shape)
        outs = _strides(x.shape)
        cmax = [x.shape[d] - upd.shape[d] for d in range(rank)]
        is64 = 1 if starts[0].dtype == I64 else 0
        d = self._new(x.shape, x.dtype)
        caux = self.ctx.add_aux([rank] + list(x.shape) + outs + [0])
        self.ctx.emit(L.Instr(L.OP_GATHER_STRIDED, dst=d.buf, a=x.buf, n=x.n,
                              aux=caux))
        _emit_dyn(self.ctx, L.OP_DYNAMIC_UPDATE_SLICE, list(upd.shape), outs,
                  cmax, [s.buf for s in starts], [0] * rank, is64, d.buf,
                  upd.buf, upd.n)
        return d

    def dynamic_update_in_place(self, x: T, upd: T, starts: list) -> T:
        """The scatter half of dynamic_update_slice alone, writing into `x`'s own
        buffer: what the reference's loop-carry fold leaves of a DUS whose operand
        is the carry (lowering.py:1126-1150, ops/dynslice.py:107-129 without the
        identity gather). Returns `x` (same buffer, now updated)."""
        from pjrt_ocl.ops.dynslice import _emit_dyn
        rank = len(x.shape)
        outs = _strides(x.shape)
        cmax = [x.shape[d] - upd.shape[d] for d in range(rank)]
        is64 = 1 if starts[0].dtype == I64 else 0
        _emit_dyn(self.ctx, L.OP_DYNAMIC_UPDATE_SLICE, list(upd.shape), outs,
                  cmax, [s.buf for s in starts], [0] * rank, is64, x.buf,
                  upd.buf, upd.n)
        return x

    def concatenate(self, xs: list, axis: int) -> T:
        """ops/concat.py: one OP_SCATTER per operand into a shared output,
        all tagged with the same `disjoint` group."""
        out_shape = list(xs[0].shape)
        out_shape[axis] = sum(x.shape[axis] for x in xs)
        d = self._new(out_shape, xs[0].dtype)
        outs = _strides(out_shape)
        group = d.buf + 1
        off = 0
        for x in xs:
            rank = len(x.shape)
            aux = self.ctx.add_aux([rank] + list(x.shape) + outs
                                   + [off * outs[axis]])
            self.ctx.emit(L.Instr(L.OP_SCATTER, dst=d.buf, a=x.buf, n=x.n,
                                  aux=aux, disjoint=group))
            off += x.shape[axis]
        return d

    # -- control flow ---------------------------------------------------------
    def fori_loop(self, trip: int, carries: list, body) -> list:
        """A counted loop as `_lower_while` + `_lower_while_regions` emit it in
        fixed-trip mode (lowering.py:936-996, 1017-1179): carries are copied
        into fresh loop buffers, the body is lowered after the root list, and
        each carry is committed in place when its producer is a lone
        elementwise op (lowering.py:1063-1101), else through the two-phase
        snapshot copy (lowering.py:1151-1168).  Must be called at top level;
        `body(asm, carries) -> new carries`."""
        assert not self._in_region
        cbufs = []
        for c in carries:
            cb = self._new(c.shape, c.dtype)
            self.ctx.emit(L.Instr(L.OP_COPY_F32, dst=cb.buf, a=c.buf, n=c.n))
            cbufs.append(cb)
        idx = len(self.ctx.instrs)
        self.ctx.emit(L.Instr(L.OP_NOP))
        self.ctx.region_queue.append((idx, trip, cbufs, body, None))
        return cbufs

    def while_loop(self, carries: list, cond, body) -> list:
        """Data-dependent loop (lowering.py:1017-1052 cond sub-list with the
        bool -> f32 flag convert, then the body as in `fori_loop`)."""
        assert not self._in_region
        cbufs = []
        for c in carries:
            cb = self._new(c.shape, c.dtype)
            self.ctx.emit(L.Instr(L.OP_COPY_F32, dst=cb.buf, a=c.buf, n=c.n))
            cbufs.append(cb)
        idx = len(self.ctx.instrs)
        self.ctx.emit(L.Instr(L.OP_NOP))
        self.ctx.region_queue.append((idx, None, cbufs, body, cond))
        return cbufs

    def _lower_regions(self) -> None:
        ctx = self.ctx
        self._in_region = True
        while ctx.region_queue:
            idx, trip, carry, body, cond = ctx.region_queue.pop(0)
            cond_start = len(ctx.instrs)
            cond_flag = 0
            if trip is None:
                c = cond(self, list(carry))
                flag = self._new((), F32)
                ctx.emit(L.Instr(L.OP_CONVERT, dst=flag.buf, a=c.buf, n=1))
                cond_flag = flag.buf
            cond_len = len(ctx.instrs) - cond_start
            body_start = len(ctx.instrs)
            rets = body(self, list(carry))
            assert len(rets) == len(carry)
            L._compose_affines(ctx)
            body_end0 = len(ctx.instrs)
            producer, dup, body_reads = {}, set(), {}
            for i in range(body_start, body_end0):
                bi = ctx.instrs[i]
                if bi.op == L.OP_NOP:
                    continue
                if bi.dst in producer:
                    dup.add(bi.dst)
                producer[bi.dst] = i
                for rb in L._reads_of(bi):
                    body_reads[rb] = body_reads.get(rb, 0) + 1
            carry_ids = {c.buf for c in carry}
            inplace = [False] * len(carry)
            for k, c in enumerate(carry):
                rb = rets[k].buf
                pidx = producer.get(rb)
                if pidx is None or rb in dup or rb in carry_ids:
                    continue
                prod = ctx.instrs[pidx]
                if prod.op not in L._EW_INPLACE_SAFE:
                    continue
                if body_reads.get(rb, 0) != 0:
                    continue
                others = body_reads.get(c.buf, 0) - (
                    1 if c.buf in L._reads_of(prod) else 0)
                if others != 0:
                    continue
                ctx.instrs[pidx] = dataclasses.replace(prod, dst=c.buf)
                inplace[k] = True
            skip = [rets[k].buf == carry[k].buf for k in range(len(carry))]
            temps = {}
            for k, c in enumerate(carry):
                if inplace[k] or skip[k]:
                    continue
                t = self._new(c.shape, c.dtype)
                ctx.emit(L.Instr(L.OP_COPY_F32, dst=t.buf, a=rets[k].buf, n=c.n))
                temps[k] = t
            for k, c in enumerate(carry):
                if inplace[k] or skip[k]:
                    continue
                ctx.emit(L.Instr(L.OP_COPY_F32, dst=c.buf, a=temps[k].buf, n=c.n))
            body_len = len(ctx.instrs) - body_start
            if trip is not None:
                ctx.instrs[idx] = L.Instr(L.OP_FOR, b=trip, n=body_start,
                                          imm=body_len)
            else:
                ctx.instrs[idx] = L.Instr(L.OP_WHILE, dst=cond_flag,
                                          a=cond_start, b=cond_len,
                                          n=body_start, imm=body_len)
        self._in_region = False

    # -- finish -----------------------------------------------------------
    def finish(self, outputs: list, *, nlanes: int, costs: dict | None = None,
               fold_2byte_views: bool = True, passes: bool = True,
               fold_2byte_matmul_views: bool = False):
        """Run the reference pass pipeline in its own order
        (lowering.py:3039-3090), schedule, serialize.  Returns (blob, program).

        `fold_2byte_views` additionally lets `_fuse_views` fold gathers into
        bf16/f16 elementwise consumers (the reference gates that fold on f32,
        lowering.py:1507,1529, although the bytecode and both validators are
        dtype-agnostic): the buffers' dtype tags are masked to f32 for the
        duration of that one pass.  `fold_2byte_matmul_views` does the same for
        `_fuse_matmul_views` (lowering.py:2381-2452): transposes feeding a bf16/f16
        dot_general become operand views of the matmul task instead of gathers."""
        ctx = self.ctx
        main_len = len(ctx.instrs)
        self._lower_regions()
        ctx.outputs = [o.buf for o in outputs]
        ctx.output_shapes = [o.shape for o in outputs]
        if passes:
            L._compose_affines(ctx)
            if fold_2byte_matmul_views:
                saved = [b.dtype for b in ctx.buffers]
                for b in ctx.buffers:
                    if b.dtype in (F16, BF16):
                        b.dtype = F32
                try:
                    L._fuse_matmul_views(ctx)
                finally:
                    for b, d in zip(ctx.buffers, saved):
                        b.dtype = d
            else:
                L._fuse_matmul_views(ctx)
            L._fuse_views(ctx)
            if fold_2byte_views:
                saved = [b.dtype for b in ctx.buffers]
                for b in ctx.buffers:
                    if b.dtype in (F16, BF16):
                        b.dtype = F32
                try:
                    L._fuse_views(ctx)
                finally:
                    for b, d in zip(ctx.buffers, saved):
                        b.dtype = d
            L._dce_nops(ctx)
            L._fuse_norm(ctx)
            L._fuse_gelu(ctx)
            L._fuse_region(ctx, main_len)
            L._dce_nops(ctx)
            L._fuse_mma_epilogue(ctx, main_len)
            L._dce_nops(ctx)
            L._fuse_attention(ctx, main_len)
            L._dce_nops(ctx)
            L._finalize_matmul_views(ctx)
            L._reuse_arena(ctx, main_len)
        prog = L.VMProgram(ctx._arena, ctx.buffers, ctx.inputs, ctx.outputs,
                           ctx.input_shapes, ctx.output_shapes, ctx.consts,
                           ctx.instrs, main_len, ctx.aux)
        sched = S.schedule_program(
            prog, S.DeviceConfig(nlanes=nlanes, costs=dict(costs or {})))
        return prog.serialize(sched), prog
