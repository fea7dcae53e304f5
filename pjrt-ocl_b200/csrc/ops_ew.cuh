// Elementwise tile op (TILE_EW) and fused lane-local chains of them.
//
// Replaces vmo_ew_tile and its per-dtype bodies (pjrt_plugin/kernels/ops/ew.cl:
// 226-658), compare/select/convert/bitcast/is_finite (ew.cl:71-127,532-636).
// Numeric conventions follow the reference's numpy validators
// (python/pjrt_ocl/ops/elementwise.py:213-266,281-286,314-319,373-430;
// ops/making.py:146-160; ops/bitcast.py:47-51).
//
// B200 design: a lane gets a contiguous element range [tile_lo*TS, tile_hi*TS);
// every thread owns groups of 4 consecutive elements (16-byte accesses for 4-byte
// types, 8-byte for 2-byte floats, 4-byte for bool, all fully coalesced), four
// groups in flight per thread per operand. Consecutive EW entries of a lane over
// the same range (the scheduler's lane-local chains, scheduler.py:552-578) run as
// ONE pass: each group's value is carried in registers from one op to the next,
// and the store of an intermediate that only the next op reads is skipped - the
// loader proves that (see loader.cc) - so a k-op chain moves the chain's true
// inputs and outputs through HBM once.
#ifndef B2VM_OPS_EW_CUH_
#define B2VM_OPS_EW_CUH_

#include <cuda_fp16.h>

#include "dev_common.cuh"

namespace b2 {

// One micro-step of the register-machine form of a chain (see ops_ew_steps.cuh).
struct EwStep {
  uint32_t code, p2, p3;
  uint32_t voff;            // byte offset of the operand's DView in the lane's shared memory
  const uint8_t *ptr;
};
constexpr int kEwMaxSteps = 6;   // forward-copy, two loads, compute, quantize, store
constexpr uint32_t kEwNoSteps = 0xffffffffu;

struct EwOp {                  // decoded chain member, lives in shared memory
  uint32_t sub, dt, adt, flags;
  uint8_t *dst;
  const uint8_t *a, *b, *c;
  uint32_t p2, p3;
  // decided once per entry (ew_decode), read every trip:
  uint32_t la, lb;          // operand load mode: 0 none (unused / forwarded), 1 plain 4-byte,
                            // 2 plain bf16, 3 4-byte through a vector-friendly view, 4 generic
  uint32_t st;              // store mode: 0 dead, 1 4-byte, 2 bf16, 3 generic, 4 LTS (element 0 only)
  uint32_t esz;             // operand element size
  const uint8_t *pfa, *pfb; // contiguous operands worth prefetching (else null)
  DView va, vb;
  uint32_t nsteps, pad;     // kEwNoSteps: this op has no micro-step form (generic executor only)
  EwStep steps[kEwMaxSteps];
};
static_assert(sizeof(EwOp) * kChainMax <= kSmemSys - kSmemChain, "chain cache fits");

__device__ __forceinline__ bool ew_is_bin(uint32_t s) { return s <= kPow || s == kAtan2 || s == kRemainder; }
__device__ __forceinline__ bool ew_is_un(uint32_t s) {
  return (s >= kCopy && s <= kSign) || (s >= kLog1p && s <= kRound) || s == kGelu;
}

// numpy maximum/minimum: NaN if either operand is NaN
__device__ __forceinline__ float np_max(float x, float y) { return (x != x || y != y) ? __int_as_float(0x7fc00000) : fmaxf(x, y); }
__device__ __forceinline__ float np_min(float x, float y) { return (x != x || y != y) ? __int_as_float(0x7fc00000) : fminf(x, y); }
// tanh-approximation GELU, 0.5 x (1 + tanh(u)) with u = 0.7978845608 (x + 0.044715 x^3),
// evaluated in the algebraically identical form x / (1 + exp(-2u)): one exp and one
// reciprocal instead of a full-accuracy tanh; absolute error is ~1e-7 |x|, far
// inside the f32 tolerance of the path.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float x2 = x * x;
  const float t = fmaf(0.044715f * x2, x, x);
  // exp(-2u) = 2^(t * (-2 * 0.7978845608 * log2 e)) on the special-function unit
  const float e = fast_ex2(t * -2.3022082f);
  return x * fast_rcp(1.0f + e);
}
// tanh from one ex2 and one reciprocal, (e^{2x} - 1) / (e^{2x} + 1), with the odd
// polynomial x - x^3/3 + 2x^5/15 - 17x^7/315 below |x| = 0.18 where the quotient
// would cancel; relative error ~3e-7 either side of the switch.
__device__ __forceinline__ float fast_tanh(float x) {
  const float ax = fabsf(x);
  if (ax < 0.18f) {
    const float x2 = x * x;
    return x * fmaf(x2, fmaf(x2, fmaf(x2, -0.05396825397f, 0.13333333333f), -0.33333333333f), 1.0f);
  }
  const float e = fast_ex2(fminf(ax, 15.0f) * 2.8853900818f);     // e^{2|x|}; tanh is 1 to f32 precision past 9
  const float r = 1.0f - 2.0f * fast_rcp(e + 1.0f);
  return copysignf(r, x);
}
// a*s + t with two roundings, as the validator computes it (no contraction)
__device__ __forceinline__ float affine2(float a, float s, float t) { return __fadd_rn(__fmul_rn(a, s), t); }

// x ** y. The exponents a lowered graph actually carries are a handful of constants
// (inverse-square laws: -1.5; norms: 2, 0.5, -0.5); for positive x those are a few
// correctly rounded operations instead of the general routine. Everything else,
// and every x <= 0 / NaN, takes powf, so the special values keep its semantics.
__device__ __forceinline__ float pow_f32(float x, float y) {
  if (x > 0.0f && x < INFINITY) {
    if (y == -1.5f) { const float r = __frsqrt_rn(x); return __fmul_rn(__fmul_rn(r, r), r); }
    if (y == 2.0f) return __fmul_rn(x, x);
    if (y == 0.5f) return __fsqrt_rn(x);
    if (y == -0.5f) return __frsqrt_rn(x);
    if (y == -1.0f) return __frcp_rn(x);
  }
  return powf(x, y);
}

__device__ __forceinline__ float alu_f(uint32_t sub, float x, float y) {
  switch (sub) {
    case kAdd: return __fadd_rn(x, y);
    case kMul: return __fmul_rn(x, y);
    case kSubt: return __fsub_rn(x, y);
    case kDiv: return __fdiv_rn(x, y);
    case kMax: return np_max(x, y);
    case kMin: return np_min(x, y);
#if B2_SHORT
    case kPow: return pow_f32(x, y);
#else
    case kPow: return powf(x, y);
#endif
    case kAtan2: return atan2f(x, y);
    case kRemainder: return fmodf(x, y);
    case kCopy: return x;
    case kNeg: return -x;
    case kExp: return expf(x);
    case kLog: return logf(x);
    case kSqrt: return __fsqrt_rn(x);
    case kRsqrt: return __fdiv_rn(1.0f, __fsqrt_rn(x));
    case kTanh: return tanhf(x);
    case kAbs: return fabsf(x);
    case kFloor: return floorf(x);
    case kCeil: return ceilf(x);
    case kSign: return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : x);
    case kLog1p: return log1pf(x);
    case kExpm1: return expm1f(x);
    case kCbrt: return cbrtf(x);
    case kSin: return sinf(x);
    case kCos: return cosf(x);
    case kTan: return tanf(x);
    case kRint: return rintf(x);
    case kRound: return roundf(x);
    case kGelu: return gelu_tanh(x);
    default: return 0.0f;
  }
}
// The straight-line map ALU shared by MAP_REGION and the matmul store epilogue
// (pjrt_plugin/kernels/vm_common.cl:173-196).
__device__ __forceinline__ float micro_alu(uint32_t kind, float x, float y, float s, float t) {
  switch (kind) {
    case kAdd: return __fadd_rn(x, y);
    case kMul: return __fmul_rn(x, y);
    case kSubt: return __fsub_rn(x, y);
    case kDiv: return __fdiv_rn(x, y);
    case kMax: return np_max(x, y);
    case kMin: return np_min(x, y);
    case kNeg: return -x;
    case kExp: return expf(x);
    case kLog: return logf(x);
    case kSqrt: return __fsqrt_rn(x);
    case kRsqrt: return __fdiv_rn(1.0f, __fsqrt_rn(x));
    case kTanh: return fast_tanh(x);
    case kAbs: return fabsf(x);
    case kAffine: return affine2(x, s, t);
    case kGelu: return gelu_tanh(x);
    default: return x;
  }
}
__device__ __forceinline__ uint32_t alu_i32(uint32_t sub, uint32_t ux, uint32_t uy, bool is_unsigned) {
  const int32_t x = static_cast<int32_t>(ux), y = static_cast<int32_t>(uy);
  switch (sub) {
    case kAdd: return ux + uy;
    case kMul: return ux * uy;
    case kSubt: return ux - uy;
    case kDiv:
      if (uy == 0u) return 0u;  // ew.cl:410
      if (is_unsigned) return ux / uy;
      if (x == INT32_MIN && y == -1) return ux;
      return static_cast<uint32_t>(x / y);
    case kMax: return is_unsigned ? (ux > uy ? ux : uy) : static_cast<uint32_t>(x > y ? x : y);
    case kMin: return is_unsigned ? (ux < uy ? ux : uy) : static_cast<uint32_t>(x < y ? x : y);
    case kCopy: return ux;
    case kNeg: return 0u - ux;
    case kAbs: return (!is_unsigned && x < 0) ? 0u - ux : ux;
    case kSign: return is_unsigned ? (ux ? 1u : 0u) : static_cast<uint32_t>(x > 0 ? 1 : (x < 0 ? -1 : 0));
    case kAnd: return ux & uy;
    case kOr: return ux | uy;
    case kXor: return ux ^ uy;
    case kNot: return ~ux;
    case kShl: return ux << (uy & 31u);
    case kShrL: return ux >> (uy & 31u);
    case kShrA: return static_cast<uint32_t>(x >> (uy & 31u));
    default: return ux;
  }
}
__device__ __forceinline__ uint32_t alu_bool(uint32_t sub, uint32_t x, uint32_t y) {
  switch (sub) {
    case kAnd: return x & y;
    case kOr: return x | y;
    case kXor: return x ^ y;
    case kNot: return x == 0u ? 1u : 0u;
    case kMax: return x > y ? x : y;
    case kMin: return x < y ? x : y;
    default: return x;
  }
}
template <typename T>
__device__ __forceinline__ uint32_t cmp_pred(uint32_t p, T x, T y) {
  switch (p) {
    case 0: return x == y;
    case 1: return x != y;
    case 2: return x < y;
    case 3: return x <= y;
    case 4: return x > y;
    default: return x >= y;
  }
}
// value conversion between 32-bit register representations (ew.cl:532-588;
// float -> int truncates toward zero, ops/making.py:146-160)
__device__ __forceinline__ uint32_t convert32(uint32_t v, uint32_t adt, uint32_t dt) {
  if (is_float_dt(adt)) {
    const float x = __uint_as_float(v);
    if (is_float_dt(dt)) return v;  // rounding to the storage width happens on store / quantize
    if (dt == kU32) return static_cast<uint32_t>(static_cast<long long>(truncf(x)));
    if (dt == kBool) return static_cast<uint32_t>(static_cast<long long>(truncf(x))) & 0xffu;
    return static_cast<uint32_t>(static_cast<int32_t>(truncf(x)));
  }
  if (is_float_dt(dt)) {
    const float f = adt == kI32 ? static_cast<float>(static_cast<int32_t>(v)) : static_cast<float>(v);
    return __float_as_uint(f);
  }
  return dt == kBool ? (v & 0xffu) : v;
}

// Load the 4-element group starting at consumer element i for one operand.
__device__ __forceinline__ void ew_load_operand(const uint8_t *p, uint32_t dt, bool viewed, const DView &v,
                                                uint32_t i, uint32_t vc, uint32_t out[4]) {
  if (!viewed) {
    if (vc == 4u) {
      load4(p, dt, i, out);
    } else {
#pragma unroll
      for (uint32_t e = 0; e < 4; ++e) out[e] = e < vc ? load1(p, dt, static_cast<int64_t>(i) + e) : 0u;
    }
    return;
  }
  if (v.vec_ok && vc == 4u) {
    const int64_t idx = view_index(v, i);
    if (v.inner_stride == 0) {
      const uint32_t s = load1(p, dt, idx);
      out[0] = out[1] = out[2] = out[3] = s;
    } else if (v.aligned4) {
      load4(p, dt, idx, out);
    } else {
#pragma unroll
      for (uint32_t e = 0; e < 4; ++e) out[e] = load1(p, dt, idx + e);
    }
    return;
  }
#pragma unroll
  for (uint32_t e = 0; e < 4; ++e) out[e] = e < vc ? load1(p, dt, view_index(v, i + e)) : 0u;
}

// A complete group of a 4-byte operand through a vector-friendly view.
__device__ __forceinline__ void load_view_w4(const uint8_t *p, const DView &v, uint32_t i, uint32_t out[4]) {
  const int64_t idx = view_index(v, i);
  const uint32_t *q = reinterpret_cast<const uint32_t *>(p) + idx;
  if (v.inner_stride == 0) {
    out[0] = out[1] = out[2] = out[3] = q[0];
  } else if (v.aligned4) {
    const uint4 w = *reinterpret_cast<const uint4 *>(q);
    out[0] = w.x; out[1] = w.y; out[2] = w.z; out[3] = w.w;
  } else {
    out[0] = q[0]; out[1] = q[1]; out[2] = q[2]; out[3] = q[3];
  }
}

constexpr int kEwU = 4;  // groups in flight per thread

// One pass of a chain of k ops over elements [lo, hi); lo % 4 == 0, all pointers
// 16-byte aligned, every dtype 1/2/4 bytes wide.
static __device__ __noinline__ void ew_chain_run(const Lane &L, const EwOp *ops, uint32_t k, uint32_t lo, uint32_t hi) {
  const uint32_t ngroups = (hi - lo + 3u) >> 2;
  for (uint32_t g0 = L.tid; g0 < ngroups; g0 += L.nthr * kEwU) {
    uint32_t X[kEwU][4], Y[kEwU][4];
    uint32_t base[kEwU], vc[kEwU];
#pragma unroll
    for (int u = 0; u < kEwU; ++u) {
      const uint32_t g = g0 + u * L.nthr;
      base[u] = lo + (g << 2);
      vc[u] = g < ngroups ? min(4u, hi - base[u]) : 0u;
#pragma unroll
      for (int e = 0; e < 4; ++e) X[u][e] = 0u;
    }
    const bool full = vc[kEwU - 1] == 4u;   // groups ascend: the last one complete => all complete
    // The ops of a chain run one after the other, so their loads cannot overlap
    // each other; instead every contiguous operand of the NEXT trip is pulled
    // into L2 now, which takes no registers and orders nothing.
    {
      const uint32_t gn = g0 + L.nthr * kEwU;
      if (gn + (kEwU - 1) * L.nthr < ngroups) {
        for (uint32_t j = 0; j < k; ++j) {
          const uint8_t *pa = ops[j].pfa, *pb = ops[j].pfb;
          if (!pa && !pb) continue;
          const uint32_t esz = ops[j].esz;
#pragma unroll
          for (int u = 0; u < kEwU; ++u) {
            const size_t off = static_cast<size_t>(lo + ((gn + u * L.nthr) << 2)) * esz;
            if (pa) prefetch_l2(pa + off);
            if (pb) prefetch_l2(pb + off);
          }
        }
      }
    }
    for (uint32_t j = 0; j < k; ++j) {
      const EwOp &o = ops[j];
      const uint32_t sub = o.sub, dt = o.dt, adt = o.adt, fl = o.flags;
      const uint32_t la = full ? o.la : (o.la ? 4u : 0u), lb = full ? o.lb : (o.lb ? 4u : 0u);
      // X holds the previous op's result on entry; operand a takes it when forwarded.
      if (fl & kFwdB) {
#pragma unroll
        for (int u = 0; u < kEwU; ++u)
#pragma unroll
          for (int e = 0; e < 4; ++e) Y[u][e] = X[u][e];
      }
      // Operand loads. The dtype / view / ragged-edge decisions are hoisted out of
      // the unrolled groups: the common cases are four unconditional 16-byte (or
      // 8-byte) loads back to back.
      if (la) {
        if (la == 1u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) {
            const uint4 w = *reinterpret_cast<const uint4 *>(o.a + static_cast<size_t>(base[u]) * 4);
            X[u][0] = w.x; X[u][1] = w.y; X[u][2] = w.z; X[u][3] = w.w;
          }
        } else if (la == 2u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) {
            const uint2 w = *reinterpret_cast<const uint2 *>(o.a + static_cast<size_t>(base[u]) * 2);
            X[u][0] = w.x << 16; X[u][1] = w.x & 0xffff0000u; X[u][2] = w.y << 16; X[u][3] = w.y & 0xffff0000u;
          }
        } else if (la == 3u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) load_view_w4(o.a, o.va, base[u], X[u]);
        } else {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
            if (vc[u]) ew_load_operand(o.a, adt, fl & kViewA, o.va, base[u], vc[u], X[u]);
        }
      }
      if (lb) {
        if (lb == 1u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) {
            const uint4 w = *reinterpret_cast<const uint4 *>(o.b + static_cast<size_t>(base[u]) * 4);
            Y[u][0] = w.x; Y[u][1] = w.y; Y[u][2] = w.z; Y[u][3] = w.w;
          }
        } else if (lb == 2u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) {
            const uint2 w = *reinterpret_cast<const uint2 *>(o.b + static_cast<size_t>(base[u]) * 2);
            Y[u][0] = w.x << 16; Y[u][1] = w.x & 0xffff0000u; Y[u][2] = w.y << 16; Y[u][3] = w.y & 0xffff0000u;
          }
        } else if (lb == 3u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) load_view_w4(o.b, o.vb, base[u], Y[u]);
        } else {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
            if (vc[u]) ew_load_operand(o.b, adt, fl & kViewB, o.vb, base[u], vc[u], Y[u]);
        }
      }
      // ---- compute (result into X) ----
      if (sub == kSelect) {
#pragma unroll
        for (int u = 0; u < kEwU; ++u) {
          if (!vc[u]) continue;
          uint32_t Z[4];
          ew_load_operand(o.c, kBool, false, o.va, base[u], vc[u], Z);
#pragma unroll
          for (int e = 0; e < 4; ++e) X[u][e] = Z[e] ? X[u][e] : Y[u][e];
        }
      } else if (sub == kCmp) {
        const uint32_t pr = o.p2;
#pragma unroll
        for (int u = 0; u < kEwU; ++u)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t x = X[u][e], y = Y[u][e];
            X[u][e] = is_float_dt(adt) ? cmp_pred<float>(pr, __uint_as_float(x), __uint_as_float(y))
                      : adt == kI32    ? cmp_pred<int32_t>(pr, static_cast<int32_t>(x), static_cast<int32_t>(y))
                                       : cmp_pred<uint32_t>(pr, x, y);
          }
      } else if (sub == kConvert) {
#pragma unroll
        for (int u = 0; u < kEwU; ++u)
#pragma unroll
          for (int e = 0; e < 4; ++e) X[u][e] = convert32(X[u][e], adt, dt);
      } else if (sub == kBitcast) {
        if ((adt == kBF16 && dt == kF16) || (adt == kF16 && dt == kBF16)) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float x = __uint_as_float(X[u][e]);
              X[u][e] = adt == kBF16 ? __float_as_uint(f16_bits_to_f32(f32_to_bf16_bits(x)))
                                     : (f32_to_f16_bits(x) << 16);
            }
        }
      } else if (sub == kIsFinite) {
#pragma unroll
        for (int u = 0; u < kEwU; ++u)
#pragma unroll
          for (int e = 0; e < 4; ++e) X[u][e] = isfinite(__uint_as_float(X[u][e])) ? 1u : 0u;
      } else if (is_float_dt(dt)) {
        if (sub == kAffine) {
          const float s = __uint_as_float(o.p2), t = __uint_as_float(o.p3);
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[u][e] = __float_as_uint(affine2(__uint_as_float(X[u][e]), s, t));
        } else if (sub == kFill) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[u][e] = o.p2;
        } else if (sub == kIotaFlat) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[u][e] = __float_as_uint(static_cast<float>(base[u] + e));
        } else if (sub == kLts) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e)
              X[u][e] = __float_as_uint(__uint_as_float(X[u][e]) < __uint_as_float(Y[u][e]) ? 1.0f : 0.0f);
        } else {
          // One switch, the 16 evaluations inside each case: keeps the code small.
#define B2_EW_F(S, EXPR)                                                        \
  case S:                                                                       \
    _Pragma("unroll") for (int u = 0; u < kEwU; ++u)                            \
    _Pragma("unroll") for (int e = 0; e < 4; ++e) {                             \
      const float x = __uint_as_float(X[u][e]), y = __uint_as_float(Y[u][e]);   \
      (void)y;                                                                  \
      X[u][e] = __float_as_uint(EXPR);                                          \
    }                                                                           \
    break;
          switch (sub) {
            B2_EW_F(kAdd, __fadd_rn(x, y))
            B2_EW_F(kMul, __fmul_rn(x, y))
            B2_EW_F(kSubt, __fsub_rn(x, y))
            B2_EW_F(kDiv, __fdiv_rn(x, y))
            B2_EW_F(kMax, np_max(x, y))
            B2_EW_F(kMin, np_min(x, y))
#if B2_SHORT
            B2_EW_F(kPow, pow_f32(x, y))
#else
            B2_EW_F(kPow, powf(x, y))
#endif
            B2_EW_F(kAtan2, atan2f(x, y))
            B2_EW_F(kRemainder, fmodf(x, y))
            B2_EW_F(kCopy, x)
            B2_EW_F(kNeg, -x)
            B2_EW_F(kExp, expf(x))
            B2_EW_F(kLog, logf(x))
            B2_EW_F(kSqrt, __fsqrt_rn(x))
            B2_EW_F(kRsqrt, __fdiv_rn(1.0f, __fsqrt_rn(x)))
            B2_EW_F(kTanh, tanhf(x))
            B2_EW_F(kAbs, fabsf(x))
            B2_EW_F(kFloor, floorf(x))
            B2_EW_F(kCeil, ceilf(x))
            B2_EW_F(kSign, (x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : x)))
            B2_EW_F(kLog1p, log1pf(x))
            B2_EW_F(kExpm1, expm1f(x))
            B2_EW_F(kCbrt, cbrtf(x))
            B2_EW_F(kSin, sinf(x))
            B2_EW_F(kCos, cosf(x))
            B2_EW_F(kTan, tanf(x))
            B2_EW_F(kRint, rintf(x))
            B2_EW_F(kRound, roundf(x))
            B2_EW_F(kGelu, gelu_tanh(x))
            default: break;
          }
#undef B2_EW_F
        }
      } else if (dt == kBool) {
        if (sub == kFill) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[u][e] = o.p2 & 0xffu;
        } else {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[u][e] = alu_bool(sub, X[u][e], Y[u][e]);
        }
      } else {  // i32 / u32
        const bool uns = dt == kU32;
        if (sub == kFill) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[u][e] = o.p2;
        } else if (sub == kIotaFlat) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) X[u][e] = base[u] + e;
        } else {
          // one switch, the 16 evaluations inside each case (as for floats)
#define B2_EW_I(S, EXPR)                                                        \
  case S:                                                                       \
    _Pragma("unroll") for (int u = 0; u < kEwU; ++u)                            \
    _Pragma("unroll") for (int e = 0; e < 4; ++e) {                             \
      const uint32_t x = X[u][e], y = Y[u][e];                                  \
      (void)y;                                                                  \
      X[u][e] = (EXPR);                                                         \
    }                                                                           \
    break;
          switch (sub) {
            B2_EW_I(kAdd, x + y)
            B2_EW_I(kMul, x * y)
            B2_EW_I(kSubt, x - y)
            B2_EW_I(kAnd, x & y)
            B2_EW_I(kOr, x | y)
            B2_EW_I(kXor, x ^ y)
            B2_EW_I(kNot, ~x)
            B2_EW_I(kNeg, 0u - x)
            B2_EW_I(kShl, x << (y & 31u))
            B2_EW_I(kShrL, x >> (y & 31u))
            B2_EW_I(kMax, uns ? max(x, y) : static_cast<uint32_t>(max(static_cast<int32_t>(x), static_cast<int32_t>(y))))
            B2_EW_I(kMin, uns ? min(x, y) : static_cast<uint32_t>(min(static_cast<int32_t>(x), static_cast<int32_t>(y))))
            default:
#pragma unroll
              for (int u = 0; u < kEwU; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e) X[u][e] = alu_i32(sub, X[u][e], Y[u][e], uns);
              break;
          }
#undef B2_EW_I
        }
      }
      if (dt == kBF16 || dt == kF16) {  // what the next chain op sees is the value as stored
#pragma unroll
        for (int u = 0; u < kEwU; ++u)
#pragma unroll
          for (int e = 0; e < 4; ++e) X[u][e] = __float_as_uint(quantize(__uint_as_float(X[u][e]), dt));
      }
      // ---- store ----
      const uint32_t st = (full || o.st == 0u || o.st == 4u) ? o.st : 3u;
      if (st) {
        if (st == 4u) {
          if (lo == 0u && g0 == 0u) store1(o.dst, dt, 0, X[0][0]);
        } else if (st == 1u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u)
            *reinterpret_cast<uint4 *>(o.dst + static_cast<size_t>(base[u]) * 4) =
                make_uint4(X[u][0], X[u][1], X[u][2], X[u][3]);
        } else if (st == 2u) {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) {   // X already holds bf16-representable values
            uint2 w;
            w.x = (X[u][0] >> 16) | (X[u][1] & 0xffff0000u);
            w.y = (X[u][2] >> 16) | (X[u][3] & 0xffff0000u);
            *reinterpret_cast<uint2 *>(o.dst + static_cast<size_t>(base[u]) * 2) = w;
          }
        } else {
#pragma unroll
          for (int u = 0; u < kEwU; ++u) {
            if (vc[u] == 4u) {
              store4(o.dst, dt, base[u], X[u]);
            } else {
#pragma unroll
              for (uint32_t e = 0; e < 4; ++e)   // static indices: X stays in registers
                if (e < vc[u]) store1(o.dst, dt, static_cast<int64_t>(base[u]) + e, X[u][e]);
            }
          }
        }
      }
    }
  }
}

// ---- generic scalar path: 8-byte dtypes and unaligned buffers ---------------------------
__device__ __forceinline__ long long ld_i64any(const uint8_t *p, uint32_t dt, int64_t i) {
  switch (dt) {
    case kI64: return reinterpret_cast<const long long *>(p)[i];
    case kI32: return reinterpret_cast<const int32_t *>(p)[i];
    case kU32: return reinterpret_cast<const uint32_t *>(p)[i];
    default: return p[i];
  }
}
__device__ __forceinline__ void st_i64any(uint8_t *p, uint32_t dt, int64_t i, long long v) {
  switch (dt) {
    case kI64: reinterpret_cast<long long *>(p)[i] = v; break;
    case kI32: case kU32: reinterpret_cast<uint32_t *>(p)[i] = static_cast<uint32_t>(v); break;
    default: p[i] = static_cast<uint8_t>(v); break;
  }
}
__device__ __forceinline__ double ld_f64any(const uint8_t *p, uint32_t dt, int64_t i) {
  if (dt == kF64) return reinterpret_cast<const double *>(p)[i];
  if (is_float_dt(dt)) return static_cast<double>(loadf(p, dt, i));
  if (dt == kU32) return static_cast<double>(reinterpret_cast<const uint32_t *>(p)[i]);
  return static_cast<double>(ld_i64any(p, dt, i));
}

static __device__ __noinline__ void ew_scalar_run(const Lane &L, const EwOp &o, uint32_t lo, uint32_t hi) {
  const uint32_t sub = o.sub, dt = o.dt, adt = o.adt;
  const bool wide = dt == kI64 || dt == kF64 || adt == kI64 || adt == kF64;
  for (uint32_t i = lo + L.tid; i < hi; i += L.nthr) {
    const int64_t ia = (o.flags & kViewA) ? view_index(o.va, i) : i;
    const int64_t ib = (o.flags & kViewB) ? view_index(o.vb, i) : i;
    if (!wide) {  // 1/2/4-byte dtypes on unaligned buffers: same ALUs as the vector path
      uint32_t x = load1(o.a, adt, ia), y = 0u, r;
      const bool needs_b = ew_is_bin(sub) || sub == kCmp || sub == kSelect || sub == kLts ||
                           (sub >= kAnd && sub <= kXor) || (sub >= kShl && sub <= kShrA);
      if (needs_b) y = load1(o.b, adt, ib);
      if (sub == kSelect) r = o.c[i] ? x : y;
      else if (sub == kCmp)
        r = is_float_dt(adt) ? cmp_pred<float>(o.p2, __uint_as_float(x), __uint_as_float(y))
            : adt == kI32    ? cmp_pred<int32_t>(o.p2, static_cast<int32_t>(x), static_cast<int32_t>(y))
                             : cmp_pred<uint32_t>(o.p2, x, y);
      else if (sub == kConvert) r = convert32(x, adt, dt);
      else if (sub == kBitcast) {
        r = x;
        if (adt == kBF16 && dt == kF16) r = __float_as_uint(f16_bits_to_f32(f32_to_bf16_bits(__uint_as_float(x))));
        if (adt == kF16 && dt == kBF16) r = f32_to_f16_bits(__uint_as_float(x)) << 16;
      } else if (sub == kIsFinite) r = isfinite(__uint_as_float(x)) ? 1u : 0u;
      else if (is_float_dt(dt)) {
        if (sub == kAffine) r = __float_as_uint(affine2(__uint_as_float(x), __uint_as_float(o.p2), __uint_as_float(o.p3)));
        else if (sub == kFill) r = o.p2;
        else if (sub == kIotaFlat) r = __float_as_uint(static_cast<float>(i));
        else if (sub == kLts) { if (i == 0u) store1(o.dst, dt, 0, __float_as_uint(__uint_as_float(x) < __uint_as_float(y) ? 1.0f : 0.0f)); continue; }
        else r = __float_as_uint(alu_f(sub, __uint_as_float(x), __uint_as_float(y)));
      } else if (dt == kBool) r = sub == kFill ? (o.p2 & 0xffu) : alu_bool(sub, x, y);
      else r = sub == kFill ? o.p2 : sub == kIotaFlat ? i : alu_i32(sub, x, y, dt == kU32);
      store1(o.dst, dt, i, r);
      continue;
    }
    // 8-byte dtypes (ew.cl:356-391 f64, :433-463 i64) and conversions to/from them
    if (sub == kConvert) {
      if (adt == kF64 || is_float_dt(adt)) {
        const double x = ld_f64any(o.a, adt, ia);
        if (dt == kF64) reinterpret_cast<double *>(o.dst)[i] = x;
        else if (is_float_dt(dt)) storef(o.dst, dt, i, static_cast<float>(x));
        else st_i64any(o.dst, dt, i, static_cast<long long>(trunc(x)));
      } else {
        const long long x = ld_i64any(o.a, adt, ia);
        if (dt == kF64) reinterpret_cast<double *>(o.dst)[i] = adt == kU32 ? static_cast<double>(static_cast<uint32_t>(x)) : static_cast<double>(x);
        else if (is_float_dt(dt)) storef(o.dst, dt, i, static_cast<float>(x));
        else st_i64any(o.dst, dt, i, x);
      }
      continue;
    }
    if (sub == kBitcast) {
      reinterpret_cast<unsigned long long *>(o.dst)[i] = reinterpret_cast<const unsigned long long *>(o.a)[ia];
      continue;
    }
    if (sub == kSelect) {
      reinterpret_cast<unsigned long long *>(o.dst)[i] =
          o.c[i] ? reinterpret_cast<const unsigned long long *>(o.a)[ia] : reinterpret_cast<const unsigned long long *>(o.b)[ib];
      continue;
    }
    if (sub == kCmp) {
      o.dst[i] = adt == kF64 ? cmp_pred<double>(o.p2, ld_f64any(o.a, adt, ia), ld_f64any(o.b, adt, ib))
                             : cmp_pred<long long>(o.p2, ld_i64any(o.a, adt, ia), ld_i64any(o.b, adt, ib));
      continue;
    }
    if (sub == kIsFinite) { o.dst[i] = isfinite(ld_f64any(o.a, adt, ia)) ? 1 : 0; continue; }
    if (dt == kF64) {
      double r;
      if (sub == kFill) r = static_cast<double>(__uint_as_float(o.p2));
      else if (sub == kIotaFlat) r = static_cast<double>(i);
      else {
        const double x = ld_f64any(o.a, adt, ia), y = ew_is_bin(sub) ? ld_f64any(o.b, adt, ib) : 0.0;
        switch (sub) {
          case kAdd: r = x + y; break; case kMul: r = x * y; break; case kSubt: r = x - y; break;
          case kDiv: r = x / y; break;
          case kMax: r = (x != x || y != y) ? nan("") : fmax(x, y); break;
          case kMin: r = (x != x || y != y) ? nan("") : fmin(x, y); break;
          case kPow: r = pow(x, y); break; case kNeg: r = -x; break; case kExp: r = exp(x); break;
          case kLog: r = log(x); break; case kSqrt: r = sqrt(x); break; case kRsqrt: r = 1.0 / sqrt(x); break;
          case kTanh: r = tanh(x); break; case kAbs: r = fabs(x); break; case kFloor: r = floor(x); break;
          case kCeil: r = ceil(x); break; case kSign: r = x > 0 ? 1.0 : (x < 0 ? -1.0 : x); break;
          default: r = x; break;
        }
      }
      reinterpret_cast<double *>(o.dst)[i] = r;
      continue;
    }
    // i64
    long long r;
    if (sub == kFill) r = static_cast<int32_t>(o.p2);
    else if (sub == kIotaFlat) r = i;
    else {
      const long long x = ld_i64any(o.a, adt, ia);
      const bool needs_y = sub <= kPow || (sub >= kAnd && sub <= kXor) || (sub >= kShl && sub <= kShrA);
      const long long y = needs_y ? ld_i64any(o.b, adt, ib) : 0;
      const unsigned long long ux = x, uy = y;
      switch (sub) {
        case kAdd: r = ux + uy; break; case kMul: r = ux * uy; break; case kSubt: r = ux - uy; break;
        case kDiv: r = y ? ((x == LLONG_MIN && y == -1) ? x : x / y) : 0; break;
        case kMax: r = x > y ? x : y; break; case kMin: r = x < y ? x : y; break;
        case kNeg: r = 0ull - ux; break; case kAbs: r = x < 0 ? static_cast<long long>(0ull - ux) : x; break;
        case kSign: r = x > 0 ? 1 : (x < 0 ? -1 : 0); break;
        case kAnd: r = x & y; break; case kOr: r = x | y; break; case kXor: r = x ^ y; break;
        case kNot: r = ~x; break;
        case kShl: r = ux << (uy & 63u); break; case kShrL: r = ux >> (uy & 63u); break;
        case kShrA: r = x >> (uy & 63u); break;
        default: r = x; break;
      }
    }
    reinterpret_cast<long long *>(o.dst)[i] = r;
  }
}

__device__ __forceinline__ void ew_decode(const KParams &P, const DTask &t, EwOp *o) {
  o->sub = t.p[0];
  o->dt = t.dt;
  o->adt = t.adt;
  o->flags = t.flags;
  o->dst = resolve(P, t.ptr[0]);
  o->a = resolve(P, t.ptr[1]);
  o->b = resolve(P, t.ptr[2]);
  o->c = resolve(P, t.ptr[3]);
  o->p2 = t.p[2];
  o->p3 = t.p[3];
  if (t.flags & (kViewA | kViewB)) {
    const DView *dv = reinterpret_cast<const DView *>(P.desc + t.desc);
    if (t.flags & kViewA) o->va = dv[0];
    if (t.flags & kViewB) o->vb = dv[1];
  }
  const uint32_t sub = o->sub, adt = o->adt, dt = o->dt, fl = o->flags;
  const bool needs_a = !(sub == kFill || sub == kIotaFlat);
  const bool needs_b = ew_is_bin(sub) || sub == kCmp || sub == kSelect || sub == kLts ||
                       (sub >= kAnd && sub <= kXor) || (sub >= kShl && sub <= kShrA);
  const bool w4 = adt == kF32 || adt == kI32 || adt == kU32;
  auto mode = [&](bool needed, bool fwd, bool viewed, const DView &v) -> uint32_t {
    if (!needed || fwd) return 0u;
    if (!viewed) return w4 ? 1u : (adt == kBF16 ? 2u : 4u);
    return (w4 && v.vec_ok) ? 3u : 4u;
  };
  o->la = mode(needs_a, fl & kFwdA, fl & kViewA, o->va);
  o->lb = mode(needs_b, fl & kFwdB, fl & kViewB, o->vb);
  o->st = (fl & kDeadStore) ? 0u : sub == kLts ? 4u
          : (dt == kF32 || dt == kI32 || dt == kU32) ? 1u : dt == kBF16 ? 2u : 3u;
  o->esz = dt_size(adt);
  o->pfa = (o->la == 1u || o->la == 2u) ? o->a : nullptr;
  o->pfb = (o->lb == 1u || o->lb == 2u) ? o->b : nullptr;
}

}  // namespace b2
#endif
