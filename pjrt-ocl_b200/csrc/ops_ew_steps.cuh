// Register-machine form of an elementwise chain.
//
// A chain of k elementwise ops over one element range is compiled, once per lane
// entry, into a short list of micro-steps over two banks X and Y of 4-element
// groups: "load operand into X / Y", "Y <- X", one arithmetic step per op,
// "round to bf16", "store X". The steps are then run block by block over the
// range (ew_steps_run). Compared with interpreting the decoded ops directly
// (ew_chain_run) the per-op ladders of mode / dtype tests leave the inner loops:
// the tests run once, when the steps are built.
//
// Ops outside the common set (transcendentals other than exp / log / tanh, f16,
// integer division, is_finite, ...) have no micro-step form; a chain containing
// one runs on ew_chain_run instead. Semantics are those of ops_ew.cuh, which
// follows pjrt_plugin/kernels/ops/ew.cl:226-658.
#ifndef B2VM_OPS_EW_STEPS_CUH_
#define B2VM_OPS_EW_STEPS_CUH_

#include "ops_ew.cuh"

namespace b2 {

enum EwStepCode : uint32_t {
  kSMovYX = 0,
  // loads: X variant, then Y variant
  kSLdXW4, kSLdYW4,          // contiguous 4-byte elements
  kSLdXBf, kSLdYBf,          // contiguous bf16
  kSLdXB1, kSLdYB1,          // contiguous bool
  kSLdXRowW4, kSLdYRowW4,    // a row vector broadcast over rows: index = off + i mod d
  kSLdXRowBf, kSLdYRowBf,
  kSLdXViewW4, kSLdYViewW4,  // any view of up to 4 (vector-friendly) or 3 (element-wise walk) collapsed dims
  kSLdXViewBf, kSLdYViewBf,
  kSLdXColW4, kSLdYColW4,    // a column vector broadcast along rows: index = off + (i / d) * stride
  kSLdXColBf, kSLdYColBf,
  kSStW4, kSStBf, kSStB1,
  kSQuantBf,
  kSAffine, kSFill, kSIotaF, kSIotaI, kSSelect,
  kSCvtF2I, kSCvtF2U, kSCvtI2F, kSCvtU2F, kSCvtF2B, kSCvtI2B,
  kSBNot, kSUMax, kSUMin,
  kSCmpF,                    // + predicate 0..5
  kSCmpI = kSCmpF + 6,
  kSCmpU = kSCmpI + 6,
  kSFlt = kSCmpU + 6,        // + ew_fcode(Sub) (float arithmetic)
  kSInt = kSFlt + 18,        // + ew_icode(Sub) (i32 / u32 / bool arithmetic)
  kSEnd = kSInt + 14,
};
// The codes are dense on purpose: the dispatch switch compiles to one jump table.
__host__ __device__ constexpr uint32_t ew_fcode(uint32_t sub) {   // kAdd..kMin, kNeg..kSign, kGelu, kPow
  return sub <= kMin ? sub : sub == kPow ? 17u : sub <= kSign ? sub - 2u : 16u;
}
__host__ __device__ constexpr uint32_t ew_icode(uint32_t sub) {
  return sub <= kSubt ? sub : sub == kMax ? 3u : sub == kMin ? 4u : sub == kNeg ? 5u : sub == kAbs ? 6u
         : sub <= kNot ? sub - 28u : sub - 31u;   // kAnd..kNot -> 7..10, kShl..kShrA -> 11..13
}

__device__ __forceinline__ bool ew_is_w4(uint32_t dt) { return dt == kF32 || dt == kI32 || dt == kU32; }

// Compile one decoded op into its micro-steps (o->nsteps = kEwNoSteps when it has none).
__device__ inline void ew_build_steps(EwOp *o, uint32_t smem_off_of_op) {
  const uint32_t sub = o->sub, dt = o->dt, adt = o->adt, fl = o->flags;
  uint32_t n = 0;
  bool ok = (fl & kVecPath) != 0 && dt != kF16 && adt != kF16;
  auto emit = [&](uint32_t code, const uint8_t *ptr, uint32_t voff, uint32_t p2, uint32_t p3) {
    if (n < kEwMaxSteps) {
      EwStep &s = o->steps[n];
      s.code = code; s.ptr = ptr; s.voff = voff; s.p2 = p2; s.p3 = p3;
    } else {
      ok = false;
    }
    ++n;
  };
  const bool needs_b = ew_is_bin(sub) || sub == kCmp || sub == kSelect || sub == kLts ||
                       (sub >= kAnd && sub <= kXor) || (sub >= kShl && sub <= kShrA);
  if ((fl & kFwdB) && needs_b) emit(kSMovYX, nullptr, 0, 0, 0);
  const uint32_t esz = dt_size(adt);
  auto load = [&](uint32_t is_y, uint32_t mode, const uint8_t *p, bool viewed, const DView &v, uint32_t voff) {
    if (mode == 0u) return;
    const bool w4 = ew_is_w4(adt), bf = adt == kBF16;
    if (!viewed) {
      if (w4) emit(kSLdXW4 + is_y, p, 0, 0, 0);
      else if (bf) emit(kSLdXBf + is_y, p, 0, 0, 0);
      else if (adt == kBool) emit(kSLdXB1 + is_y, p, 0, 0, 0);
      else ok = false;
      return;
    }
    if (!(w4 || bf)) { ok = false; return; }
    if (!v.vec_ok) {
#if B2_SHORT
      // the 4 elements of a group are not adjacent in the source (an innermost axis of 3,
      // a strided slice): the general view load walks the coordinates element by element
      if (v.rank < 1 || v.rank > 3) { ok = false; return; }
      emit((w4 ? kSLdXViewW4 : kSLdXViewBf) + is_y, p, voff, 0, 0);
#else
      ok = false;
#endif
      return;
    }
    if (v.rank == 1 && v.inner_stride == 1 && v.aligned4) {      // an offset slice: contiguous
      emit((w4 ? kSLdXW4 : kSLdXBf) + is_y, p + v.off * static_cast<int64_t>(esz), 0, 0, 0);
    } else if (v.rank == 2 && v.stride[0] == 0 && v.inner_stride == 1 && v.aligned4) {
      emit((w4 ? kSLdXRowW4 : kSLdXRowBf) + is_y, p, voff, 0, 0);
    } else if (v.rank == 2 && v.inner_stride == 0) {
      emit((w4 ? kSLdXColW4 : kSLdXColBf) + is_y, p, voff, 0, 0);
    } else {
      emit((w4 ? kSLdXViewW4 : kSLdXViewBf) + is_y, p, voff, 0, 0);
    }
  };
  const uint32_t va_off = smem_off_of_op + static_cast<uint32_t>(offsetof(EwOp, va));
  const uint32_t vb_off = smem_off_of_op + static_cast<uint32_t>(offsetof(EwOp, vb));
  load(0u, o->la, o->a, (fl & kViewA) != 0, o->va, va_off);
  load(1u, o->lb, o->b, (fl & kViewB) != 0, o->vb, vb_off);

  const bool fdt = dt == kF32 || dt == kBF16;
  const bool fadt = adt == kF32 || adt == kBF16;
  bool quant = dt == kBF16;
  switch (sub) {
    case kSelect:
      emit(kSSelect, o->c, 0, 0, 0);
      quant = false;
      break;
    case kCmp:
      if (o->p2 > 5u) ok = false;
      emit((fadt ? kSCmpF : adt == kI32 ? kSCmpI : kSCmpU) + o->p2, nullptr, 0, 0, 0);
      break;
    case kConvert:
      if (fadt) {
        if (dt == kI32) emit(kSCvtF2I, nullptr, 0, 0, 0);
        else if (dt == kU32) emit(kSCvtF2U, nullptr, 0, 0, 0);
        else if (dt == kBool) emit(kSCvtF2B, nullptr, 0, 0, 0);
        else if (!fdt) ok = false;
      } else if (fdt) {
        emit(adt == kI32 ? kSCvtI2F : kSCvtU2F, nullptr, 0, 0, 0);
      } else if (dt == kBool) {
        emit(kSCvtI2B, nullptr, 0, 0, 0);
      }
      break;
    case kBitcast:
      if (!(adt == dt || (ew_is_w4(adt) && ew_is_w4(dt)))) ok = false;
      quant = false;
      break;
    case kIsFinite:
    case kLts:
      ok = false;
      break;
    default:
      if (fdt) {
        if (sub == kAffine) emit(kSAffine, nullptr, 0, o->p2, o->p3);
        else if (sub == kFill) emit(kSFill, nullptr, 0, o->p2, 0);
        else if (sub == kIotaFlat) emit(kSIotaF, nullptr, 0, 0, 0);
        else if (sub == kCopy) quant = quant && adt != kBF16;
        else if (sub <= (B2_SHORT ? kPow : kMin) || (sub >= kNeg && sub <= kSign) || sub == kGelu) {
          emit(kSFlt + ew_fcode(sub), nullptr, 0, 0, 0);
          if ((sub == kNeg || sub == kAbs || sub == kMax || sub == kMin) && adt == kBF16) quant = false;
        } else ok = false;
      } else if (dt == kBool) {
        if (sub == kFill) emit(kSFill, nullptr, 0, o->p2 & 0xffu, 0);
        else if (sub == kAnd || sub == kOr || sub == kXor) emit(kSInt + ew_icode(sub), nullptr, 0, 0, 0);
        else if (sub == kMax) emit(kSInt + ew_icode(kOr), nullptr, 0, 0, 0);
        else if (sub == kMin) emit(kSInt + ew_icode(kAnd), nullptr, 0, 0, 0);
        else if (sub == kNot) emit(kSBNot, nullptr, 0, 0, 0);
        else if (sub != kCopy) ok = false;
      } else if (dt == kI32 || dt == kU32) {
        const bool uns = dt == kU32;
        if (sub == kFill) emit(kSFill, nullptr, 0, o->p2, 0);
        else if (sub == kIotaFlat) emit(kSIotaI, nullptr, 0, 0, 0);
        else if (sub == kMax && uns) emit(kSUMax, nullptr, 0, 0, 0);
        else if (sub == kMin && uns) emit(kSUMin, nullptr, 0, 0, 0);
        else if (sub == kAdd || sub == kMul || sub == kSubt || sub == kMax || sub == kMin || sub == kNeg ||
                 (sub >= kAnd && sub <= kNot) || sub == kShl || sub == kShrL || sub == kShrA)
          emit(kSInt + ew_icode(sub), nullptr, 0, 0, 0);
        else if (sub == kAbs && !uns) emit(kSInt + ew_icode(kAbs), nullptr, 0, 0, 0);
        else if (!(sub == kCopy || (sub == kAbs && uns))) ok = false;
      } else {
        ok = false;
      }
      break;
  }
  if (quant) emit(kSQuantBf, nullptr, 0, 0, 0);
  switch (o->st) {
    case 0u: break;
    case 1u: emit(kSStW4, o->dst, 0, 0, 0); break;
    case 2u: emit(kSStBf, o->dst, 0, 0, 0); break;
    case 3u:
      if (dt == kBool) emit(kSStB1, o->dst, 0, 0, 0);
      else ok = false;
      break;
    default: ok = false; break;
  }
  o->nsteps = (ok && n <= kEwMaxSteps) ? n : kEwNoSteps;
}

// n / d and n mod d through the view's precomputed magic for dimension k.
__device__ __forceinline__ uint32_t view_mod(const DView &v, int k, uint32_t n) {
  const uint32_t mh = __umulhi(n, v.magic[k]);
  const uint32_t q = (((n - mh) >> 1) + mh) >> v.shift[k];
  return n - q * v.dim[k];
}

// The chain's steps in execution order, flattened by ew_plan (one thread) so the
// trip loop is a single counted loop; lives after the EwOp array.
struct EwFlat {
  uint32_t n;
  uint32_t tier;            // smallest EwTier that has every step of the chain
  EwStep s[kChainMax * kEwMaxSteps];
};
constexpr int kSmemEwFlat = kSmemChain + static_cast<int>(sizeof(EwOp)) * kChainMax;
static_assert(kSmemEwFlat + sizeof(EwFlat) <= kSmemSys, "flattened steps fit the system area");

// The trip loop is compiled five times ("tiers"), each containing only some of the step
// bodies: the compiler's code for the common steps is markedly better (fewer register
// moves around the dispatch, no spills) when the rarely used, long or register-hungry
// bodies are not in the same function. A chain runs in the smallest tier that has all
// its steps:
//   kTierF32  4-byte contiguous / row-vector loads, 4-byte store, float add mul sub max min neg abs
//             gelu, affine, fill
//   kTierBf   the same with bf16 loads / stores / rounding added
//   kTierInt  4-byte loads / stores and the integer ops
//   kTierHot  every short body
//   kTierAll  everything (division, transcendentals, rounding, conversions, general strided and
//             column-broadcast loads)
enum EwTier : int { kTierF32 = 0, kTierBf, kTierInt, kTierHot, kTierAll };

__host__ __device__ constexpr bool ew_is_cheap_float(uint32_t c) {
  return c >= kSFlt && c < kSInt &&
         (c - kSFlt == ew_fcode(kAdd) || c - kSFlt == ew_fcode(kMul) || c - kSFlt == ew_fcode(kSubt) ||
          c - kSFlt == ew_fcode(kMax) || c - kSFlt == ew_fcode(kMin) || c - kSFlt == ew_fcode(kNeg) ||
          c - kSFlt == ew_fcode(kAbs) || c - kSFlt == ew_fcode(kGelu));
}
__host__ __device__ constexpr bool ew_step_is_cold(uint32_t c) {
  return (c >= kSFlt && c < kSInt && !ew_is_cheap_float(c)) || c == kSIotaF || c == kSIotaI ||
         (c >= kSCvtF2I && c <= kSBNot) || (c >= kSLdXViewW4 && c <= kSLdYColBf);
}
__host__ __device__ constexpr bool ew_tier_has(int tier, uint32_t c) {
  if (tier == kTierAll) return true;
  if (tier == kTierHot) return !ew_step_is_cold(c);
  const bool f32core = c == kSMovYX || c == kSLdXW4 || c == kSLdYW4 || c == kSLdXRowW4 || c == kSLdYRowW4 ||
                       c == kSStW4 || c == kSAffine || c == kSFill || ew_is_cheap_float(c);
  if (tier == kTierF32) return f32core;
  if (tier == kTierBf)
    return f32core || c == kSLdXBf || c == kSLdYBf || c == kSLdXRowBf || c == kSLdYRowBf || c == kSStBf || c == kSQuantBf;
  // kTierInt
  return c == kSMovYX || c == kSLdXW4 || c == kSLdYW4 || c == kSStW4 || c == kSFill || c == kSUMax || c == kSUMin ||
         (c >= kSInt && c < kSEnd);
}

// One thread, after every op's steps are built.
//
// Row vectors broadcast over rows (LdRow steps) are read by every lane over and
// over: left in global memory they turn a handful of L2 lines into a hot spot
// that every SM queues on. They are copied into the lane's shared memory once per
// entry instead (p2 = 1, p3 = byte offset) when they fit.
__device__ inline void ew_plan(EwOp *ops, uint32_t k, EwFlat *fl, uint32_t smem_bytes) {
  const uint8_t *sm = reinterpret_cast<const uint8_t *>(ops) - kSmemChain;
  uint32_t n = 0, used = 0;
  bool in_tier[5] = {true, true, true, true, true};
  const uint32_t avail = smem_bytes > static_cast<uint32_t>(kSmemSys) ? smem_bytes - kSmemSys : 0u;
  for (uint32_t j = 0; j < k && ops[j].nsteps != kEwNoSteps; ++j)
    for (uint32_t si = 0; si < ops[j].nsteps; ++si) {
      EwStep st = ops[j].steps[si];
      if (st.code >= kSLdXRowW4 && st.code <= kSLdYRowBf) {
        const DView &v = *reinterpret_cast<const DView *>(sm + st.voff);
        const uint32_t esz = (st.code == kSLdXRowBf || st.code == kSLdYRowBf) ? 2u : 4u;
        const uint32_t b = (v.dim[1] * esz + 15u) & ~15u;
        if (used + b <= avail) { st.p2 = 1u; st.p3 = kSmemSys + used; used += b; }
      }
      for (int tr = 0; tr < 5; ++tr) in_tier[tr] = in_tier[tr] && ew_tier_has(tr, st.code);
      fl->s[n++] = st;
    }
  fl->n = n;
  fl->tier = in_tier[0] ? 0u : in_tier[1] ? 1u : in_tier[2] ? 2u : in_tier[3] ? 3u : 4u;
}

// Copy the cached row vectors in (all threads of the lane; 8-byte words, which is
// as aligned as a bf16 vector is guaranteed to be).
__device__ __forceinline__ void ew_stage_rows(const Lane &L, const EwFlat *fl) {
  bool any = false;
  for (uint32_t i = 0; i < fl->n; ++i) {
    const EwStep &st = fl->s[i];
    if (!(st.code >= kSLdXRowW4 && st.code <= kSLdYRowBf) || !st.p2) continue;
    const DView &v = *reinterpret_cast<const DView *>(L.smem + st.voff);
    const uint32_t esz = (st.code == kSLdXRowBf || st.code == kSLdYRowBf) ? 2u : 4u;
    const uint8_t *src = st.ptr + v.off * static_cast<int64_t>(esz);
    uint2 *dst = reinterpret_cast<uint2 *>(L.smem + st.p3);
    const uint32_t words = v.dim[1] * esz / 8u;
    for (uint32_t w = L.tid; w < words; w += L.nthr) dst[w] = ldg_v2(src + static_cast<size_t>(w) * 8);
    any = true;
  }
  if (any) __syncthreads();
}

// Trips over the complete 4-element groups [gb, ge) of the range starting at
// element `lo`. Per trip a thread owns kEwU groups (group g0 + u * nthr), held in
// the register banks X and Y across the steps; each step body is the 16
// evaluations, fully unrolled. FULL: every trip has all kEwU groups (ge - gb is a
// multiple of nthr * kEwU), so no access is predicated. TIER: which step bodies are
// compiled in (ew_tier_has).
template <bool FULL, int TIER>
static __device__ __noinline__ void ew_steps_run(uint32_t tid, uint32_t nthr, uint32_t lo, uint32_t gb, uint32_t ge) {
  B2_DYN_SMEM(sm);
  const EwFlat &fl = *reinterpret_cast<const EwFlat *>(sm + kSmemEwFlat);
  const uint32_t nsteps = fl.n;
  const uint32_t trip_groups = nthr * kEwU;
  const uint32_t estep = nthr << 2;                 // elements between a thread's groups
  const size_t trip_elems = static_cast<size_t>(trip_groups) * 4;
  for (uint32_t t0 = gb; t0 < ge; t0 += trip_groups) {
    uint32_t X[kEwU][4], Y[kEwU][4];
    const uint32_t g0 = t0 + tid;
    const uint32_t eb = lo + (g0 << 2);             // first element of group 0; group u adds u * estep
    bool on[kEwU];
#pragma unroll
    for (int u = 0; u < kEwU; ++u) {
      on[u] = FULL || g0 + u * nthr < ge;
#pragma unroll
      for (int e = 0; e < 4; ++e) X[u][e] = Y[u][e] = 0u;
    }
    // the whole next trip exists: its contiguous operands are pulled into L2 now
    const bool pf = t0 + 2u * trip_groups <= ge;

#define B2_GROUPS _Pragma("unroll") for (int u = 0; u < kEwU; ++u) if (FULL || on[u])
#define B2_SET(R, W) { const uint4 w_ = (W); R[u][0] = w_.x; R[u][1] = w_.y; R[u][2] = w_.z; R[u][3] = w_.w; }
    auto unpack_bf = [](uint2 w) { return make_uint4(w.x << 16, w.x & 0xffff0000u, w.y << 16, w.y & 0xffff0000u); };
    auto ld_w4 = [&](uint32_t (&R)[kEwU][4], const EwStep &st) {
      const uint8_t *q = st.ptr + static_cast<size_t>(eb) * 4;
      B2_GROUPS B2_SET(R, ldg_v4(q + static_cast<size_t>(u) * estep * 4))
      if (pf) {
#pragma unroll
        for (int u = 0; u < kEwU; ++u) prefetch_l2(q + trip_elems * 4 + static_cast<size_t>(u) * estep * 4);
      }
    };
    auto ld_bf = [&](uint32_t (&R)[kEwU][4], const EwStep &st) {
      const uint8_t *q = st.ptr + static_cast<size_t>(eb) * 2;
      B2_GROUPS B2_SET(R, unpack_bf(ldg_v2(q + static_cast<size_t>(u) * estep * 2)))
      if (pf) {
#pragma unroll
        for (int u = 0; u < kEwU; ++u) prefetch_l2(q + trip_elems * 2 + static_cast<size_t>(u) * estep * 2);
      }
    };
    auto ld_b1 = [&](uint32_t (&R)[kEwU][4], const EwStep &st) {
      const uint8_t *q = st.ptr + eb;
      B2_GROUPS {
        const uint32_t w = ldg_u32(q + static_cast<size_t>(u) * estep);
        B2_SET(R, make_uint4(w & 0xffu, (w >> 8) & 0xffu, (w >> 16) & 0xffu, w >> 24))
      }
    };
    auto ld_at = [&](const uint8_t *p, int64_t idx, bool bf, bool bcast, bool al4) -> uint4 {
      if (bf) {
        const uint8_t *q = p + idx * 2;
        if (bcast) { const uint32_t v = ldg_u16(q) << 16; return make_uint4(v, v, v, v); }
        if (al4) return unpack_bf(ldg_v2(q));
        return make_uint4(ldg_u16(q) << 16, ldg_u16(q + 2) << 16, ldg_u16(q + 4) << 16, ldg_u16(q + 6) << 16);
      }
      const uint8_t *q = p + idx * 4;
      if (bcast) { const uint32_t v = ldg_u32(q); return make_uint4(v, v, v, v); }
      if (al4) return ldg_v4(q);
      return make_uint4(ldg_u32(q), ldg_u32(q + 4), ldg_u32(q + 8), ldg_u32(q + 12));
    };
    auto ld_row = [&](uint32_t (&R)[kEwU][4], const EwStep &st, bool bf) {
      const DView &v = *reinterpret_cast<const DView *>(sm + st.voff);
      if (st.p2) {   // the vector sits in shared memory
        const uint8_t *c0 = sm + st.p3;
        B2_GROUPS {
          const uint32_t c = view_mod(v, 1, eb + u * estep);
          if (bf) B2_SET(R, unpack_bf(*reinterpret_cast<const uint2 *>(c0 + c * 2u)))
          else B2_SET(R, *reinterpret_cast<const uint4 *>(c0 + c * 4u))
        }
        return;
      }
      const uint8_t *p = st.ptr + v.off * (bf ? 2 : 4);
      B2_GROUPS {
        const uint32_t c = view_mod(v, 1, eb + u * estep);
        if (bf) B2_SET(R, unpack_bf(ldg_v2(p + static_cast<size_t>(c) * 2)))
        else B2_SET(R, ldg_v4(p + static_cast<size_t>(c) * 4))
      }
    };
    // one value per row, the same for the 4 elements of a group (a group never straddles a row)
    auto ld_col = [&](uint32_t (&R)[kEwU][4], const EwStep &st, bool bf) {
      const DView &v = *reinterpret_cast<const DView *>(sm + st.voff);
      const uint32_t mg = v.magic[1], sh = v.shift[1];
      const int64_t off = v.off, s0 = v.stride[0];
      B2_GROUPS {
        const uint32_t n = eb + u * estep, mh = __umulhi(n, mg);
        const uint32_t row = (((n - mh) >> 1) + mh) >> sh;
        const int64_t idx = off + row * s0;
        const uint32_t val = bf ? (ldg_u16(st.ptr + idx * 2) << 16) : ldg_u32(st.ptr + idx * 4);
        R[u][0] = R[u][1] = R[u][2] = R[u][3] = val;
      }
    };
    auto ld_view = [&](uint32_t (&R)[kEwU][4], const EwStep &st, bool bf) {
      const DView &v = *reinterpret_cast<const DView *>(sm + st.voff);
#if B2_SHORT
      if (!v.vec_ok) {
        const ViewWalk w = view_walk(v);
        B2_GROUPS {
          uint32_t cA, cB, cO;
          view_walk_seek(w, eb + u * estep, cA, cB, cO);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int64_t idx = view_walk_index(w, cA, cB, cO);
            R[u][e] = bf ? (ldg_u16(st.ptr + idx * 2) << 16) : ldg_u32(st.ptr + idx * 4);
            view_walk_next(w, cA, cB, cO);
          }
        }
        return;
      }
#endif
      const bool bcast = v.inner_stride == 0, al4 = v.aligned4 != 0;
      B2_GROUPS B2_SET(R, ld_at(st.ptr, view_index(v, eb + u * estep), bf, bcast, al4))
    };

#define B2_ALL(...)                                                    \
  _Pragma("unroll") for (int u = 0; u < kEwU; ++u)                     \
  _Pragma("unroll") for (int e = 0; e < 4; ++e) { __VA_ARGS__; }
#define B2_SF(S, EXPR)                                                           \
  case kSFlt + ew_fcode(S):                                                              \
    if constexpr (ew_tier_has(TIER, kSFlt + ew_fcode(S))) {                      \
      B2_ALL(const float x = __uint_as_float(X[u][e]), y = __uint_as_float(Y[u][e]); \
             (void)y; X[u][e] = __float_as_uint(EXPR))                           \
    }                                                                            \
    break;
#define B2_SFC(S, EXPR)                                                          \
  case kSFlt + ew_fcode(S):                                                              \
    if constexpr (ew_tier_has(TIER, kSFlt + ew_fcode(S))) {                      \
      B2_ALL(const float x = __uint_as_float(X[u][e]); X[u][e] = __float_as_uint(EXPR)) \
    }                                                                            \
    break;
#define B2_SI(S, EXPR)                                                           \
  case kSInt + ew_icode(S):                                                              \
    if constexpr (ew_tier_has(TIER, kSInt + ew_icode(S))) {                      \
      B2_ALL(const uint32_t x = X[u][e], y = Y[u][e]; (void)y; X[u][e] = (EXPR)) \
    }                                                                            \
    break;
#define B2_SCMP(BASE, CAST)                                                                   \
  case BASE + 0: if constexpr (ew_tier_has(TIER, BASE + 0)) { B2_ALL(X[u][e] = (CAST(X[u][e]) == CAST(Y[u][e])) ? 1u : 0u) } break;         \
  case BASE + 1: if constexpr (ew_tier_has(TIER, BASE + 1)) { B2_ALL(X[u][e] = (CAST(X[u][e]) != CAST(Y[u][e])) ? 1u : 0u) } break;         \
  case BASE + 2: if constexpr (ew_tier_has(TIER, BASE + 2)) { B2_ALL(X[u][e] = (CAST(X[u][e]) < CAST(Y[u][e])) ? 1u : 0u) } break;          \
  case BASE + 3: if constexpr (ew_tier_has(TIER, BASE + 3)) { B2_ALL(X[u][e] = (CAST(X[u][e]) <= CAST(Y[u][e])) ? 1u : 0u) } break;         \
  case BASE + 4: if constexpr (ew_tier_has(TIER, BASE + 4)) { B2_ALL(X[u][e] = (CAST(X[u][e]) > CAST(Y[u][e])) ? 1u : 0u) } break;          \
  case BASE + 5: if constexpr (ew_tier_has(TIER, BASE + 5)) { B2_ALL(X[u][e] = (CAST(X[u][e]) >= CAST(Y[u][e])) ? 1u : 0u) } break;

    for (uint32_t si = 0; si < nsteps; ++si) {
      const EwStep &st = fl.s[si];
      switch (st.code) {
          case kSMovYX: if constexpr (ew_tier_has(TIER, kSMovYX)) { B2_ALL(Y[u][e] = X[u][e]) } break;
          case kSLdXW4: if constexpr (ew_tier_has(TIER, kSLdXW4)) { ld_w4(X, st); } break;
          case kSLdYW4: if constexpr (ew_tier_has(TIER, kSLdYW4)) { ld_w4(Y, st); } break;
          case kSLdXBf: if constexpr (ew_tier_has(TIER, kSLdXBf)) { ld_bf(X, st); } break;
          case kSLdYBf: if constexpr (ew_tier_has(TIER, kSLdYBf)) { ld_bf(Y, st); } break;
          case kSLdXB1: if constexpr (ew_tier_has(TIER, kSLdXB1)) { ld_b1(X, st); } break;
          case kSLdYB1: if constexpr (ew_tier_has(TIER, kSLdYB1)) { ld_b1(Y, st); } break;
          case kSLdXRowW4: if constexpr (ew_tier_has(TIER, kSLdXRowW4)) { ld_row(X, st, false); } break;
          case kSLdYRowW4: if constexpr (ew_tier_has(TIER, kSLdYRowW4)) { ld_row(Y, st, false); } break;
          case kSLdXRowBf: if constexpr (ew_tier_has(TIER, kSLdXRowBf)) { ld_row(X, st, true); } break;
          case kSLdYRowBf: if constexpr (ew_tier_has(TIER, kSLdYRowBf)) { ld_row(Y, st, true); } break;
          case kSLdXColW4: if constexpr (TIER == kTierAll) ld_col(X, st, false); break;
          case kSLdYColW4: if constexpr (TIER == kTierAll) ld_col(Y, st, false); break;
          case kSLdXColBf: if constexpr (TIER == kTierAll) ld_col(X, st, true); break;
          case kSLdYColBf: if constexpr (TIER == kTierAll) ld_col(Y, st, true); break;
          case kSLdXViewW4: if constexpr (TIER == kTierAll) ld_view(X, st, false); break;
          case kSLdYViewW4: if constexpr (TIER == kTierAll) ld_view(Y, st, false); break;
          case kSLdXViewBf: if constexpr (TIER == kTierAll) ld_view(X, st, true); break;
          case kSLdYViewBf: if constexpr (TIER == kTierAll) ld_view(Y, st, true); break;
          case kSStW4: if constexpr (ew_tier_has(TIER, kSStW4)) {
            uint8_t *q = const_cast<uint8_t *>(st.ptr) + static_cast<size_t>(eb) * 4;
            B2_GROUPS stg_v4(q + static_cast<size_t>(u) * estep * 4, make_uint4(X[u][0], X[u][1], X[u][2], X[u][3]));
            break;
          }
          case kSStBf: if constexpr (ew_tier_has(TIER, kSStBf)) {   // X holds bf16-representable values here
            uint8_t *q = const_cast<uint8_t *>(st.ptr) + static_cast<size_t>(eb) * 2;
            B2_GROUPS stg_v2(q + static_cast<size_t>(u) * estep * 2,
                             make_uint2((X[u][0] >> 16) | (X[u][1] & 0xffff0000u), (X[u][2] >> 16) | (X[u][3] & 0xffff0000u)));
            break;
          }
          case kSStB1: if constexpr (ew_tier_has(TIER, kSStB1)) {
            uint8_t *q = const_cast<uint8_t *>(st.ptr) + eb;
            B2_GROUPS stg_u32(q + static_cast<size_t>(u) * estep,
                              (X[u][0] & 0xffu) | ((X[u][1] & 0xffu) << 8) | ((X[u][2] & 0xffu) << 16) | (X[u][3] << 24));
            break;
          }
          case kSQuantBf:
            if constexpr (ew_tier_has(TIER, kSQuantBf)) {
#pragma unroll
              for (int u = 0; u < kEwU; ++u)
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                  const uint32_t w = cvt_bf16x2(__uint_as_float(X[u][e + 1]), __uint_as_float(X[u][e]));
                  X[u][e] = w << 16;
                  X[u][e + 1] = w & 0xffff0000u;
                }
            }
            break;
          case kSAffine: if constexpr (ew_tier_has(TIER, kSAffine)) {
            const float sc = __uint_as_float(st.p2), sh = __uint_as_float(st.p3);
            B2_ALL(X[u][e] = __float_as_uint(affine2(__uint_as_float(X[u][e]), sc, sh)))
            break;
          }
          case kSFill: if constexpr (ew_tier_has(TIER, kSFill)) { const uint32_t f = st.p2; B2_ALL(X[u][e] = f) } break;
          case kSIotaF: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = __float_as_uint(static_cast<float>(eb + u * estep + e))) } break;
          case kSIotaI: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = eb + u * estep + e) } break;
          case kSSelect: if constexpr (ew_tier_has(TIER, kSSelect)) {
            const uint8_t *q = st.ptr + eb;
            B2_GROUPS {
              const uint32_t w = ldg_u32(q + static_cast<size_t>(u) * estep);
              X[u][0] = (w & 0xffu) ? X[u][0] : Y[u][0];
              X[u][1] = (w & 0xff00u) ? X[u][1] : Y[u][1];
              X[u][2] = (w & 0xff0000u) ? X[u][2] : Y[u][2];
              X[u][3] = (w & 0xff000000u) ? X[u][3] : Y[u][3];
            }
            break;
          }
          case kSCvtF2I: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = static_cast<uint32_t>(static_cast<int32_t>(truncf(__uint_as_float(X[u][e]))))) } break;
          case kSCvtF2U: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = static_cast<uint32_t>(static_cast<long long>(truncf(__uint_as_float(X[u][e]))))) } break;
          case kSCvtF2B: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = static_cast<uint32_t>(static_cast<long long>(truncf(__uint_as_float(X[u][e])))) & 0xffu) } break;
          case kSCvtI2F: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = __float_as_uint(static_cast<float>(static_cast<int32_t>(X[u][e])))) } break;
          case kSCvtU2F: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = __float_as_uint(static_cast<float>(X[u][e]))) } break;
          case kSCvtI2B: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] &= 0xffu) } break;
          case kSBNot: if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = X[u][e] == 0u ? 1u : 0u) } break;
          case kSUMax: if constexpr (ew_tier_has(TIER, kSUMax)) { B2_ALL(X[u][e] = max(X[u][e], Y[u][e])) } break;
          case kSUMin: if constexpr (ew_tier_has(TIER, kSUMin)) { B2_ALL(X[u][e] = min(X[u][e], Y[u][e])) } break;
          B2_SCMP(kSCmpF, __uint_as_float)
          B2_SCMP(kSCmpI, static_cast<int32_t>)
          B2_SCMP(kSCmpU, static_cast<uint32_t>)
          B2_SF(kAdd, __fadd_rn(x, y))
          B2_SF(kMul, __fmul_rn(x, y))
          B2_SF(kSubt, __fsub_rn(x, y))
          case kSFlt + ew_fcode(kDiv):
            if constexpr (TIER == kTierAll) { B2_ALL(X[u][e] = __float_as_uint(__fdiv_rn(__uint_as_float(X[u][e]), __uint_as_float(Y[u][e])))) }
            break;
          B2_SF(kMax, np_max(x, y))
          B2_SF(kMin, np_min(x, y))
          B2_SF(kNeg, -x)
          B2_SFC(kExp, expf(x))
          B2_SFC(kLog, logf(x))
          B2_SFC(kSqrt, __fsqrt_rn(x))
          B2_SFC(kRsqrt, __fdiv_rn(1.0f, __fsqrt_rn(x)))
          B2_SFC(kTanh, tanhf(x))
          B2_SF(kAbs, fabsf(x))
          B2_SFC(kFloor, floorf(x))
          B2_SFC(kCeil, ceilf(x))
          B2_SFC(kSign, (x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : x)))
          B2_SF(kGelu, gelu_tanh(x))
#if B2_SHORT
          B2_SF(kPow, pow_f32(x, y))
#endif
          B2_SI(kAdd, x + y)
          B2_SI(kMul, x * y)
          B2_SI(kSubt, x - y)
          B2_SI(kAnd, x & y)
          B2_SI(kOr, x | y)
          B2_SI(kXor, x ^ y)
          B2_SI(kNot, ~x)
          B2_SI(kNeg, 0u - x)
          B2_SI(kAbs, (static_cast<int32_t>(x) < 0 ? 0u - x : x))
          B2_SI(kShl, x << (y & 31u))
          B2_SI(kShrL, x >> (y & 31u))
          B2_SI(kShrA, static_cast<uint32_t>(static_cast<int32_t>(x) >> (y & 31u)))
          B2_SI(kMax, static_cast<uint32_t>(max(static_cast<int32_t>(x), static_cast<int32_t>(y))))
          B2_SI(kMin, static_cast<uint32_t>(min(static_cast<int32_t>(x), static_cast<int32_t>(y))))
          default: break;
      }
    }
#undef B2_SCMP
#undef B2_SI
#undef B2_SFC
#undef B2_SF
#undef B2_ALL
#undef B2_SET
#undef B2_GROUPS
  }
}

__device__ __forceinline__ void ew_entries(const Lane &L, const DEntry *e0, uint32_t chain) {
  const KParams &P = *L.P;
  EwOp *ops = reinterpret_cast<EwOp *>(L.smem + kSmemChain);
  __syncthreads();  // previous users of the chain cache are done
  if (L.tid < chain) {
    ew_decode(P, P.tasks[e0[L.tid].task], &ops[L.tid]);
    ew_build_steps(&ops[L.tid], kSmemChain + L.tid * static_cast<uint32_t>(sizeof(EwOp)));
  }
  __syncthreads();
  EwFlat *fl = reinterpret_cast<EwFlat *>(L.smem + kSmemEwFlat);
  if (L.tid == 0) ew_plan(ops, chain, fl, L.smem_bytes);
  __syncthreads();
  const uint32_t n = P.tasks[e0->task].p[1];
  const uint64_t lo64 = static_cast<uint64_t>(e0->tile_lo) * kEwTs;
  uint64_t hi64 = static_cast<uint64_t>(e0->tile_hi) * kEwTs;
  if (hi64 > n) hi64 = n;
  if (lo64 >= hi64) return;
  const uint32_t lo = static_cast<uint32_t>(lo64), hi = static_cast<uint32_t>(hi64);
  bool vec = true, steps = true;
  for (uint32_t j = 0; j < chain; ++j) {
    vec = vec && (ops[j].flags & kVecPath);
    steps = steps && ops[j].nsteps != kEwNoSteps;
  }
  if (steps) {
    // complete groups on the micro-step machine, the ragged last group (if any) generically
    const uint32_t ngroups = (hi - lo) >> 2;
    const uint32_t trip = L.nthr * kEwU, nfull = ngroups / trip * trip;
    if (ngroups) ew_stage_rows(L, fl);
    switch (fl->tier) {
#define B2_TIER(T)                                                                              \
  case T:                                                                                       \
    if (nfull) ew_steps_run<true, T>(L.tid, L.nthr, lo, 0u, nfull);                             \
    if (nfull < ngroups) ew_steps_run<false, T>(L.tid, L.nthr, lo, nfull, ngroups);             \
    break;
      B2_TIER(kTierF32) B2_TIER(kTierBf) B2_TIER(kTierInt) B2_TIER(kTierHot)
      default:
        if (nfull) ew_steps_run<true, kTierAll>(L.tid, L.nthr, lo, 0u, nfull);
        if (nfull < ngroups) ew_steps_run<false, kTierAll>(L.tid, L.nthr, lo, nfull, ngroups);
        break;
#undef B2_TIER
    }
    if (lo + (ngroups << 2) < hi) ew_chain_run(L, ops, chain, lo + (ngroups << 2), hi);
  } else if (vec) {
    ew_chain_run(L, ops, chain, lo, hi);
  } else {
    // No forwarding on this path (the loader never sets the flags for it): one op
    // at a time, published to the whole lane between ops.
    for (uint32_t j = 0; j < chain; ++j) {
      if (j) { __threadfence_block(); __syncthreads(); }
      ew_scalar_run(L, ops[j], lo, hi);
    }
  }
}

}  // namespace b2
#endif
