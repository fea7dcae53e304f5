// MAP_REGION: a straight-line micro-program of pure-map ops over <= 8 value
// slots and <= 8 same-length inputs, one load per input and one store.
//
// Replaces vmo_map_region (pjrt_plugin/kernels/ops/region.cl:43-98). Descriptor
// (python/pjrt_ocl/ops/region.py:19-23), u32 words at aux[p0]:
//   [0]=n_in [1]=out_slot [2]=n_micro, in_slot[n_in],
//   n_micro x {kind, dst_slot, a_slot, b_slot, s_bits, t_bits}
// Input k is task field a, b, p2..p7 in that order.
//
// B200 design: the micro-program is decoded once per entry into shared memory (a dense
// dispatch code, so that the switch is a jump table, and the slot offsets ready to use);
// each thread keeps its slots as 16-byte vectors in its own shared-memory column
// (slot-major, conflict-free) and works on U groups of 4 elements per dispatch: U = 4 when
// the program's slots fit the workspace (the dispatch and the decode of a micro-op are
// paid once per 16 elements), else 2.
#ifndef B2VM_OPS_REGION_CUH_
#define B2VM_OPS_REGION_CUH_

#include "dev_common.cuh"
#include "ops_ew.cuh"

namespace b2 {

constexpr uint32_t kRegionSlots = 8;
constexpr uint32_t kRegionMaxMicro = 96;

// dense dispatch codes (the wire kinds are 0..5, 8..14, 40 and "anything else copies")
enum RegionCode : uint32_t { kRcAdd = 0, kRcMul, kRcSub, kRcDiv, kRcMax, kRcMin, kRcNeg, kRcExp, kRcLog, kRcSqrt, kRcRsqrt,
                             kRcTanh, kRcAbs, kRcAffine, kRcGelu, kRcCopy };
__device__ __forceinline__ uint32_t region_code(uint32_t kind) {
  switch (kind) {
    case kAdd: return kRcAdd; case kMul: return kRcMul; case kSubt: return kRcSub; case kDiv: return kRcDiv;
    case kMax: return kRcMax; case kMin: return kRcMin; case kNeg: return kRcNeg; case kExp: return kRcExp;
    case kLog: return kRcLog; case kSqrt: return kRcSqrt; case kRsqrt: return kRcRsqrt; case kTanh: return kRcTanh;
    case kAbs: return kRcAbs; case kAffine: return kRcAffine; case kGelu: return kRcGelu;
    default: return kRcCopy;
  }
}

// One trip loop for a lane's element range, U groups of 4 elements per thread per trip.
// in_slot[n_in] and micro (shared memory): per micro-op 8 words {code, dst_off, a_off, b_off, s, t, 0, 0} with
// the offsets in uint4 units (slot * pitch).
template <int U>
static __device__ __forceinline__ void region_trips(const Lane &L, const uint32_t *in_slot, const uint32_t *micro, uint4 *slots, const uint8_t *const *in_ptr,
                                                    uint8_t *dst, uint32_t n_in, uint32_t n_micro, uint32_t out_slot, uint32_t n_slots,
                                                    uint32_t lo, uint32_t hi, uint32_t adt, uint32_t dt, bool vec) {
  const uint32_t ngroups = (hi - lo + 3u) >> 2;
  const uint32_t col = L.tid, pitch = L.nthr;   // slot s, unroll u -> slots[(u * n_slots + s) * pitch + col]
  const uint32_t ublock = n_slots * pitch;      // uint4s between the slot sets of two unroll positions
  for (uint32_t g0 = L.tid; g0 < ngroups; g0 += L.nthr * U) {
    uint32_t base[U], vc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t g = g0 + u * L.nthr;
      base[u] = lo + (g << 2);
      vc[u] = g < ngroups ? min(4u, hi - base[u]) : 0u;
    }
    for (uint32_t k = 0; k < n_in; ++k) {
      const uint32_t s = in_slot[k] & 7u;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        uint32_t v[4] = {0u, 0u, 0u, 0u};
        if (vc[u] == 4u && vec) load4(in_ptr[k], adt, base[u], v);
        else
          for (uint32_t e = 0; e < vc[u]; ++e) v[e] = load1(in_ptr[k], adt, static_cast<int64_t>(base[u]) + e);
        slots[u * ublock + s * pitch + col] = make_uint4(v[0], v[1], v[2], v[3]);
      }
    }
    for (uint32_t m = 0; m < n_micro; ++m) {
      const uint4 q = *reinterpret_cast<const uint4 *>(micro + m * 8u);        // code, dst, a, b offsets
      const uint2 st = *reinterpret_cast<const uint2 *>(micro + m * 8u + 4u);  // s, t
      const float s = __uint_as_float(st.x), tt = __uint_as_float(st.y);
      uint4 *pd = slots + q.y + col;
      const uint4 *pa = slots + q.z + col, *pb = slots + q.w + col;
      // one dispatch per micro-op, the 4 U evaluations inside each case
#define B2_RG(K, EXPR)                                                              \
  case K:                                                                           \
    _Pragma("unroll") for (int u = 0; u < U; ++u) {                                 \
      const uint4 a = pa[u * ublock];                                               \
      const uint4 b = pb[u * ublock];                                               \
      uint4 r;                                                                      \
      { const float x = __uint_as_float(a.x), y = __uint_as_float(b.x); (void)y; r.x = __float_as_uint(EXPR); } \
      { const float x = __uint_as_float(a.y), y = __uint_as_float(b.y); (void)y; r.y = __float_as_uint(EXPR); } \
      { const float x = __uint_as_float(a.z), y = __uint_as_float(b.z); (void)y; r.z = __float_as_uint(EXPR); } \
      { const float x = __uint_as_float(a.w), y = __uint_as_float(b.w); (void)y; r.w = __float_as_uint(EXPR); } \
      pd[u * ublock] = r;                                                           \
    }                                                                               \
    break;
#define B2_RG1(K, EXPR)                                                             \
  case K:                                                                           \
    _Pragma("unroll") for (int u = 0; u < U; ++u) {                                 \
      const uint4 a = pa[u * ublock];                                               \
      uint4 r;                                                                      \
      { const float x = __uint_as_float(a.x); r.x = __float_as_uint(EXPR); }        \
      { const float x = __uint_as_float(a.y); r.y = __float_as_uint(EXPR); }        \
      { const float x = __uint_as_float(a.z); r.z = __float_as_uint(EXPR); }        \
      { const float x = __uint_as_float(a.w); r.w = __float_as_uint(EXPR); }        \
      pd[u * ublock] = r;                                                           \
    }                                                                               \
    break;
      switch (q.x) {
        B2_RG(kRcAdd, __fadd_rn(x, y))
        B2_RG(kRcMul, __fmul_rn(x, y))
        B2_RG(kRcSub, __fsub_rn(x, y))
        B2_RG(kRcDiv, __fdiv_rn(x, y))
        B2_RG(kRcMax, np_max(x, y))
        B2_RG(kRcMin, np_min(x, y))
        B2_RG1(kRcNeg, -x)
        B2_RG1(kRcExp, expf(x))
        B2_RG1(kRcLog, logf(x))
        B2_RG1(kRcSqrt, __fsqrt_rn(x))
        B2_RG1(kRcRsqrt, __fdiv_rn(1.0f, __fsqrt_rn(x)))
        B2_RG1(kRcTanh, fast_tanh(x))
        B2_RG1(kRcAbs, fabsf(x))
        B2_RG1(kRcAffine, affine2(x, s, tt))
        B2_RG1(kRcGelu, gelu_tanh(x))
        default:   // copy
          _Pragma("unroll") for (int u = 0; u < U; ++u) pd[u * ublock] = pa[u * ublock];
          break;
      }
#undef B2_RG
#undef B2_RG1
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!vc[u]) continue;
      const uint4 r = slots[u * ublock + out_slot * pitch + col];
      const uint32_t v[4] = {r.x, r.y, r.z, r.w};
      if (vc[u] == 4u && vec) store4(dst, dt, base[u], v);
      else
        for (uint32_t e = 0; e < vc[u]; ++e) store1(dst, dt, static_cast<int64_t>(base[u]) + e, v[e]);
    }
  }
}

static __device__ __noinline__ void region_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const int32_t *x = P.aux + t.p[0];
  const uint32_t n_in = static_cast<uint32_t>(x[0]), out_slot = static_cast<uint32_t>(x[1]) & 7u,
                 n_micro = static_cast<uint32_t>(x[2]);
  const DRegion &dr = *reinterpret_cast<const DRegion *>(P.desc + t.desc);
  // workspace: the decoded micro-program (n_in words, then 8 words per micro-op, 16-byte aligned), then
  // the per-thread slot columns
  uint32_t *prog = reinterpret_cast<uint32_t *>(L.smem + kSmemSys);
  const uint32_t in_words = (n_in + 3u) & ~3u;
  const uint32_t prog_words = in_words + n_micro * 8u;
  uint4 *slots = reinterpret_cast<uint4 *>(L.smem + kSmemSys + prog_words * 4u);
  const uint8_t **in_ptr = reinterpret_cast<const uint8_t **>(L.smem + kSmemPtrs);
  const bool vec = (t.flags & kVecPath) != 0;
  const uint32_t pitch = L.nthr;
  __syncthreads();
  for (uint32_t k = L.tid; k < n_in; k += L.nthr) prog[k] = static_cast<uint32_t>(x[3 + k]);
  for (uint32_t m = L.tid; m < n_micro; m += L.nthr) {
    const int32_t *q = x + 3 + n_in + 6 * m;
    uint32_t *o = prog + in_words + 8u * m;
    o[0] = region_code(static_cast<uint32_t>(q[0]));
    o[1] = (static_cast<uint32_t>(q[1]) & 7u) * pitch;
    o[2] = (static_cast<uint32_t>(q[2]) & 7u) * pitch;
    o[3] = (static_cast<uint32_t>(q[3]) & 7u) * pitch;
    o[4] = static_cast<uint32_t>(q[4]);
    o[5] = static_cast<uint32_t>(q[5]);
    o[6] = 0u; o[7] = 0u;
  }
  if (L.tid < 8) in_ptr[L.tid] = L.tid < n_in ? resolve(P, dr.in[L.tid]) : nullptr;
  __syncthreads();
  // slots in use: 1 + the highest slot any input, micro-op or the output names (read back from the decoded copy)
  uint32_t n_slots = out_slot + 1u;
  for (uint32_t k = 0; k < n_in; ++k) n_slots = max(n_slots, (prog[k] & 7u) + 1u);
  for (uint32_t m = 0; m < n_micro; ++m) {
    const uint4 q = *reinterpret_cast<const uint4 *>(prog + in_words + 8u * m);
    n_slots = max(n_slots, max(q.y, max(q.z, q.w)) / pitch + 1u);
  }
  const uint32_t room = (L.smem_bytes - kSmemSys - prog_words * 4u) / (16u * pitch);     // slot columns that fit
  const bool wide = n_slots * 4u <= room;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint32_t n = t.p[1], adt = t.adt, dt = t.dt;
  const uint64_t lo64 = static_cast<uint64_t>(tile_lo) * kEwTs;
  uint64_t hi64 = static_cast<uint64_t>(tile_hi) * kEwTs;
  if (hi64 > n) hi64 = n;
  if (lo64 >= hi64) return;
  const uint32_t lo = static_cast<uint32_t>(lo64), hi = static_cast<uint32_t>(hi64);
  // 16 elements per dispatch pay when every thread gets them; a short range is spread thinner instead
  if (wide && hi - lo >= 16u * L.nthr) region_trips<4>(L, prog, prog + in_words, slots, in_ptr, dst, n_in, n_micro, out_slot, n_slots, lo, hi, adt, dt, vec);
  else region_trips<2>(L, prog, prog + in_words, slots, in_ptr, dst, n_in, n_micro, out_slot, kRegionSlots, lo, hi, adt, dt, vec);
}

}  // namespace b2
#endif
