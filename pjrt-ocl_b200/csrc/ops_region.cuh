// MAP_REGION: a straight-line micro-program of pure-map ops over <= 8 value
// slots and <= 8 same-length inputs, one load per input and one store.
//
// Replaces vmo_map_region (pjrt_plugin/kernels/ops/region.cl:43-98). Descriptor
// (python/pjrt_ocl/ops/region.py:19-23), u32 words at aux[p0]:
//   [0]=n_in [1]=out_slot [2]=n_micro, in_slot[n_in],
//   n_micro x {kind, dst_slot, a_slot, b_slot, s_bits, t_bits}
// Input k is task field a, b, p2..p7 in that order.
//
// B200 design: the micro-program is copied to shared memory once per entry; each
// thread keeps its slots as 16-byte vectors in its own shared-memory column
// (slot-major, conflict-free), two groups of 4 elements in flight per thread.
#ifndef B2VM_OPS_REGION_CUH_
#define B2VM_OPS_REGION_CUH_

#include "dev_common.cuh"
#include "ops_ew.cuh"

namespace b2 {

constexpr uint32_t kRegionSlots = 8;
constexpr uint32_t kRegionMaxMicro = 96;
constexpr int kRegionU = 2;


static __device__ __noinline__ void region_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const int32_t *x = P.aux + t.p[0];
  const uint32_t n_in = static_cast<uint32_t>(x[0]), out_slot = static_cast<uint32_t>(x[1]) & 7u,
                 n_micro = static_cast<uint32_t>(x[2]);
  const DRegion &dr = *reinterpret_cast<const DRegion *>(P.desc + t.desc);
  // workspace: micro-program copy, then the per-thread slot columns
  uint32_t *prog = reinterpret_cast<uint32_t *>(L.smem + kSmemSys);
  const uint32_t prog_words = n_in + n_micro * 6u;
  uint4 *slots = reinterpret_cast<uint4 *>(L.smem + kSmemSys + ((prog_words * 4u + 15u) & ~15u));
  const uint8_t **in_ptr = reinterpret_cast<const uint8_t **>(L.smem + kSmemPtrs);
  const bool vec = (t.flags & kVecPath) != 0;
  __syncthreads();
  for (uint32_t w = L.tid; w < prog_words; w += L.nthr) prog[w] = static_cast<uint32_t>(x[3 + w]);
  if (L.tid < 8) in_ptr[L.tid] = L.tid < n_in ? resolve(P, dr.in[L.tid]) : nullptr;
  __syncthreads();
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint32_t n = t.p[1], adt = t.adt, dt = t.dt;
  const uint64_t lo64 = static_cast<uint64_t>(tile_lo) * kEwTs;
  uint64_t hi64 = static_cast<uint64_t>(tile_hi) * kEwTs;
  if (hi64 > n) hi64 = n;
  if (lo64 >= hi64) return;
  const uint32_t lo = static_cast<uint32_t>(lo64), hi = static_cast<uint32_t>(hi64);
  const uint32_t ngroups = (hi - lo + 3u) >> 2;
  const uint32_t *micro = prog + n_in;
  const uint32_t col = L.tid, pitch = L.nthr;   // slot s, unroll u -> slots[(u*kRegionSlots + s) * pitch + col]
  for (uint32_t g0 = L.tid; g0 < ngroups; g0 += L.nthr * kRegionU) {
    uint32_t base[kRegionU], vc[kRegionU];
#pragma unroll
    for (int u = 0; u < kRegionU; ++u) {
      const uint32_t g = g0 + u * L.nthr;
      base[u] = lo + (g << 2);
      vc[u] = g < ngroups ? min(4u, hi - base[u]) : 0u;
    }
    for (uint32_t k = 0; k < n_in; ++k) {
      const uint32_t s = prog[k] & 7u;
#pragma unroll
      for (int u = 0; u < kRegionU; ++u) {
        uint32_t v[4] = {0u, 0u, 0u, 0u};
        if (vc[u] == 4u && vec) load4(in_ptr[k], adt, base[u], v);
        else
          for (uint32_t e = 0; e < vc[u]; ++e) v[e] = load1(in_ptr[k], adt, static_cast<int64_t>(base[u]) + e);
        slots[(u * kRegionSlots + s) * pitch + col] = make_uint4(v[0], v[1], v[2], v[3]);
      }
    }
    for (uint32_t m = 0; m < n_micro; ++m) {
      const uint32_t *q = micro + m * 6u;
      const uint32_t kind = q[0], ds = q[1] & 7u, as = q[2] & 7u, bs = q[3] & 7u;
      const float s = __uint_as_float(q[4]), tt = __uint_as_float(q[5]);
      // one dispatch per micro-op, the 8 evaluations inside each case
#define B2_RG(K, EXPR)                                                              \
  case K:                                                                           \
    _Pragma("unroll") for (int u = 0; u < kRegionU; ++u) {                          \
      const uint4 a = slots[(u * kRegionSlots + as) * pitch + col];                 \
      const uint4 b = slots[(u * kRegionSlots + bs) * pitch + col];                 \
      uint4 r;                                                                      \
      { const float x = __uint_as_float(a.x), y = __uint_as_float(b.x); (void)y; r.x = __float_as_uint(EXPR); } \
      { const float x = __uint_as_float(a.y), y = __uint_as_float(b.y); (void)y; r.y = __float_as_uint(EXPR); } \
      { const float x = __uint_as_float(a.z), y = __uint_as_float(b.z); (void)y; r.z = __float_as_uint(EXPR); } \
      { const float x = __uint_as_float(a.w), y = __uint_as_float(b.w); (void)y; r.w = __float_as_uint(EXPR); } \
      slots[(u * kRegionSlots + ds) * pitch + col] = r;                             \
    }                                                                               \
    break;
      switch (kind) {
        B2_RG(kAdd, __fadd_rn(x, y))
        B2_RG(kMul, __fmul_rn(x, y))
        B2_RG(kSubt, __fsub_rn(x, y))
        B2_RG(kDiv, __fdiv_rn(x, y))
        B2_RG(kMax, np_max(x, y))
        B2_RG(kMin, np_min(x, y))
        B2_RG(kNeg, -x)
        B2_RG(kExp, expf(x))
        B2_RG(kLog, logf(x))
        B2_RG(kSqrt, __fsqrt_rn(x))
        B2_RG(kRsqrt, __fdiv_rn(1.0f, __fsqrt_rn(x)))
        B2_RG(kTanh, fast_tanh(x))
        B2_RG(kAbs, fabsf(x))
        B2_RG(kAffine, affine2(x, s, tt))
        B2_RG(kGelu, gelu_tanh(x))
        default:   // copy
          _Pragma("unroll") for (int u = 0; u < kRegionU; ++u)
            slots[(u * kRegionSlots + ds) * pitch + col] = slots[(u * kRegionSlots + as) * pitch + col];
          break;
      }
#undef B2_RG
    }
#pragma unroll
    for (int u = 0; u < kRegionU; ++u) {
      if (!vc[u]) continue;
      const uint4 r = slots[(u * kRegionSlots + out_slot) * pitch + col];
      const uint32_t v[4] = {r.x, r.y, r.z, r.w};
      if (vc[u] == 4u && vec) store4(dst, dt, base[u], v);
      else
        for (uint32_t e = 0; e < vc[u]; ++e) store1(dst, dt, static_cast<int64_t>(base[u]) + e, v[e]);
    }
  }
}

}  // namespace b2
#endif
