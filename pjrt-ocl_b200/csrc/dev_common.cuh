// Device-side helpers shared by every tile op: lane context, buffer-reference
// resolution, dtype conversion, typed scalar access, view indexing, CTA reductions.
#ifndef B2VM_DEV_COMMON_CUH_
#define B2VM_DEV_COMMON_CUH_

#include <limits.h>
#include <math.h>

#include <cuda_fp16.h>

#include "format.h"
#include "ptx.cuh"

// Short-run paths (segments of 2..8 elements, views whose source runs are shorter than 16 bytes, pow with
// constant exponents): compiled only into the builds that carry that family (vm_kernel.cu sets B2_SHORT).
#ifndef B2_SHORT
#define B2_SHORT 1
#endif

namespace b2 {

// Shared-memory map of one lane (CTA). The first kSmemSys bytes are reserved for
// the interpreter and CTA-wide reductions; tile ops carve the rest.
constexpr int kSmemRed = 0;          // 64 x 16 B reduction scratch
constexpr int kSmemPtrs = 512;       // 8 resolved pointers (MAP_REGION inputs)
constexpr int kSmemFlag = 576;       // grid-barrier outcome, broadcast from thread 0
constexpr int kSmemChain = 1024;     // decoded elementwise chain (EwOp[kChainMax])
constexpr int kSmemSys = 8192;
constexpr int kChainMax = 8;

struct Lane {
  const KParams *P;
  uint8_t *smem;       // dynamic shared memory base
  uint32_t smem_bytes;
  uint32_t lane;
  uint32_t tid;
  uint32_t nthr;
};

__device__ __forceinline__ uint8_t *resolve(const KParams &P, BufRef r) {
  return (r & kPortBit) ? static_cast<uint8_t *>(P.io.p[r & (kMaxIoPorts - 1)])
                        : reinterpret_cast<uint8_t *>(static_cast<uintptr_t>(r));
}

// Record the first device-side error and raise the abort flag every wait polls.
__device__ __forceinline__ void set_status(const KParams &P, uint32_t code, uint32_t lane, uint32_t where,
                                           uint32_t detail) {
  if (atomicCAS(&P.sync->status[0], 0u, code) == 0u) {
    P.sync->status[1] = lane;
    P.sync->status[2] = where;
    P.sync->status[3] = detail;
  }
  __threadfence();
  atomicExch(&P.sync->abort, 1u);
}

// ---- dtype conversion ---------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
// round-to-nearest-even, NaN stays NaN (quiet)
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (u >> 16) | 0x0040u;
  return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}
__device__ __forceinline__ uint32_t f32_to_f16_bits(float f) {
  return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(f)));
}
__device__ __forceinline__ float quantize(float v, uint32_t dt) {
  if (dt == kBF16) return bf16_bits_to_f32(f32_to_bf16_bits(v));
  if (dt == kF16) return f16_bits_to_f32(f32_to_f16_bits(v));
  return v;
}
__device__ __forceinline__ bool is_float_dt(uint32_t dt) { return dt == kF32 || dt == kF16 || dt == kBF16; }
__device__ __forceinline__ uint32_t dt_size(uint32_t dt) {
  return dt == kBool ? 1u : (dt == kF16 || dt == kBF16) ? 2u : (dt == kI64 || dt == kF64) ? 8u : 4u;
}

// Typed scalar access in the 32-bit register representation: floats of any
// storage width as f32 bits, i32/u32 as the integer, bool as 0/1.
__device__ __forceinline__ uint32_t load1(const uint8_t *p, uint32_t dt, int64_t i) {
  switch (dt) {
    case kBool: return p[i];
    case kF16: return __float_as_uint(f16_bits_to_f32(reinterpret_cast<const uint16_t *>(p)[i]));
    case kBF16: return static_cast<uint32_t>(reinterpret_cast<const uint16_t *>(p)[i]) << 16;
    default: return reinterpret_cast<const uint32_t *>(p)[i];
  }
}
__device__ __forceinline__ void store1(uint8_t *p, uint32_t dt, int64_t i, uint32_t v) {
  switch (dt) {
    case kBool: p[i] = static_cast<uint8_t>(v); break;
    case kF16: reinterpret_cast<uint16_t *>(p)[i] = static_cast<uint16_t>(f32_to_f16_bits(__uint_as_float(v))); break;
    case kBF16: reinterpret_cast<uint16_t *>(p)[i] = static_cast<uint16_t>(f32_to_bf16_bits(__uint_as_float(v))); break;
    default: reinterpret_cast<uint32_t *>(p)[i] = v; break;
  }
}
__device__ __forceinline__ float loadf(const uint8_t *p, uint32_t dt, int64_t i) {
  return __uint_as_float(load1(p, dt, i));
}
__device__ __forceinline__ void storef(uint8_t *p, uint32_t dt, int64_t i, float v) {
  store1(p, dt, i, __float_as_uint(v));
}

// 4 consecutive elements starting at element i (i % 4 == 0, base 16-byte aligned).
__device__ __forceinline__ void load4(const uint8_t *p, uint32_t dt, int64_t i, uint32_t out[4]) {
  if (dt == kBool) {
    const uint32_t w = *reinterpret_cast<const uint32_t *>(p + i);
    out[0] = w & 0xffu; out[1] = (w >> 8) & 0xffu; out[2] = (w >> 16) & 0xffu; out[3] = w >> 24;
  } else if (dt == kBF16) {
    const uint2 w = *reinterpret_cast<const uint2 *>(p + i * 2);
    out[0] = w.x << 16; out[1] = w.x & 0xffff0000u; out[2] = w.y << 16; out[3] = w.y & 0xffff0000u;
  } else if (dt == kF16) {
    const uint2 w = *reinterpret_cast<const uint2 *>(p + i * 2);
    out[0] = __float_as_uint(f16_bits_to_f32(w.x & 0xffffu)); out[1] = __float_as_uint(f16_bits_to_f32(w.x >> 16));
    out[2] = __float_as_uint(f16_bits_to_f32(w.y & 0xffffu)); out[3] = __float_as_uint(f16_bits_to_f32(w.y >> 16));
  } else {
    const uint4 w = *reinterpret_cast<const uint4 *>(p + i * 4);
    out[0] = w.x; out[1] = w.y; out[2] = w.z; out[3] = w.w;
  }
}
__device__ __forceinline__ void store4(uint8_t *p, uint32_t dt, int64_t i, const uint32_t v[4]) {
  if (dt == kBool) {
    *reinterpret_cast<uint32_t *>(p + i) = (v[0] & 0xffu) | ((v[1] & 0xffu) << 8) | ((v[2] & 0xffu) << 16) | (v[3] << 24);
  } else if (dt == kBF16) {
    uint2 w;
    w.x = f32_to_bf16_bits(__uint_as_float(v[0])) | (f32_to_bf16_bits(__uint_as_float(v[1])) << 16);
    w.y = f32_to_bf16_bits(__uint_as_float(v[2])) | (f32_to_bf16_bits(__uint_as_float(v[3])) << 16);
    *reinterpret_cast<uint2 *>(p + i * 2) = w;
  } else if (dt == kF16) {
    uint2 w;
    w.x = f32_to_f16_bits(__uint_as_float(v[0])) | (f32_to_f16_bits(__uint_as_float(v[1])) << 16);
    w.y = f32_to_f16_bits(__uint_as_float(v[2])) | (f32_to_f16_bits(__uint_as_float(v[3])) << 16);
    *reinterpret_cast<uint2 *>(p + i * 2) = w;
  } else {
    *reinterpret_cast<uint4 *>(p + i * 4) = make_uint4(v[0], v[1], v[2], v[3]);
  }
}

// ---- views -----------------------------------------------------------------------
// Source element index of consumer element i under a collapsed view.
__device__ __forceinline__ int64_t view_index(const DView &v, uint32_t i) {
  int64_t idx = v.off;
  uint32_t rem = i;
  // trip count = rank - 1 (1 for the common row / column broadcasts): a real loop,
  // not a predicated unroll over all kViewDims
#pragma unroll 1
  for (int k = v.rank - 1; k >= 1; --k) {
    const uint32_t d = v.dim[k];
    const uint32_t mh = __umulhi(rem, v.magic[k]);
    const uint32_t q = (((rem - mh) >> 1) + mh) >> v.shift[k];
    idx += static_cast<int64_t>(static_cast<int32_t>(rem - q * d)) * v.stride[k];
    rem = q;
  }
  // i < prod(dim): what is left is the outermost coordinate itself
  if (v.rank > 0) idx += static_cast<int64_t>(rem) * v.stride[0];
  return idx;
}
// Walking a view of rank 1..3 element by element: the coordinates of the first
// element cost the divisions, every following one an increment with carry. The
// fields live in registers, so a run of consecutive consumer elements whose source
// elements are not adjacent (an innermost axis of 3, a strided slice) costs a few
// instructions per element instead of a descriptor walk each.
struct ViewWalk {
  uint32_t dA, dB;          // innermost / middle dimension (0xFFFFFFFF where that level never wraps)
  uint32_t mgA, shA, mgB, shB;
  int64_t stA, stB, stO, off;
  int rank;
};
__device__ __forceinline__ ViewWalk view_walk(const DView &v) {
  ViewWalk w;
  const int r = v.rank;
  w.rank = r;
  w.dA = r >= 2 ? v.dim[r - 1] : 0xFFFFFFFFu;
  w.dB = r >= 3 ? v.dim[1] : 0xFFFFFFFFu;
  w.mgA = v.magic[r - 1]; w.shA = v.shift[r - 1];
  w.mgB = v.magic[1]; w.shB = v.shift[1];
  w.stA = v.stride[r - 1];
  w.stB = r >= 3 ? v.stride[1] : (r == 2 ? v.stride[0] : 0);
  w.stO = r >= 3 ? v.stride[0] : 0;
  w.off = v.off;
  return w;
}
__device__ __forceinline__ void view_walk_seek(const ViewWalk &w, uint32_t i, uint32_t &cA, uint32_t &cB, uint32_t &cO) {
  cA = i; cB = 0u; cO = 0u;
  if (w.rank >= 2) {
    const uint32_t mh = __umulhi(i, w.mgA);
    const uint32_t q = (((i - mh) >> 1) + mh) >> w.shA;
    cA = i - q * w.dA;
    cB = q;
  }
  if (w.rank >= 3) {
    const uint32_t mh = __umulhi(cB, w.mgB);
    const uint32_t q = (((cB - mh) >> 1) + mh) >> w.shB;
    cB -= q * w.dB;
    cO = q;
  }
}
__device__ __forceinline__ int64_t view_walk_index(const ViewWalk &w, uint32_t cA, uint32_t cB, uint32_t cO) {
  return w.off + static_cast<int64_t>(cA) * w.stA + static_cast<int64_t>(cB) * w.stB + static_cast<int64_t>(cO) * w.stO;
}
__device__ __forceinline__ void view_walk_next(const ViewWalk &w, uint32_t &cA, uint32_t &cB, uint32_t &cO) {
  if (++cA == w.dA) {
    cA = 0u;
    if (++cB == w.dB) { cB = 0u; ++cO; }
  }
}

// Uncollapsed aux-pool descriptor {rank, dims[rank], strides[rank], src_off}
// (pjrt_plugin/kernels/ops/ew.cl:174-185): used where a view exceeds 4 dims.
__device__ __forceinline__ int64_t aux_view_index(const int32_t *x, uint32_t i) {
  const int rank = x[0];
  int64_t idx = x[1 + 2 * rank];
  uint32_t rem = i;
  for (int e = rank - 1; e >= 0; --e) {
    const uint32_t d = static_cast<uint32_t>(x[1 + e]);
    const uint32_t q = rem / d;
    idx += static_cast<int64_t>(rem - q * d) * x[1 + rank + e];
    rem = q;
  }
  return idx;
}

// ---- CTA-wide reductions -------------------------------------------------------------
// All threads of the lane must call. `red` = 64 x 8-byte scratch in shared memory.
template <typename T, typename F>
__device__ __forceinline__ T block_reduce(const Lane &L, T v, F f, T identity) {
  T *red = reinterpret_cast<T *>(L.smem + kSmemRed);
  v = warp_reduce(v, f);
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = (L.nthr + kWarp - 1) / kWarp;
  __syncthreads();  // scratch may still be read by a previous reduction
  if (l == 0) red[w] = v;
  __syncthreads();
  T r = (l < nw) ? red[l] : identity;
  r = warp_reduce(r, f);
  return r;  // every thread holds the result
}

}  // namespace b2
#endif
