// TILE_MMA, CUDA-core path: batched C[g] = A[g] . B[g] on 128x128 output tiles with
// optional strided operand views and the store epilogue.
//
// Replaces vmo_mma_tile + vmo_mma_epi (pjrt_plugin/kernels/ops/mma.cl:74-96,
// 136-434). Semantics: python/pjrt_ocl/ops/dot.py:206-293 - tile index runs over
// batch x tiles_m x tiles_n; A/B may be read through the gather descriptors at
// p4-1 / p5-1 over the contiguous [G,M,K] / [G,K,N] flat index; the epilogue at
// p6-1 is a micro-program {kind, src, s, t} applied to each accumulator before the
// store (src 1: residual element of p7, src 2: per-column element of p7).
//
// This path takes every dtype (operands are widened to f32 in shared memory, f32
// accumulate with FMA) and every view; it is the f32 route the contraction
// contract allows ("f32 via FFMA") and the fallback for shapes the tensor-core
// path (ops_mma_tc.cuh) does not take.
#ifndef B2VM_OPS_MMA_CUH_
#define B2VM_OPS_MMA_CUH_

#include "dev_common.cuh"
#include "ops_ew.cuh"

namespace b2 {


constexpr int kMmaBK = 16;
constexpr int kMmaPitchA = kMmaT + 4;

__device__ __forceinline__ float mma_epilogue(const KParams &P, const DTask &t, const uint8_t *res, float v,
                                              int64_t g, int64_t r, int64_t c, int64_t M, int64_t N) {
  const int32_t *e = P.aux + (t.p[6] - 1u);
  const int nm = e[0];
  for (int m = 0; m < nm; ++m) {
    const int32_t *q = e + 1 + 4 * m;
    float y = v;
    if (q[1] == 1) y = loadf(res, t.cdt, (g * M + r) * N + c);
    else if (q[1] == 2) y = loadf(res, t.cdt, c);
    v = micro_alu(static_cast<uint32_t>(q[0]), v, y, __int_as_float(q[2]), __int_as_float(q[3]));
  }
  return v;
}

template <int NT>
static __device__ __noinline__ void mma_simt_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  constexpr int TC = NT / 32;          // thread columns
  constexpr int TN = kMmaT / TC;       // output columns per thread
  constexpr int TM = 4;                // output rows per thread (32 thread rows x 4 = 128)
  static_assert(TN % 4 == 0 && TC * TN == static_cast<int>(kMmaT), "thread grid covers the tile");
  const KParams &P = *L.P;
  const DMma &dm = *reinterpret_cast<const DMma *>(P.desc + t.desc);
  const int64_t M = t.p[0], N = t.p[1], K = t.p[2], G = t.p[3] ? t.p[3] : 1;
  const uint32_t adt = t.adt, dt = t.dt;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *A = resolve(P, t.ptr[1]);
  const uint8_t *B = resolve(P, t.ptr[2]);
  const uint8_t *res = t.p[6] ? resolve(P, t.ptr[3]) : nullptr;
  const bool av = t.flags & kViewA, bv = t.flags & kViewB;
  const int64_t tn = (N + kMmaT - 1) / kMmaT, tm = (M + kMmaT - 1) / kMmaT, per = tm * tn;
  float *As = reinterpret_cast<float *>(L.smem + kSmemSys);            // [kMmaBK][kMmaPitchA]
  float *Bs = As + kMmaBK * kMmaPitchA;                                // [kMmaBK][kMmaT]
  const int tr = L.tid / TC, tc = L.tid % TC;
  for (uint32_t tile = tile_lo; tile < tile_hi; ++tile) {
    const int64_t g = tile / per, loc = tile % per;
    const int64_t r0 = (loc / tn) * kMmaT, c0 = (loc % tn) * kMmaT;
    if (g >= G || r0 >= M || c0 >= N) continue;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    for (int64_t k0 = 0; k0 < K; k0 += kMmaBK) {
      __syncthreads();  // the previous block's reads are done
      for (int idx = L.tid; idx < static_cast<int>(kMmaT) * kMmaBK; idx += NT) {
        const int m = idx / kMmaBK, k = idx % kMmaBK;
        float v = 0.0f;
        if (r0 + m < M && k0 + k < K) {
          const int64_t flat = (g * M + r0 + m) * K + k0 + k;
          v = loadf(A, adt, av ? view_index(dm.va, static_cast<uint32_t>(flat)) : flat);
        }
        As[k * kMmaPitchA + m] = v;
      }
      for (int idx = L.tid; idx < static_cast<int>(kMmaT) * kMmaBK; idx += NT) {
        const int k = idx / static_cast<int>(kMmaT), n = idx % static_cast<int>(kMmaT);
        float v = 0.0f;
        if (k0 + k < K && c0 + n < N) {
          const int64_t flat = (g * K + k0 + k) * N + c0 + n;
          v = loadf(B, adt, bv ? view_index(dm.vb, static_cast<uint32_t>(flat)) : flat);
        }
        Bs[k * kMmaT + n] = v;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < kMmaBK; ++k) {
        const float4 a4 = *reinterpret_cast<const float4 *>(&As[k * kMmaPitchA + tr * TM]);
        const float a[TM] = {a4.x, a4.y, a4.z, a4.w};
        float b[TN];
#pragma unroll
        for (int j = 0; j < TN; j += 4) {
          const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[k * kMmaT + tc * TN + j]);
          b[j] = b4.x; b[j + 1] = b4.y; b[j + 2] = b4.z; b[j + 3] = b4.w;
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int64_t r = r0 + tr * TM + i;
      if (r >= M) continue;
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int64_t c = c0 + tc * TN + j;
        if (c >= N) continue;
        float v = acc[i][j];
        if (t.p[6]) v = mma_epilogue(P, t, res, v, g, r, c, M, N);
        storef(dst, dt, (g * M + r) * N + c, v);
      }
    }
  }
}

}  // namespace b2
#endif
