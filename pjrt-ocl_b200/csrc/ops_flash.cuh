// TILE_FLASH_ATTN, CUDA-core path: one (head, query row) per tile, online softmax.
//
// Replaces vmo_flash_attn (pjrt_plugin/kernels/ops/attention.cl:49-159).
// Semantics: python/pjrt_ocl/ops/attention.py:52-66 - descriptor
// [H, T, C, hd, scale_bits, causal, qv, kv, vv] at aux[p3]; Q is [H,T,hd], K is
// the QK^T matmul's B operand [H,hd,C], V is [H,C,hd], each optionally read
// through a gather view over that flat index; with `causal` the T queries are the
// last T positions of the C-long window (key c is masked when c > m + C - T).
//
// One warp per query row: a lane owns one key of the current 32-key chunk for the
// score, and output columns lane, lane+32, ... for the PV accumulation; masked
// chunks are never visited. Takes every float dtype and every view; the
// tensor-core path (ops_flash_tc.cuh) takes the large 2-byte-float cases.
#ifndef B2VM_OPS_FLASH_CUH_
#define B2VM_OPS_FLASH_CUH_

#include "dev_common.cuh"
#include "ops_ew.cuh"

namespace b2 {


constexpr int kFlashMaxHd = 256;

__device__ __noinline__ void flash_simt_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const int32_t *x = P.aux + t.p[3];
  const int64_t H = x[0], T = x[1], C = x[2], hd = x[3];
  const float scale = __int_as_float(x[4]);
  const bool causal = x[5] != 0;
  const DFlash &df = *reinterpret_cast<const DFlash *>(P.desc + t.desc);
  uint8_t *out = resolve(P, t.ptr[0]);
  const uint8_t *Q = resolve(P, t.ptr[1]);
  const uint8_t *Kp = resolve(P, t.ptr[2]);
  const uint8_t *V = resolve(P, t.ptr[3]);
  const uint32_t adt = t.adt, dt = t.dt;
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = L.nthr / kWarp;
  float *qs = reinterpret_cast<float *>(L.smem + kSmemSys) + static_cast<size_t>(w) * kFlashMaxHd;
  const int64_t hi = min(static_cast<int64_t>(tile_hi), H * T);
  __syncthreads();  // workspace handover from the previous op
  for (int64_t tile = tile_lo + w; tile < hi; tile += nw) {
    const int64_t g = tile / T, m = tile % T;
    const int64_t qpos = m + (C - T);
    const int64_t c_end = causal ? min(C, qpos + 1) : C;
    __syncwarp();
    for (int64_t d = l; d < hd; d += kWarp) {
      const int64_t qi = (g * T + m) * hd + d;
      qs[d] = loadf(Q, adt, df.has_q ? view_index(df.vq, static_cast<uint32_t>(qi)) : qi);
    }
    __syncwarp();
    float m_run = -INFINITY, l_run = 0.0f;
    float o[kFlashMaxHd / kWarp];
#pragma unroll
    for (int j = 0; j < kFlashMaxHd / kWarp; ++j) o[j] = 0.0f;
    for (int64_t c0 = 0; c0 < c_end; c0 += kWarp) {
      const int64_t c = c0 + l;
      float s = -INFINITY;
      if (c < c_end) {
        float acc = 0.0f;
        for (int64_t d = 0; d < hd; ++d) {
          const int64_t ki = (g * hd + d) * C + c;
          acc = fmaf(qs[d], loadf(Kp, adt, df.has_k ? view_index(df.vk, static_cast<uint32_t>(ki)) : ki), acc);
        }
        s = acc * scale;
      }
      const float cmax = warp_reduce(s, [](float a, float b) { return fmaxf(a, b); });
      const float m_new = fmaxf(m_run, cmax);
      const float alpha = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
      const float p = (c < c_end) ? expf(s - m_new) : 0.0f;
      const float psum = warp_reduce(p, [](float a, float b) { return a + b; });
      l_run = l_run * alpha + psum;
      m_run = m_new;
#pragma unroll
      for (int j = 0; j < kFlashMaxHd / kWarp; ++j) o[j] *= alpha;
      const int64_t cn = min(static_cast<int64_t>(kWarp), c_end - c0);
      for (int64_t cc = 0; cc < cn; ++cc) {
        const float pc = __shfl_sync(0xffffffffu, p, static_cast<int>(cc));
#pragma unroll
        for (int j = 0; j < kFlashMaxHd / kWarp; ++j) {
          const int64_t d = l + j * kWarp;
          if (d < hd) {
            const int64_t vi = (g * C + c0 + cc) * hd + d;
            o[j] = fmaf(pc, loadf(V, adt, df.has_v ? view_index(df.vv, static_cast<uint32_t>(vi)) : vi), o[j]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kFlashMaxHd / kWarp; ++j) {
      const int64_t d = l + j * kWarp;
      if (d < hd) storef(out, dt, (g * T + m) * hd + d, __fdiv_rn(o[j], l_run));
    }
  }
}

}  // namespace b2
#endif
