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

// Decode-shaped tasks (DFlash::dec_mode): every (head, query row) tile is worked on by the whole
// lane. LPK = hd / 8 threads share one key: each holds 8 consecutive d of q (pre-scaled by
// scale * log2 e) and reads the same 8 d of the key's K row and V row as one 16-byte load
// each. A warp covers 32 / LPK keys per load and 8 loads per operand and trip (16 loads in
// flight per thread); the lane's warps take trips round-robin, keep their own running (max, sum,
// accumulator) in the base-2 domain, and are merged through shared memory.
template <int HD, bool BF>
static __device__ __noinline__ void flash_decode_tiles(const Lane &L, const DTask &t, const DFlash &df, uint32_t tile_lo,
                                                          int64_t hi, int64_t T, int64_t C, float scale, bool causal) {
  constexpr int LPK = HD / 8;              // threads per key
  constexpr int KPL = 32 / LPK;            // keys per warp-wide load
  constexpr int U = 8;                     // loads in flight per operand
  constexpr int KPT = KPL * U;             // keys per warp trip
  const KParams &P = *L.P;
  uint8_t *out = resolve(P, t.ptr[0]);
  const uint16_t *Q = reinterpret_cast<const uint16_t *>(resolve(P, t.ptr[1]));
  const uint16_t *K = reinterpret_cast<const uint16_t *>(resolve(P, t.ptr[2])) + df.dk_off;
  const uint16_t *V = reinterpret_cast<const uint16_t *>(resolve(P, t.ptr[3])) + df.dv_off;
  constexpr bool bf = BF;
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = L.nthr / kWarp;
  const uint32_t part = l % LPK, sub = l / LPK;
  float *ml = reinterpret_cast<float *>(L.smem + kSmemSys);                          // [nw][2]
  float *os = ml + 2 * 32;                                                           // [nw][HD]
  auto unpack8 = [&](const uint4 &v, float (&f)[8]) {
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = bf ? __uint_as_float(wd[i] << 16) : f16_bits_to_f32(wd[i] & 0xffffu);
      f[2 * i + 1] = bf ? __uint_as_float(wd[i] & 0xffff0000u) : f16_bits_to_f32(wd[i] >> 16);
    }
  };
  const float sl2 = scale * 1.4426950408889634f;
  for (int64_t tile = tile_lo; tile < hi; ++tile) {
    const int64_t g = tile / T, m = tile % T;
    const int64_t c_end = causal ? min(C, m + (C - T) + 1) : C;
    float q[8];
    unpack8(ldg_v4(Q + (g * T + m) * HD + part * 8), q);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] *= sl2;
    const uint16_t *Kg = K + g * df.dk_g + part * 8, *Vg = V + g * df.dv_g + part * 8;
    float m_run = -INFINITY, l_run = 0.0f, o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.0f;
    auto load = [&](uint4 (&kk)[U], uint4 (&vv)[U], int64_t c0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t key = c0 + u * KPL + sub;
        kk[u] = key < c_end ? ldg_v4(Kg + key * df.dk_c) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t key = c0 + u * KPL + sub;
        vv[u] = key < c_end ? ldg_v4(Vg + key * df.dv_c) : make_uint4(0u, 0u, 0u, 0u);
      }
    };
    auto compute = [&](const uint4 (&kk)[U], const uint4 (&vv)[U], int64_t c0) {
      float sc[U], cmax = -INFINITY;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float kf[8];
        unpack8(kk[u], kf);
        float a = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) a = fmaf(q[i], kf[i], a);
#pragma unroll
        for (int d = 1; d < LPK; d <<= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
        sc[u] = (c0 + u * KPL + sub) < c_end ? a : -INFINITY;
        cmax = fmaxf(cmax, sc[u]);
      }
#pragma unroll
      for (int d = LPK; d < 32; d <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, d));
      const float m_new = fmaxf(m_run, cmax);       // finite: the trip's first key exists
      const float alpha = m_run == -INFINITY ? 0.0f : fast_ex2(m_run - m_new);
      m_run = m_new;
      l_run *= alpha;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] *= alpha;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float pr = sc[u] == -INFINITY ? 0.0f : fast_ex2(sc[u] - m_new);
        l_run += pr;
        float vf[8];
        unpack8(vv[u], vf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = fmaf(pr, vf[i], o[i]);
      }
    };
    for (int64_t c0 = static_cast<int64_t>(KPT) * w; c0 < c_end; c0 += static_cast<int64_t>(KPT) * nw) {
      uint4 kk[U], vv[U];
      load(kk, vv, c0);
      compute(kk, vv, c0);
    }
    // the warp's threads hold partial sums over their own keys: add across the key groups
#pragma unroll
    for (int d = LPK; d < 32; d <<= 1) {
      l_run += __shfl_xor_sync(0xffffffffu, l_run, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += __shfl_xor_sync(0xffffffffu, o[i], d);
    }
    __syncthreads();            // the previous tile's merge has read the workspace
    if (l == 0) { ml[2 * w] = m_run; ml[2 * w + 1] = l_run; }
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) os[w * HD + part * 8 + i] = o[i];
    }
    __syncthreads();
    for (int64_t d = L.tid; d < HD; d += L.nthr) {
      float M = -INFINITY;
      for (uint32_t ww = 0; ww < nw; ++ww) M = fmaxf(M, ml[2 * ww]);
      float num = 0.0f, den = 0.0f;
      for (uint32_t ww = 0; ww < nw; ++ww) {
        const float e = ml[2 * ww] == -INFINITY ? 0.0f : fast_ex2(ml[2 * ww] - M);
        num = fmaf(os[ww * HD + d], e, num);
        den = fmaf(ml[2 * ww + 1], e, den);
      }
      storef(out, t.dt, (g * T + m) * HD + d, __fdiv_rn(num, den));
    }
  }
  __syncthreads();
}

// The same decode-shaped task when the K and V rows of a head are contiguous (key pitch == head_dim: a plain
// [H, C, hd] cache): K and V stream through a ring of shared-memory stages filled by bulk asynchronous copies
// (one thread issues them; 256 keys = 32 KB of K + 32 KB of V per stage at head_dim 64, three stages), so that
// two stages are in flight while one is worked on, at no cost in registers. A warp takes 16 keys of every
// stage (4 per load position, as in flash_decode_tiles); the ring runs on across the lane's tiles, so the next
// head's first stages arrive during this head's merge.
template <int HD, bool BF>
static __device__ __noinline__ void flash_decode_ring(const Lane &L, const DTask &t, const DFlash &df, uint32_t tile_lo,
                                                      int64_t hi, int64_t T, int64_t C, float scale, bool causal) {
  constexpr int LPK = HD / 8;              // threads per key
  constexpr int KPL = 32 / LPK;            // keys per warp-wide load
  constexpr uint32_t kDepth = 3;
  constexpr uint32_t kRowB = HD * 2u;      // bytes of one key's row
  const KParams &P = *L.P;
  uint8_t *out = resolve(P, t.ptr[0]);
  const uint16_t *Q = reinterpret_cast<const uint16_t *>(resolve(P, t.ptr[1]));
  const uint8_t *K = reinterpret_cast<const uint8_t *>(reinterpret_cast<const uint16_t *>(resolve(P, t.ptr[2])) + df.dk_off);
  const uint8_t *V = reinterpret_cast<const uint8_t *>(reinterpret_cast<const uint16_t *>(resolve(P, t.ptr[3])) + df.dv_off);
  constexpr bool bf = BF;
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = L.nthr / kWarp;
  const uint32_t part = l % LPK, sub = l / LPK;
  const uint32_t kps = nw * 4u * KPL;      // keys per stage: every warp gets 4 load positions of KPL keys
  const uint32_t stage_b = kps * kRowB;    // bytes of K (and of V) per stage
  float *ml = reinterpret_cast<float *>(L.smem + kSmemSys);                          // [nw][2]
  float *os = ml + 2 * 32;                                                           // [nw][HD]
  uint64_t *full = reinterpret_cast<uint64_t *>(L.smem + kSmemSys + 256 + 4u * 32u * HD);   // after ml / os
  uint64_t *empty = full + 2u * kDepth;           // full[2 b] : K of buffer b has landed, full[2 b + 1] : V
  uint8_t *ring = L.smem + ((kSmemSys + 256 + 4u * 32u * HD + 96 + 127) & ~127u);
  auto unpack8 = [&](const uint4 &v, float (&f)[8]) {
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = bf ? __uint_as_float(wd[i] << 16) : f16_bits_to_f32(wd[i] & 0xffffu);
      f[2 * i + 1] = bf ? __uint_as_float(wd[i] & 0xffff0000u) : f16_bits_to_f32(wd[i] >> 16);
    }
  };
  // the lane's stages, in order: tile by tile, kps keys each (the last of a tile ragged)
  auto c_end_of = [&](int64_t tile) { const int64_t m = tile % T; return causal ? min(C, m + (C - T) + 1) : C; };
  auto stages_of = [&](int64_t tile) { return static_cast<uint32_t>((c_end_of(tile) + kps - 1) / kps); };
  // producer state (thread 0): the next stage to request
  int64_t p_tile = tile_lo;
  uint32_t p_stage = 0, p_seq = 0;
  auto request = [&]() {          // thread 0: issue the copies of the next stage, if any is left
    while (p_tile < hi && p_stage >= stages_of(p_tile)) { ++p_tile; p_stage = 0; }
    if (p_tile >= hi) return;
    const int64_t g = p_tile / T, c_end = c_end_of(p_tile);
    const int64_t k0 = static_cast<int64_t>(p_stage) * kps;
    const uint32_t bytes = static_cast<uint32_t>(min(static_cast<int64_t>(kps), c_end - k0)) * kRowB;
    const uint32_t b = p_seq % kDepth;
    mbar_arrive_expect_tx(&full[2u * b], bytes);
    bulk_g2s(ring + b * 2u * stage_b, K + (g * df.dk_g + k0 * HD) * 2, bytes, &full[2u * b]);
    mbar_arrive_expect_tx(&full[2u * b + 1u], bytes);
    bulk_g2s(ring + b * 2u * stage_b + stage_b, V + (g * df.dv_g + k0 * HD) * 2, bytes, &full[2u * b + 1u]);
    ++p_stage; ++p_seq;
  };
  __syncthreads();
  if (L.tid == 0) {
    for (uint32_t i = 0; i < kDepth; ++i) { mbar_init(&full[2u * i], 1); mbar_init(&full[2u * i + 1u], 1); mbar_init(&empty[i], nw); }
    fence_mbar_init();
    for (uint32_t i = 0; i < kDepth; ++i) request();
  }
  __syncthreads();
  const float sl2 = scale * 1.4426950408889634f;
  uint32_t seq = 0;                // stages consumed so far by this lane (all threads count alike)
  bool ok = true;
  for (int64_t tile = tile_lo; tile < hi && ok; ++tile) {
    const int64_t g = tile / T, m = tile % T;
    const int64_t c_end = c_end_of(tile);
    float q[8];
    unpack8(ldg_v4(Q + (g * T + m) * HD + part * 8), q);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] *= sl2;
    float m_run = -INFINITY, l_run = 0.0f, o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.0f;
    const uint32_t ns = stages_of(tile);
    for (uint32_t sg = 0; sg < ns && ok; ++sg, ++seq) {
      const uint32_t b = seq % kDepth, par = (seq / kDepth) & 1u;
      if (L.tid == 0 && seq >= 1u) {
        // the buffer of the previous stage goes to the stage kDepth - 1 ahead once every warp has left it
        if (mbar_wait_bounded(&empty[(seq - 1u) % kDepth], ((seq - 1u) / kDepth) & 1u, P.wait_budget_ns)) {
          fence_proxy_async_smem();
          request();
        } else {
          set_status(P, kStTensorTimeout, L.lane, static_cast<uint32_t>(tile), kTopFlashAttn);
        }
      }
      if (!mbar_wait_bounded(&full[2u * b], par, P.wait_budget_ns) || !mbar_wait_bounded(&full[2u * b + 1u], par, P.wait_budget_ns)) {
        set_status(P, kStTensorTimeout, L.lane, static_cast<uint32_t>(tile), kTopFlashAttn);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int64_t k0 = static_cast<int64_t>(sg) * kps + w * 4u * KPL;      // this warp's first key of the stage
      if (k0 < c_end) {
        const uint8_t *ks = ring + b * 2u * stage_b + (w * 4u * KPL + sub) * kRowB + part * 16u, *vs = ks + stage_b;
        float sc[4], cmax = -INFINITY;
        uint4 vv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const bool valid = k0 + u * KPL + sub < c_end;
          const uint4 kk = valid ? *reinterpret_cast<const uint4 *>(ks + u * KPL * kRowB) : make_uint4(0u, 0u, 0u, 0u);
          vv[u] = valid ? *reinterpret_cast<const uint4 *>(vs + u * KPL * kRowB) : make_uint4(0u, 0u, 0u, 0u);
          float kf[8];
          unpack8(kk, kf);
          float a = 0.0f;
#pragma unroll
          for (int i = 0; i < 8; ++i) a = fmaf(q[i], kf[i], a);
#pragma unroll
          for (int d = 1; d < LPK; d <<= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
          sc[u] = valid ? a : -INFINITY;
          cmax = fmaxf(cmax, sc[u]);
        }
#pragma unroll
        for (int d = LPK; d < 32; d <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, d));
        const float m_new = fmaxf(m_run, cmax);       // finite: the warp's first key of the stage exists
        const float alpha = m_run == -INFINITY ? 0.0f : fast_ex2(m_run - m_new);
        m_run = m_new;
        l_run *= alpha;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] *= alpha;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float pr = sc[u] == -INFINITY ? 0.0f : fast_ex2(sc[u] - m_new);
          l_run += pr;
          float vf[8];
          unpack8(vv[u], vf);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = fmaf(pr, vf[i], o[i]);
        }
      }
      __syncwarp();
      if (l == 0) mbar_arrive(&empty[b]);
    }
    if (!ok) break;
    // the warp's threads hold partial sums over their own keys: add across the key groups
#pragma unroll
    for (int d = LPK; d < 32; d <<= 1) {
      l_run += __shfl_xor_sync(0xffffffffu, l_run, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += __shfl_xor_sync(0xffffffffu, o[i], d);
    }
    __syncthreads();            // the previous tile's merge has read the workspace
    if (l == 0) { ml[2 * w] = m_run; ml[2 * w + 1] = l_run; }
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) os[w * HD + part * 8 + i] = o[i];
    }
    __syncthreads();
    for (int64_t d = L.tid; d < HD; d += L.nthr) {
      float M = -INFINITY;
      for (uint32_t ww = 0; ww < nw; ++ww) M = fmaxf(M, ml[2 * ww]);
      float num = 0.0f, den = 0.0f;
      for (uint32_t ww = 0; ww < nw; ++ww) {
        const float e = ml[2 * ww] == -INFINITY ? 0.0f : fast_ex2(ml[2 * ww] - M);
        num = fmaf(os[ww * HD + d], e, num);
        den = fmaf(ml[2 * ww + 1], e, den);
      }
      storef(out, t.dt, (g * T + m) * HD + d, __fdiv_rn(num, den));
    }
  }
  __syncthreads();
  if (L.tid == 0 && ok)
    for (uint32_t i = 0; i < kDepth; ++i) { mbar_inval(&full[2u * i]); mbar_inval(&full[2u * i + 1u]); mbar_inval(&empty[i]); }
  __syncthreads();
}

static __device__ __noinline__ void flash_simt_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
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
  if (df.dec_mode && df.dk_c == hd && df.dv_c == hd && L.nthr == 512u &&
      L.smem_bytes >= kSmemSys + 256u + 4u * 32u * static_cast<uint32_t>(hd) + 192u + 3u * 2u * (L.nthr / kWarp) * 4u * (256u / static_cast<uint32_t>(hd)) * static_cast<uint32_t>(hd) * 2u) {
    // contiguous K / V rows: the ring of bulk copies
    if (hd == 64 && adt == kBF16) flash_decode_ring<64, true>(L, t, df, tile_lo, hi, T, C, scale, causal);
    else if (hd == 64) flash_decode_ring<64, false>(L, t, df, tile_lo, hi, T, C, scale, causal);
    else if (adt == kBF16) flash_decode_ring<128, true>(L, t, df, tile_lo, hi, T, C, scale, causal);
    else flash_decode_ring<128, false>(L, t, df, tile_lo, hi, T, C, scale, causal);
    return;
  }
  if (df.dec_mode) {
    if (hd == 64 && adt == kBF16) flash_decode_tiles<64, true>(L, t, df, tile_lo, hi, T, C, scale, causal);
    else if (hd == 64) flash_decode_tiles<64, false>(L, t, df, tile_lo, hi, T, C, scale, causal);
    else if (adt == kBF16) flash_decode_tiles<128, true>(L, t, df, tile_lo, hi, T, C, scale, causal);
    else flash_decode_tiles<128, false>(L, t, df, tile_lo, hi, T, C, scale, causal);
    return;
  }
  if ((hi - static_cast<int64_t>(tile_lo)) * 2 <= static_cast<int64_t>(nw) && hd <= 128) {
    // Few query rows for this lane (a decode step): a warp per row would leave most
    // warps idle and each row's keys in one warp's serial loop. Instead the lane's
    // warps split every row's keys (chunk c0 = 32 w, 32 (w + nw), ...), each keeps
    // its own running (max, sum, accumulator), and the partial results are merged
    // through shared memory: out = sum_w o_w e^{m_w - M} / sum_w l_w e^{m_w - M}.
    float *q_all = reinterpret_cast<float *>(L.smem + kSmemSys);                     // [hd]
    float *ml = q_all + kFlashMaxHd;                                                 // [nw][2]
    float *os = ml + 2 * 32;                                                         // [nw][hd]
    const bool plain = !df.has_q && !df.has_k && !df.has_v && (adt == kBF16 || adt == kF16);
    for (int64_t tile = tile_lo; tile < hi; ++tile) {
      const int64_t g = tile / T, m = tile % T;
      const int64_t qpos = m + (C - T);
      const int64_t c_end = causal ? min(C, qpos + 1) : C;
      __syncthreads();
      for (int64_t d = L.tid; d < hd; d += L.nthr) {
        const int64_t qi = (g * T + m) * hd + d;
        q_all[d] = loadf(Q, adt, df.has_q ? view_index(df.vq, static_cast<uint32_t>(qi)) : qi);
      }
      __syncthreads();
      float m_run = -INFINITY, l_run = 0.0f;
      float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};                                        // columns l, l+32, l+64, l+96
      for (int64_t c0 = static_cast<int64_t>(kWarp) * w; c0 < c_end; c0 += static_cast<int64_t>(kWarp) * nw) {
        const int64_t c = c0 + l;
        float sc = -INFINITY;
        if (c < c_end) {
          float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
          if (plain) {
            const uint16_t *kp = reinterpret_cast<const uint16_t *>(Kp) + g * hd * C + c;
            for (int64_t d = 0; d < hd; d += 4) {        // four independent loads in flight
              const uint32_t k0 = kp[d * C], k1 = kp[(d + 1) * C], k2 = kp[(d + 2) * C], k3 = kp[(d + 3) * C];
              const bool bf = adt == kBF16;
              a0 = fmaf(q_all[d], bf ? bf16_bits_to_f32(k0) : f16_bits_to_f32(k0), a0);
              a1 = fmaf(q_all[d + 1], bf ? bf16_bits_to_f32(k1) : f16_bits_to_f32(k1), a1);
              a2 = fmaf(q_all[d + 2], bf ? bf16_bits_to_f32(k2) : f16_bits_to_f32(k2), a2);
              a3 = fmaf(q_all[d + 3], bf ? bf16_bits_to_f32(k3) : f16_bits_to_f32(k3), a3);
            }
          } else {
            for (int64_t d = 0; d < hd; ++d) {
              const int64_t ki = (g * hd + d) * C + c;
              a0 = fmaf(q_all[d], loadf(Kp, adt, df.has_k ? view_index(df.vk, static_cast<uint32_t>(ki)) : ki), a0);
            }
          }
          sc = ((a0 + a1) + (a2 + a3)) * scale;
        }
        const float cmax = warp_reduce(sc, [](float a, float b) { return fmaxf(a, b); });
        const float m_new = fmaxf(m_run, cmax);
        const float alpha = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
        const float p = (c < c_end) ? expf(sc - m_new) : 0.0f;
        const float psum = warp_reduce(p, [](float a, float b) { return a + b; });
        l_run = l_run * alpha + psum;
        m_run = m_new;
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] *= alpha;
        const int64_t cn = min(static_cast<int64_t>(kWarp), c_end - c0);
        for (int64_t cc = 0; cc < cn; ++cc) {
          const float pc = __shfl_sync(0xffffffffu, p, static_cast<int>(cc));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int64_t d = l + j * kWarp;
            if (d < hd) {
              const int64_t vi = (g * C + c0 + cc) * hd + d;
              o[j] = fmaf(pc, loadf(V, adt, df.has_v ? view_index(df.vv, static_cast<uint32_t>(vi)) : vi), o[j]);
            }
          }
        }
      }
      if (l == 0) { ml[2 * w] = m_run; ml[2 * w + 1] = l_run; }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (l + j * kWarp < hd) os[w * kFlashMaxHd + l + j * kWarp] = o[j];
      __syncthreads();
      for (int64_t d = L.tid; d < hd; d += L.nthr) {
        float M = -INFINITY;
        for (uint32_t ww = 0; ww < nw; ++ww) M = fmaxf(M, ml[2 * ww]);
        float num = 0.0f, den = 0.0f;
        for (uint32_t ww = 0; ww < nw; ++ww) {
          const float e = ml[2 * ww] == -INFINITY ? 0.0f : expf(ml[2 * ww] - M);
          num = fmaf(os[ww * kFlashMaxHd + d], e, num);
          den = fmaf(ml[2 * ww + 1], e, den);
        }
        storef(out, dt, (g * T + m) * hd + d, __fdiv_rn(num, den));
      }
    }
    __syncthreads();
    return;
  }
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
