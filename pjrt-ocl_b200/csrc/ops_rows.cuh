// Fused row ops: SOFTMAX_SEG and LAYERNORM_SEG over the innermost `seg` elements.
//
// Replaces vmo_softmax_seg / vmo_layernorm_seg (pjrt_plugin/kernels/ops/
// reduce.cl:304-479), which stage one row of at most 1024 floats in local memory.
// Semantics: python/pjrt_ocl/ops/reduce.py:464-475 - softmax = exp(x - max) / sum;
// layernorm core = (x - mean) / sqrt(E[x^2] - mean^2 + eps), one-pass variance.
//
// B200 design: any segment length. Rows whose byte length is a multiple of 16
// (and that fit the staging buffers) are streamed HBM -> shared memory by the
// bulk asynchronous copy engine (TMA, untiled form) with an mbarrier per buffer:
// the lane is split into groups of 4 warps, each group double-buffers its rows,
// so the next row is in flight while the current one is reduced and normalised
// out of shared memory; every element is read from HBM exactly once and written
// once. Other rows (ragged / tiny / huge) take a warp-per-row path that re-reads
// the row through L1/L2.
#ifndef B2VM_OPS_ROWS_CUH_
#define B2VM_OPS_ROWS_CUH_

#include "dev_common.cuh"
#include "ops_ew.cuh"

namespace b2 {

constexpr int kRowGroupWarps = 4;
constexpr int kRowGroupThreads = kRowGroupWarps * kWarp;
constexpr int kRowMaxBufs = 4;     // staged rows per group (at least 2)
constexpr int kRowHdr = 1024;      // mbarriers + reduction slots ahead of the row buffers

// Reduce across the 4 warps of a row group. `slot` = 4 floats of scratch per group.
template <typename F>
__device__ __forceinline__ float group_reduce(float v, F f, float *slot, int barrier_id, uint32_t gl) {
  v = warp_reduce(v, f);
  bar_sync(barrier_id, kRowGroupThreads);          // previous users of `slot` are done
  if ((gl & (kWarp - 1)) == 0) slot[gl / kWarp] = v;
  bar_sync(barrier_id, kRowGroupThreads);
  float r = slot[0];
#pragma unroll
  for (int w = 1; w < kRowGroupWarps; ++w) r = f(r, slot[w]);
  return r;
}

// kRowCarrySum: the lane's carry word (an f32 in the scratch, after the lane totals) takes the sum of the
// values this entry stored. Only this lane ever touches its word; all threads call.
__device__ __forceinline__ void rows_carry_add(const Lane &L, float v) {
  const KParams &P = *L.P;
  v = block_reduce(L, v, [](float a, float c) { return a + c; }, 0.0f);
  if (L.tid == 0) {
    RedScratch *sc = reinterpret_cast<RedScratch *>(P.scratch);
    float *w = reinterpret_cast<float *>(&sc->total[P.n_lanes + L.lane]);
    *w += v;
  }
}

// The same for the paths that do not sum as they store: read the rows back (this lane just wrote them).
__device__ __forceinline__ void rows_carry_reread(const Lane &L, const DTask &t, uint32_t lo, uint32_t hi) {
  const uint8_t *dst = resolve(*L.P, t.ptr[0]);
  const uint32_t seg = t.p[1], dt = t.dt;
  __threadfence_block();
  __syncthreads();
  float s = 0.0f;
  const uint64_t e_lo = static_cast<uint64_t>(lo) * seg, e_hi = static_cast<uint64_t>(hi) * seg;
  for (uint64_t i = e_lo + L.tid; i < e_hi; i += L.nthr) s += __uint_as_float(load1(dst, dt, i));
  rows_carry_add(L, s);
}

// rows [tile_lo, tile_hi) through the staged pipeline. Preconditions (checked by
// the caller): seg*esz % 16 == 0, both buffers 16-byte aligned, 2 buffers per group fit.
__device__ __forceinline__ void rows_staged(const Lane &L, const DTask &t, uint32_t lo, uint32_t hi, bool softmax) {
  const KParams &P = *L.P;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *src = resolve(P, t.ptr[1]);
  const uint32_t seg = t.p[1], adt = t.adt, dt = t.dt;
  const uint32_t in_bytes = seg * dt_size(adt);
  const float eps = __uint_as_float(t.p[2]);
  const uint32_t ngroups = L.nthr / kRowGroupThreads;
  const uint32_t gi = L.tid / kRowGroupThreads, gl = L.tid % kRowGroupThreads;
  uint64_t *bars = reinterpret_cast<uint64_t *>(L.smem + kSmemSys);               // [ngroups][kRowMaxBufs]
  float *slots = reinterpret_cast<float *>(L.smem + kSmemSys + 512);              // [ngroups][4]
  const uint32_t buf_stride = (in_bytes + 127u) & ~127u;
  // as many row buffers per group as fit (2..kRowMaxBufs): rows in flight hide the HBM latency
  const uint32_t nbuf = min(static_cast<uint32_t>(kRowMaxBufs),
                            (L.smem_bytes - kSmemSys - kRowHdr) / (ngroups * buf_stride));
  uint8_t *bufs = L.smem + kSmemSys + kRowHdr + static_cast<size_t>(gi) * nbuf * buf_stride;

  __syncthreads();
  if (L.tid == 0) {
    for (uint32_t i = 0; i < ngroups * kRowMaxBufs; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
  }
  __syncthreads();

  uint64_t *bar = bars + gi * kRowMaxBufs;
  float *slot = slots + gi * 4;
  const bool carry = (t.flags & kRowCarrySum) != 0u;
  float csum = 0.0f;     // this thread's share of the values it stored (kRowCarrySum)
  const int bid = 1 + static_cast<int>(gi);
  const uint32_t first = lo + gi;
  if (gl == 0) {
    for (uint32_t k = 0; k + 1 < nbuf; ++k) {
      const uint32_t r = first + k * ngroups;
      if (r >= hi) break;
      mbar_arrive_expect_tx(&bar[k], in_bytes);
      bulk_g2s(bufs + k * buf_stride, src + static_cast<size_t>(r) * in_bytes, in_bytes, &bar[k]);
    }
  }
  // Every group runs the same trip count so the lane-wide vote below stays uniform;
  // a group that has run out of rows just votes.
  const uint32_t max_it = (hi - lo + ngroups - 1) / ngroups;
  for (uint32_t it = 0; it < max_it; ++it) {
    const uint32_t row = first + it * ngroups;
    const bool active = row < hi;
    const uint32_t b = it % nbuf, parity = (it / nbuf) & 1u;
    bool ok = true;
    if (active && !mbar_wait_bounded(&bar[b], parity, P.wait_budget_ns)) {
      set_status(P, kStTensorTimeout, L.lane, row, t.op);
      ok = false;
    }
    // Lane-wide vote: (1) a copy that never landed abandons the op for everybody,
    // (2) every thread has left the previous iteration, so the other buffer is free.
    if (!__syncthreads_and(ok)) break;
    // refill the buffer that was consumed in the previous iteration
    const uint32_t next = row + (nbuf - 1u) * ngroups;
    const uint32_t nb = (it + nbuf - 1u) % nbuf;
    if (gl == 0 && next < hi) {
      // that buffer was last read through the generic proxy: order those reads
      // before the asynchronous-proxy write that refills it.
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(&bar[nb], in_bytes);
      bulk_g2s(bufs + nb * buf_stride, src + static_cast<size_t>(next) * in_bytes, in_bytes, &bar[nb]);
    }
    if (!active) continue;
    const uint8_t *rowp = bufs + b * buf_stride;
    uint8_t *outp = dst + static_cast<size_t>(row) * seg * dt_size(dt);
    const uint32_t ng = seg >> 2;   // the caller checked seg % 4 == 0
    if (adt == kF32 && dt == kF32) {
      // f32 in, f32 out: the common case, written without any per-element dispatch.
      const float4 *r4 = reinterpret_cast<const float4 *>(rowp);
      float4 *w4 = reinterpret_cast<float4 *>(const_cast<uint8_t *>(rowp));
      float4 *o4 = reinterpret_cast<float4 *>(outp);
      if (softmax) {
        float m = -INFINITY;
        for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
          const float4 v = r4[g];
          m = fmaxf(m, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
        }
        m = group_reduce(m, [](float a, float c) { return fmaxf(a, c); }, slot, bid, gl);
        // exp(x - m) = 2^(x*log2(e) - m*log2(e)): one FMA and one ex2 per element; the
        // result stays in the staged row so the third pass only scales it.
        constexpr float kLog2e = 1.4426950408889634f;
        const float mb = m * kLog2e;
        float s = 0.0f;
        for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
          const float4 v = r4[g];
          float4 e;
          e.x = fast_ex2(fmaf(v.x, kLog2e, -mb));
          e.y = fast_ex2(fmaf(v.y, kLog2e, -mb));
          e.z = fast_ex2(fmaf(v.z, kLog2e, -mb));
          e.w = fast_ex2(fmaf(v.w, kLog2e, -mb));
          s += (e.x + e.y) + (e.z + e.w);
          w4[g] = e;
        }
        s = group_reduce(s, [](float a, float c) { return a + c; }, slot, bid, gl);
        const float rs = __fdiv_rn(1.0f, s);
        for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
          float4 v = r4[g];
          v.x *= rs; v.y *= rs; v.z *= rs; v.w *= rs;
          o4[g] = v;
          csum += (v.x + v.y) + (v.z + v.w);
        }
      } else {
        float s = 0.0f, s2 = 0.0f;
        for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
          const float4 v = r4[g];
          s += (v.x + v.y) + (v.z + v.w);
          s2 = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s2))));
        }
        s = group_reduce(s, [](float a, float c) { return a + c; }, slot, bid, gl);
        s2 = group_reduce(s2, [](float a, float c) { return a + c; }, slot, bid, gl);
        const float inv_n = 1.0f / static_cast<float>(seg);
        const float mu = s * inv_n;
        const float var = __fsub_rn(s2 * inv_n, __fmul_rn(mu, mu));
        const float rden = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
        for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
          float4 v = r4[g];
          v.x = (v.x - mu) * rden; v.y = (v.y - mu) * rden; v.z = (v.z - mu) * rden; v.w = (v.w - mu) * rden;
          o4[g] = v;
          csum += (v.x + v.y) + (v.z + v.w);
        }
      }
    } else if (adt == kBF16 && dt == kBF16 && (seg & 7u) == 0u) {
      // bf16 in, bf16 out: 8 elements per 16-byte word, f32 arithmetic, hardware ex2.
      const uint4 *r8 = reinterpret_cast<const uint4 *>(rowp);
      uint4 *o8 = reinterpret_cast<uint4 *>(outp);
      const uint32_t ng8 = seg >> 3;
      auto unpack8 = [](const uint4 w, float (&f)[8]) {
        f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xffff0000u);
        f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xffff0000u);
        f[4] = __uint_as_float(w.z << 16); f[5] = __uint_as_float(w.z & 0xffff0000u);
        f[6] = __uint_as_float(w.w << 16); f[7] = __uint_as_float(w.w & 0xffff0000u);
      };
      auto pack8 = [](const float (&f)[8]) {
        return make_uint4(cvt_bf16x2(f[1], f[0]), cvt_bf16x2(f[3], f[2]), cvt_bf16x2(f[5], f[4]), cvt_bf16x2(f[7], f[6]));
      };
      auto sum8 = [&](const uint4 w) {     // the eight values as stored (rounded to bf16)
        float f[8];
        unpack8(w, f);
        return ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
      };
      if (softmax) {
        float m = -INFINITY;
        for (uint32_t g = gl; g < ng8; g += kRowGroupThreads) {
          float f[8];
          unpack8(r8[g], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) m = fmaxf(m, f[e]);
        }
        m = group_reduce(m, [](float a, float c) { return fmaxf(a, c); }, slot, bid, gl);
        constexpr float kLog2e = 1.4426950408889634f;
        const float mb = m * kLog2e;
        float sum = 0.0f;
        for (uint32_t g = gl; g < ng8; g += kRowGroupThreads) {
          float f[8];
          unpack8(r8[g], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) sum += fast_ex2(fmaf(f[e], kLog2e, -mb));
        }
        sum = group_reduce(sum, [](float a, float c) { return a + c; }, slot, bid, gl);
        const float rs = __fdiv_rn(1.0f, sum);
        for (uint32_t g = gl; g < ng8; g += kRowGroupThreads) {
          float f[8];
          unpack8(r8[g], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = fast_ex2(fmaf(f[e], kLog2e, -mb)) * rs;
          const uint4 w = pack8(f);
          o8[g] = w;
          if (carry) csum += sum8(w);
        }
      } else {
        float sum = 0.0f, s2 = 0.0f;
        for (uint32_t g = gl; g < ng8; g += kRowGroupThreads) {
          float f[8];
          unpack8(r8[g], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) { sum += f[e]; s2 = fmaf(f[e], f[e], s2); }
        }
        sum = group_reduce(sum, [](float a, float c) { return a + c; }, slot, bid, gl);
        s2 = group_reduce(s2, [](float a, float c) { return a + c; }, slot, bid, gl);
        const float inv_n = 1.0f / static_cast<float>(seg);
        const float mu = sum * inv_n;
        const float var = __fsub_rn(s2 * inv_n, __fmul_rn(mu, mu));
        const float rden = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
        for (uint32_t g = gl; g < ng8; g += kRowGroupThreads) {
          float f[8];
          unpack8(r8[g], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = (f[e] - mu) * rden;
          const uint4 w = pack8(f);
          o8[g] = w;
          if (carry) csum += sum8(w);
        }
      }
    } else if (softmax) {
      float m = -INFINITY;
      for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
        uint32_t v[4];
        load4(rowp, adt, g << 2, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) m = fmaxf(m, __uint_as_float(v[e]));   // a NaN still poisons the row through the sum
      }
      m = group_reduce(m, [](float a, float c) { return np_max(a, c); }, slot, bid, gl);
      // exp(x - max) has a non-positive argument of modest size: the hardware ex2 of
      // x*log2(e) is within ~1e-6 relative there. f32 rows keep it in the staged row (each thread revisits exactly
      // the groups it wrote), so the exponential is evaluated once per element.
      const bool keep = adt == kF32;
      float *roww = reinterpret_cast<float *>(const_cast<uint8_t *>(rowp));
      float s = 0.0f;
      for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
        uint32_t v[4];
        load4(rowp, adt, g << 2, v);
        float ex[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          ex[e] = __expf(__uint_as_float(v[e]) - m);
          s += ex[e];
        }
        if (keep) *reinterpret_cast<float4 *>(roww + (g << 2)) = make_float4(ex[0], ex[1], ex[2], ex[3]);
      }
      s = group_reduce(s, [](float a, float c) { return a + c; }, slot, bid, gl);
      const float rs = __fdiv_rn(1.0f, s);
      for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
        uint32_t v[4];
        load4(rowp, adt, g << 2, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float ev = keep ? __uint_as_float(v[e]) : __expf(__uint_as_float(v[e]) - m);
          v[e] = __float_as_uint(ev * rs);
        }
        store4(outp, dt, g << 2, v);
      }
    } else {
      float s = 0.0f, s2 = 0.0f;
      for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
        uint32_t v[4];
        load4(rowp, adt, g << 2, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float x = __uint_as_float(v[e]);
          s += x;
          s2 = fmaf(x, x, s2);
        }
      }
      s = group_reduce(s, [](float a, float c) { return a + c; }, slot, bid, gl);
      s2 = group_reduce(s2, [](float a, float c) { return a + c; }, slot, bid, gl);
      const float inv_n = 1.0f / static_cast<float>(seg);
      const float mu = s * inv_n;
      const float var = __fsub_rn(s2 * inv_n, __fmul_rn(mu, mu));
      const float rden = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
      for (uint32_t g = gl; g < ng; g += kRowGroupThreads) {
        uint32_t v[4];
        load4(rowp, adt, g << 2, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = __float_as_uint((__uint_as_float(v[e]) - mu) * rden);
        store4(outp, dt, g << 2, v);
      }
    }
  }
  __syncthreads();
  if (L.tid == 0)
    for (uint32_t i = 0; i < ngroups * kRowMaxBufs; ++i) mbar_inval(&bars[i]);
  __syncthreads();
  if (carry) {
    if ((adt == kF32 && dt == kF32) || (adt == kBF16 && dt == kBF16 && (seg & 7u) == 0u)) rows_carry_add(L, csum);
    else rows_carry_reread(L, t, lo, hi);
  }
}

// warp per row; re-reads the row (L1/L2) instead of staging it.
__device__ __forceinline__ void rows_generic(const Lane &L, const DTask &t, uint32_t lo, uint32_t hi, bool softmax) {
  const KParams &P = *L.P;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *src = resolve(P, t.ptr[1]);
  const uint32_t seg = t.p[1], adt = t.adt, dt = t.dt;
  const float eps = __uint_as_float(t.p[2]);
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = L.nthr / kWarp;
  for (uint32_t row = lo + w; row < hi; row += nw) {
    const int64_t base = static_cast<int64_t>(row) * seg;
    if (softmax) {
      float m = -INFINITY;
      for (uint32_t j = l; j < seg; j += kWarp) m = np_max(m, loadf(src, adt, base + j));
      m = warp_reduce(m, [](float a, float c) { return np_max(a, c); });
      float s = 0.0f;
      for (uint32_t j = l; j < seg; j += kWarp) s += expf(loadf(src, adt, base + j) - m);
      s = warp_reduce(s, [](float a, float c) { return a + c; });
      for (uint32_t j = l; j < seg; j += kWarp)
        storef(dst, dt, base + j, __fdiv_rn(expf(loadf(src, adt, base + j) - m), s));
    } else {
      float s = 0.0f, s2 = 0.0f;
      for (uint32_t j = l; j < seg; j += kWarp) {
        const float x = loadf(src, adt, base + j);
        s += x;
        s2 = fmaf(x, x, s2);
      }
      s = warp_reduce(s, [](float a, float c) { return a + c; });
      s2 = warp_reduce(s2, [](float a, float c) { return a + c; });
      const float inv_n = 1.0f / static_cast<float>(seg);
      const float mu = s * inv_n;
      const float var = __fsub_rn(s2 * inv_n, __fmul_rn(mu, mu));
      const float den = __fsqrt_rn(__fadd_rn(var, eps));
      for (uint32_t j = l; j < seg; j += kWarp)
        storef(dst, dt, base + j, __fdiv_rn(__fsub_rn(loadf(src, adt, base + j), mu), den));
    }
  }
}

static __device__ __noinline__ void rows_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi, bool softmax) {
  const KParams &P = *L.P;
  const uint32_t n_out = t.p[0], seg = t.p[1];
  const uint32_t hi = min(tile_hi, n_out);
  if (tile_lo >= hi) return;
  const uint32_t in_bytes = seg * dt_size(t.adt);
  const uint32_t ngroups = L.nthr / kRowGroupThreads;
  const uint32_t buf_stride = (in_bytes + 127u) & ~127u;
  const uint8_t *src = resolve(P, t.ptr[1]);
  uint8_t *dst = resolve(P, t.ptr[0]);
  const bool staged = ngroups >= 1 && L.nthr % kRowGroupThreads == 0 && ngroups <= 15 &&
                      seg >= 1024 && seg % 4 == 0 && in_bytes % 16 == 0 && dt_size(t.adt) <= 4 && dt_size(t.dt) <= 4 &&
                      reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                      static_cast<size_t>(kSmemSys) + kRowHdr + static_cast<size_t>(ngroups) * 2 * buf_stride <= L.smem_bytes;
  if (staged) {
    rows_staged(L, t, tile_lo, hi, softmax);
  } else {
    rows_generic(L, t, tile_lo, hi, softmax);
    if (t.flags & kRowCarrySum) rows_carry_reread(L, t, tile_lo, hi);
  }
}

// kTopRmsRows: what the loader makes of the decomposed RMS norm over bf16 rows
//   xf = f32(x); ss = rowsum(xf * xf); r = 1 / sqrt(ss * s + t); y = bf16((xf * r) * g)
// (convert, multiply, RED_SEG, a MAP_REGION {affine, rsqrt} on the row sums, two multiplies through broadcast views,
// convert: seven tile ops, five phases, four f32 intermediates of the tensor's size). One pass instead: a warp owns a
// row, every lane keeps its W 16-byte words of the row in registers, the row sum is a warp reduction and the scaled
// row leaves as bf16. Same roundings per element as the separate ops (f32 multiply, f32 multiply, round to bf16;
// affine with two roundings, correctly rounded square root and division); the row sum's order differs.
// p[0] rows, p[1] row length (256 W, W = 1, 2, 4 or 8), p[2] / p[4] the affine's s / t (f32 bits), p[3] != 0: g is
// bf16; ptr[0] result, ptr[1] x, ptr[2] g (f32 or bf16, one per column). Entries name elementwise tiles of the result.
template <uint32_t W>
__device__ __forceinline__ void rms_rows_w(const Lane &L, const DTask &t, uint32_t r_lo, uint32_t r_hi) {
  const KParams &P = *L.P;
  const uint4 *x = reinterpret_cast<const uint4 *>(resolve(P, t.ptr[1]));
  uint4 *y = reinterpret_cast<uint4 *>(resolve(P, t.ptr[0]));
  const uint8_t *g = resolve(P, t.ptr[2]);
  const float as = __uint_as_float(t.p[2]), at = __uint_as_float(t.p[4]);
  const bool g16 = t.p[3] != 0u;
  const uint32_t w = L.tid / kWarp, lane = L.tid % kWarp, nw = L.nthr / kWarp;
  auto unpack8 = [](const uint4 q, float (&f)[8]) {
    f[0] = __uint_as_float(q.x << 16); f[1] = __uint_as_float(q.x & 0xffff0000u);
    f[2] = __uint_as_float(q.y << 16); f[3] = __uint_as_float(q.y & 0xffff0000u);
    f[4] = __uint_as_float(q.z << 16); f[5] = __uint_as_float(q.z & 0xffff0000u);
    f[6] = __uint_as_float(q.w << 16); f[7] = __uint_as_float(q.w & 0xffff0000u);
  };
  for (uint32_t row = r_lo + w; row < r_hi; row += nw) {
    const uint4 *xr = x + static_cast<size_t>(row) * (W * kWarp);
    uint4 v[W];
#pragma unroll
    for (uint32_t k = 0; k < W; ++k) v[k] = ldg_v4(xr + k * kWarp + lane);
    float ss = 0.0f;
#pragma unroll
    for (uint32_t k = 0; k < W; ++k) {
      float f[8];
      unpack8(v[k], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = __fadd_rn(ss, __fmul_rn(f[i], f[i]));
    }
    ss = warp_reduce(ss, [](float a, float c) { return a + c; });
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(affine2(ss, as, at)));
    uint4 *yr = y + static_cast<size_t>(row) * (W * kWarp);
#pragma unroll
    for (uint32_t k = 0; k < W; ++k) {
      float f[8], gg[8];
      unpack8(v[k], f);
      if (g16) {      // the gain still in bf16 (its convert to f32 was folded in too)
        unpack8(reinterpret_cast<const uint4 *>(g)[k * kWarp + lane], gg);
      } else {
        const float4 *g4 = reinterpret_cast<const float4 *>(g);
        const float4 ga = g4[(k * kWarp + lane) * 2u], gb = g4[(k * kWarp + lane) * 2u + 1u];
        gg[0] = ga.x; gg[1] = ga.y; gg[2] = ga.z; gg[3] = ga.w; gg[4] = gb.x; gg[5] = gb.y; gg[6] = gb.z; gg[7] = gb.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __fmul_rn(__fmul_rn(f[i], r), gg[i]);
      yr[k * kWarp + lane] = make_uint4(cvt_bf16x2(f[1], f[0]), cvt_bf16x2(f[3], f[2]), cvt_bf16x2(f[5], f[4]), cvt_bf16x2(f[7], f[6]));
    }
  }
}

static __device__ __noinline__ void rms_rows_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const uint32_t rows = t.p[0], d = t.p[1];
  const uint64_t e_lo = static_cast<uint64_t>(tile_lo) * kEwTs, e_hi = min(static_cast<uint64_t>(tile_hi) * kEwTs, static_cast<uint64_t>(rows) * d);
  if (e_lo >= e_hi) return;
  const uint32_t r_lo = static_cast<uint32_t>(e_lo / d), r_hi = static_cast<uint32_t>(e_hi / d);
  switch (d >> 8) {
    case 1: rms_rows_w<1>(L, t, r_lo, r_hi); break;
    case 2: rms_rows_w<2>(L, t, r_lo, r_hi); break;
    case 4: rms_rows_w<4>(L, t, r_lo, r_hi); break;
    case 8: rms_rows_w<8>(L, t, r_lo, r_hi); break;
    default: break;      // the loader only makes the op for these row lengths
  }
}

}  // namespace b2
#endif
