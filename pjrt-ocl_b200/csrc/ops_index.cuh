// Windowed reductions, data-dependent gather / scatter and direct convolution.
//
// Replaces vmo_redwin_tile (pjrt_plugin/kernels/ops/reduce_window.cl:19-70),
// vmo_gather_index_tile (ops/gather.cl:84-152), vmo_scatter_index_tile
// (ops/scatter.cl:56-179) and vmo_conv_tile (ops/conv.cl:23-72). Semantics follow
// the reference's numpy validators (python/pjrt_ocl/ops/reduce_window.py:160-200,
// gather_index.py:154-186, scatter_index.py:216-260, conv.py:160-208): float max /
// min propagate NaN, window padding is the reduction's identity (skipped), start
// indices are clamped to [0, clamp_max].
//
// All four tile like an elementwise op: tile t covers output (or update) elements
// [t * 4096, (t + 1) * 4096). B200 mapping: consecutive threads own consecutive
// elements, so whatever is contiguous in the output is coalesced in the input -
// the channel axis of a channel-last pooling or convolution, the row of an
// embedding lookup. Where that contiguous run is a whole number of 16-byte
// words (and the loader found the layout friendly) a thread moves or reduces a
// 16-byte word at a time. The descriptors (collapsed dims, magic-number
// dividers, resolved index buffer) are built once at load (loader.cc).
#ifndef B2VM_OPS_INDEX_CUH_
#define B2VM_OPS_INDEX_CUH_

#include "dev_common.cuh"
#include "ops_ew.cuh"

namespace b2 {

// n / d for a divisor whose magic pair the loader computed (d >= 1).
__device__ __forceinline__ uint32_t idx_div(uint32_t n, uint32_t d, uint32_t magic, uint32_t shift) {
  if (d == 1u) return n;
  const uint32_t mh = __umulhi(n, magic);
  return (((n - mh) >> 1) + mh) >> shift;
}

// ---- RED_WINDOW -----------------------------------------------------------------
template <typename T, typename F>
__device__ __forceinline__ void red_window_body(const Lane &L, const DWindow &w, T *dst, const T *src, uint32_t lo,
                                                uint32_t hi, T ident, F f) {
  const int rank = static_cast<int>(w.rank);
  if (w.vec4) {
    // the innermost axis is untouched by the window: 4 neighbouring outputs share one window walk
    for (uint32_t i = lo + 4u * L.tid; i < hi; i += 4u * L.nthr) {
      uint32_t rem = i;
      int32_t base[kWinDims];
#pragma unroll
      for (int d = kWinDims - 1; d >= 0; --d) {
        if (d >= rank) continue;
        const uint32_t q = idx_div(rem, w.odim[d], w.omagic[d], w.oshift[d]);
        base[d] = static_cast<int32_t>((rem - q * w.odim[d]) * w.wstr[d]) - w.plow[d];
        rem = q;
      }
      T acc[4] = {ident, ident, ident, ident};
      for (uint32_t wi = 0; wi < w.wcount; ++wi) {
        uint32_t rw = wi;
        int64_t off = 0;
        bool inb = true;
#pragma unroll
        for (int d = kWinDims - 1; d >= 0; --d) {
          if (d >= rank) continue;
          const uint32_t q = rw / w.wdim[d];
          const int32_t ic = base[d] + static_cast<int32_t>(rw - q * w.wdim[d]);
          rw = q;
          inb = inb && ic >= 0 && ic < static_cast<int32_t>(w.idim[d]);
          off += static_cast<int64_t>(ic) * w.istr[d];
        }
        if (!inb) continue;
        const uint4 v = ldg_v4(src + off);
        T x[4];
        memcpy(x, &v, 16);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = f(acc[e], x[e]);
      }
      uint4 o;
      memcpy(&o, acc, 16);
      stg_v4(dst + i, o);
    }
    return;
  }
  for (uint32_t i = lo + L.tid; i < hi; i += L.nthr) {
    uint32_t rem = i;
    int32_t base[kWinDims];
#pragma unroll
    for (int d = kWinDims - 1; d >= 0; --d) {
      if (d >= rank) continue;
      const uint32_t q = idx_div(rem, w.odim[d], w.omagic[d], w.oshift[d]);
      base[d] = static_cast<int32_t>((rem - q * w.odim[d]) * w.wstr[d]) - w.plow[d];
      rem = q;
    }
    T acc = ident;
    for (uint32_t wi = 0; wi < w.wcount; ++wi) {
      uint32_t rw = wi;
      int64_t off = 0;
      bool inb = true;
#pragma unroll
      for (int d = kWinDims - 1; d >= 0; --d) {
        if (d >= rank) continue;
        const uint32_t q = rw / w.wdim[d];
        const int32_t ic = base[d] + static_cast<int32_t>(rw - q * w.wdim[d]);
        rw = q;
        inb = inb && ic >= 0 && ic < static_cast<int32_t>(w.idim[d]);
        off += static_cast<int64_t>(ic) * w.istr[d];
      }
      if (inb) acc = f(acc, src[off]);
    }
    dst[i] = acc;
  }
}

static __device__ __noinline__ void red_window_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const DWindow &w = *reinterpret_cast<const DWindow *>(P.desc + t.desc);
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *src = resolve(P, t.ptr[1]);
  const uint32_t n = t.p[1];
  const uint32_t lo = tile_lo * kEwTs;
  const uint32_t hi = static_cast<uint32_t>(min(static_cast<uint64_t>(tile_hi) * kEwTs, static_cast<uint64_t>(n)));
  if (lo >= hi) return;
  const uint32_t kind = w.kind;
  if (t.dt == kF32) {
    float *d = reinterpret_cast<float *>(dst);
    const float *s = reinterpret_cast<const float *>(src);
    if (kind == kSum) red_window_body(L, w, d, s, lo, hi, 0.0f, [](float a, float b) { return a + b; });
    else if (kind == kRMax) red_window_body(L, w, d, s, lo, hi, -INFINITY, [](float a, float b) { return np_max(a, b); });
    else red_window_body(L, w, d, s, lo, hi, INFINITY, [](float a, float b) { return np_min(a, b); });
  } else if (t.dt == kU32) {
    uint32_t *d = reinterpret_cast<uint32_t *>(dst);
    const uint32_t *s = reinterpret_cast<const uint32_t *>(src);
    if (kind == kSum) red_window_body(L, w, d, s, lo, hi, 0u, [](uint32_t a, uint32_t b) { return a + b; });
    else if (kind == kRMax) red_window_body(L, w, d, s, lo, hi, 0u, [](uint32_t a, uint32_t b) { return max(a, b); });
    else red_window_body(L, w, d, s, lo, hi, 0xffffffffu, [](uint32_t a, uint32_t b) { return min(a, b); });
  } else {   // i32 (the loader admits nothing else)
    int32_t *d = reinterpret_cast<int32_t *>(dst);
    const int32_t *s = reinterpret_cast<const int32_t *>(src);
    if (kind == kSum)
      red_window_body(L, w, d, s, lo, hi, 0, [](int32_t a, int32_t b) { return static_cast<int32_t>(static_cast<uint32_t>(a) + static_cast<uint32_t>(b)); });
    else if (kind == kRMax) red_window_body(L, w, d, s, lo, hi, INT_MIN, [](int32_t a, int32_t b) { return max(a, b); });
    else red_window_body(L, w, d, s, lo, hi, INT_MAX, [](int32_t a, int32_t b) { return min(a, b); });
  }
}

// ---- GATHER_INDEX / SCATTER_INDEX ---------------------------------------------------
// Offset (in elements) into the operand for element i of the output (gather) or of
// the updates (scatter): static part from the element's coordinates, dynamic part
// from the start indices they select.
__device__ __forceinline__ int64_t indexed_offset(const DIndexed &x, const uint8_t *idx, uint32_t i) {
  uint32_t rem = i;
  int64_t off = 0, sb = 0;
  const int rank = static_cast<int>(x.rank);
#pragma unroll
  for (int e = kIdxDims - 1; e >= 0; --e) {
    if (e >= rank) continue;
    const uint32_t q = idx_div(rem, x.dim[e], x.magic[e], x.shift[e]);
    const int64_t c = rem - q * x.dim[e];
    rem = q;
    off += c * x.op_stride[e];
    sb += c * x.si_stride[e];
  }
  for (uint32_t k = 0; k < x.nidx; ++k) {
    const int64_t at = sb + static_cast<int64_t>(k) * x.vec_stride;
    int64_t s = x.is64 ? reinterpret_cast<const long long *>(idx)[at] : reinterpret_cast<const int32_t *>(idx)[at];
    s = s < 0 ? 0 : (s > x.clamp_max[k] ? x.clamp_max[k] : s);
    off += s * x.idx_op_stride[k];
  }
  return off;
}

__device__ __forceinline__ void idx_copy_elem(uint8_t *d, int64_t di, const uint8_t *s, int64_t si, uint32_t esz) {
  switch (esz) {
    case 1: d[di] = s[si]; break;
    case 2: reinterpret_cast<uint16_t *>(d)[di] = reinterpret_cast<const uint16_t *>(s)[si]; break;
    case 8: reinterpret_cast<unsigned long long *>(d)[di] = reinterpret_cast<const unsigned long long *>(s)[si]; break;
    default: reinterpret_cast<uint32_t *>(d)[di] = reinterpret_cast<const uint32_t *>(s)[si]; break;
  }
}

// numpy maximum / minimum on the f32 at *p, atomically (NaN from either side sticks).
__device__ __forceinline__ void atomic_np_f32(float *p, float v, bool is_max) {
  uint32_t *up = reinterpret_cast<uint32_t *>(p);
  uint32_t old = *up;
  for (int tries = 0; tries < (1 << 20); ++tries) {   // bounded: contention on one word ends
    const float cur = __uint_as_float(old);
    const float nv = is_max ? np_max(cur, v) : np_min(cur, v);
    if (__float_as_uint(nv) == old) return;
    const uint32_t seen = atomicCAS(up, old, __float_as_uint(nv));
    if (seen == old) return;
    old = seen;
  }
}

static __device__ __noinline__ void indexed_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi, bool scatter) {
  const KParams &P = *L.P;
  const DIndexed &x = *reinterpret_cast<const DIndexed *>(P.desc + t.desc);
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *a = resolve(P, t.ptr[1]);
  const uint8_t *idx = resolve(P, x.idx);
  const uint32_t n = t.p[1], esz = x.esz;
  const uint32_t lo = tile_lo * kEwTs;
  const uint32_t hi = static_cast<uint32_t>(min(static_cast<uint64_t>(tile_hi) * kEwTs, static_cast<uint64_t>(n)));
  if (lo >= hi) return;
  if (!scatter || x.kind == 0u) {
    // plain moves. x.chunk elements (16 bytes) at a time when the innermost run allows it and both
    // addresses turn out 16-byte aligned; the linear side (gather: dst, scatter: a) is checked once.
    const uint8_t *lin = scatter ? a : dst;
    const uint32_t c = (x.chunk && (reinterpret_cast<uintptr_t>(lin) & 15u) == 0) ? x.chunk : 1u;
    for (uint32_t i = lo + c * L.tid; i < hi; i += c * L.nthr) {
      const int64_t off = indexed_offset(x, idx, i);
      const uint8_t *sp = scatter ? a + static_cast<size_t>(i) * esz : a + off * static_cast<int64_t>(esz);
      uint8_t *dp = scatter ? dst + off * static_cast<int64_t>(esz) : dst + static_cast<size_t>(i) * esz;
      if (c > 1u && i + c <= hi && ((reinterpret_cast<uintptr_t>(sp) | reinterpret_cast<uintptr_t>(dp)) & 15u) == 0) {
        stg_v4(dp, ldg_v4(sp));
      } else {
        const uint32_t m = min(c, hi - i);   // the run is contiguous on both sides (stride 1)
        for (uint32_t e = 0; e < m; ++e) idx_copy_elem(dp, e, sp, e, esz);
      }
    }
    return;
  }
  // combining scatter: one atomic per update element (4-byte types only; the loader checked)
  const bool is_max = x.kind == 2u;
  for (uint32_t i = lo + L.tid; i < hi; i += L.nthr) {
    const int64_t off = indexed_offset(x, idx, i);
    if (t.dt == kF32) {
      float *d = reinterpret_cast<float *>(dst) + off;
      const float v = reinterpret_cast<const float *>(a)[i];
      if (x.kind == 1u) atomicAdd(d, v);
      else atomic_np_f32(d, v, is_max);
    } else if (t.dt == kU32) {
      uint32_t *d = reinterpret_cast<uint32_t *>(dst) + off;
      const uint32_t v = reinterpret_cast<const uint32_t *>(a)[i];
      if (x.kind == 1u) atomicAdd(d, v);
      else if (is_max) atomicMax(d, v);
      else atomicMin(d, v);
    } else {
      int32_t *d = reinterpret_cast<int32_t *>(dst) + off;
      const int32_t v = reinterpret_cast<const int32_t *>(a)[i];
      if (x.kind == 1u) atomicAdd(d, v);
      else if (is_max) atomicMax(d, v);
      else atomicMin(d, v);
    }
  }
}

// ---- CONV ---------------------------------------------------------------------------------
// out[b, o.., oc] = sum over window taps and input channels of in[b, o*stride + tap*dil - pad, ic]
// * w[tap, ic, oc]. Consecutive threads own consecutive output channels: the
// weight reads of a warp are one coalesced line per (tap, ic) and the input value
// is one broadcast load. With Cout a multiple of 4 a thread carries 4 channels
// (16-byte weight loads, 4 accumulators).
template <int V>
__device__ __forceinline__ void conv_body(const Lane &L, const DConv &c, float *dst, const float *in, const float *wt,
                                          uint32_t lo, uint32_t hi) {
  const int sdim = static_cast<int>(c.sdim);
  const uint32_t cin = c.cin, cout = c.cout;
  for (uint32_t i = lo + V * L.tid; i < hi; i += V * L.nthr) {
    uint32_t rem = i / cout;
    const uint32_t oc = i - rem * cout;
    int32_t base[4];
#pragma unroll
    for (int d = 3; d >= 0; --d) {
      if (d >= sdim) continue;
      const uint32_t q = rem / c.osp[d];
      base[d] = static_cast<int32_t>((rem - q * c.osp[d]) * c.str[d]) - c.plow[d];
      rem = q;
    }
    const float *inb = in + static_cast<int64_t>(rem) * c.ibatch;
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.0f;
    for (uint32_t w = 0; w < c.wcount; ++w) {
      uint32_t rw = w;
      int64_t off = 0;
      bool ok = true;
#pragma unroll
      for (int d = 3; d >= 0; --d) {
        if (d >= sdim) continue;
        const uint32_t q = rw / c.win[d];
        const int32_t ic = base[d] + static_cast<int32_t>((rw - q * c.win[d]) * c.dil[d]);
        rw = q;
        ok = ok && ic >= 0 && ic < static_cast<int32_t>(c.isp[d]);
        off += static_cast<int64_t>(ic) * c.istr[d];
      }
      if (!ok) continue;
      const float *ip = inb + off;
      const float *wp = wt + (static_cast<int64_t>(w) * cin) * cout + oc;
      for (uint32_t ch = 0; ch < cin; ++ch) {
        const float xv = ip[ch];
        if (V == 4) {
          const uint4 wv = ldg_v4(wp + static_cast<int64_t>(ch) * cout);
          acc[0] = fmaf(xv, __uint_as_float(wv.x), acc[0]);
          acc[1] = fmaf(xv, __uint_as_float(wv.y), acc[1]);
          acc[2] = fmaf(xv, __uint_as_float(wv.z), acc[2]);
          acc[3] = fmaf(xv, __uint_as_float(wv.w), acc[3]);
        } else {
          acc[0] = fmaf(xv, wp[static_cast<int64_t>(ch) * cout], acc[0]);
        }
      }
    }
    if (V == 4) stg_v4(dst + i, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])));
    else dst[i] = acc[0];
  }
}

static __device__ __noinline__ void conv_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const DConv &c = *reinterpret_cast<const DConv *>(P.desc + t.desc);
  float *dst = reinterpret_cast<float *>(resolve(P, t.ptr[0]));
  const float *in = reinterpret_cast<const float *>(resolve(P, t.ptr[1]));
  const float *wt = reinterpret_cast<const float *>(resolve(P, t.ptr[2]));
  const uint32_t n = t.p[1];
  const uint32_t lo = tile_lo * kEwTs;
  const uint32_t hi = static_cast<uint32_t>(min(static_cast<uint64_t>(tile_hi) * kEwTs, static_cast<uint64_t>(n)));
  if (lo >= hi) return;
  const bool v4 = c.cout % 4u == 0u && ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(wt)) & 15u) == 0;
  if (v4) conv_body<4>(L, c, dst, in, wt, lo, hi);
  else conv_body<1>(L, c, dst, in, wt, lo, hi);
}

}  // namespace b2
#endif
