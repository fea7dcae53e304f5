// Reduction tile ops: RED_PART / RED_COMB (two-phase full reduce), RED_SEG
// (innermost-segment reduce, incl. the GEMV "dot mode") and RED_STRIDED
// (interior / prefix axis block).
//
// Replaces vmo_reduce_part_tile / vmo_reduce_comb_tile / vmo_redseg_tile /
// vmo_redstrided_tile (pjrt_plugin/kernels/ops/reduce.cl:45-281,488-549).
// Semantics: python/pjrt_ocl/ops/reduce.py:252-266,307-326,372-382,432-444.
// Kinds 0 sum 1 max 2 min 3 prod 4 and 5 or 6 xor; floats accumulate in f32 with
// warp-shuffle trees (any association is within the f32 tolerance), integers are
// exact in any order, float max/min propagate NaN like numpy.
//
// B200 design: instead of one local-memory tree per segment, the cooperating
// group scales with the segment: one thread per segment for tiny segments (the
// 16.7 M segments of 3 of the n-body step stay coalesced), one warp per segment
// with 16-byte lane loads up to 16 K elements, the whole lane beyond.
#ifndef B2VM_OPS_REDUCE_CUH_
#define B2VM_OPS_REDUCE_CUH_

#include "dev_common.cuh"
#include "ops_ew.cuh"

namespace b2 {

__device__ __forceinline__ float red_f(uint32_t kind, float a, float b) {
  switch (kind) {
    case kSum: return a + b;
    case kRMax: return np_max(a, b);
    case kRMin: return np_min(a, b);
    default: return a * b;
  }
}
__device__ __forceinline__ float red_f_identity(uint32_t kind) {
  return kind == kSum ? 0.0f : kind == kProd ? 1.0f : kind == kRMax ? -INFINITY : INFINITY;
}
// 32-bit integer / bool accumulators (dt decides signedness of max/min)
__device__ __forceinline__ uint32_t red_i(uint32_t kind, uint32_t dt, uint32_t a, uint32_t b) {
  switch (kind) {
    case kSum: return a + b;
    case kProd: return a * b;
    case kRMax: return dt == kI32 ? static_cast<uint32_t>(max(static_cast<int32_t>(a), static_cast<int32_t>(b))) : max(a, b);
    case kRMin: return dt == kI32 ? static_cast<uint32_t>(min(static_cast<int32_t>(a), static_cast<int32_t>(b))) : min(a, b);
    case kRAnd: return a & b;
    case kROr: return a | b;
    default: return a ^ b;
  }
}
__device__ __forceinline__ uint32_t red_i_identity(uint32_t kind, uint32_t dt) {
  switch (kind) {
    case kSum: case kROr: case kRXor: return 0u;
    case kProd: return 1u;
    case kRMax: return dt == kI32 ? 0x80000000u : 0u;
    case kRMin: return dt == kI32 ? 0x7fffffffu : (dt == kBool ? 1u : 0xffffffffu);
    default: return dt == kBool ? 1u : 0xffffffffu;  // and
  }
}
__device__ __forceinline__ long long red_l(uint32_t kind, long long a, long long b) {
  switch (kind) {
    case kSum: return static_cast<long long>(static_cast<unsigned long long>(a) + static_cast<unsigned long long>(b));
    case kProd: return static_cast<long long>(static_cast<unsigned long long>(a) * static_cast<unsigned long long>(b));
    case kRMax: return a > b ? a : b;
    case kRMin: return a < b ? a : b;
    case kRAnd: return a & b;
    case kROr: return a | b;
    default: return a ^ b;
  }
}
__device__ __forceinline__ long long red_l_identity(uint32_t kind) {
  switch (kind) {
    case kSum: case kROr: case kRXor: return 0;
    case kProd: return 1;
    case kRMax: return LLONG_MIN;
    case kRMin: return LLONG_MAX;
    default: return -1;
  }
}
__device__ __forceinline__ double red_d(uint32_t kind, double a, double b) {
  switch (kind) {
    case kSum: return a + b;
    case kRMax: return (a != a || b != b) ? nan("") : fmax(a, b);
    case kRMin: return (a != a || b != b) ? nan("") : fmin(a, b);
    default: return a * b;
  }
}

// A 64-bit accumulator that holds whichever representation `dt` needs, so the
// drivers below are written once. f32-class and 32-bit integers use the low word.
struct Acc {
  unsigned long long bits;
};
__device__ __forceinline__ Acc acc_identity(uint32_t kind, uint32_t dt) {
  Acc a;
  if (is_float_dt(dt)) a.bits = __float_as_uint(red_f_identity(kind));
  else if (dt == kF64) a.bits = __double_as_longlong(static_cast<double>(red_f_identity(kind)));
  else if (dt == kI64) a.bits = static_cast<unsigned long long>(red_l_identity(kind));
  else a.bits = red_i_identity(kind, dt);
  return a;
}
__device__ __forceinline__ Acc acc_load(const uint8_t *p, uint32_t dt, int64_t i) {
  Acc a;
  if (dt == kF64 || dt == kI64) a.bits = reinterpret_cast<const unsigned long long *>(p)[i];
  else a.bits = load1(p, dt, i);
  return a;
}
__device__ __forceinline__ Acc acc_combine(uint32_t kind, uint32_t dt, Acc a, Acc b) {
  Acc r;
  if (is_float_dt(dt))
    r.bits = __float_as_uint(red_f(kind, __uint_as_float(static_cast<uint32_t>(a.bits)), __uint_as_float(static_cast<uint32_t>(b.bits))));
  else if (dt == kF64)
    r.bits = __double_as_longlong(red_d(kind, __longlong_as_double(a.bits), __longlong_as_double(b.bits)));
  else if (dt == kI64)
    r.bits = static_cast<unsigned long long>(red_l(kind, static_cast<long long>(a.bits), static_cast<long long>(b.bits)));
  else
    r.bits = red_i(kind, dt, static_cast<uint32_t>(a.bits), static_cast<uint32_t>(b.bits));
  return r;
}
__device__ __forceinline__ void acc_store(uint8_t *p, uint32_t dt, int64_t i, Acc a) {
  if (dt == kF64 || dt == kI64) reinterpret_cast<unsigned long long *>(p)[i] = a.bits;
  else store1(p, dt, i, static_cast<uint32_t>(a.bits));
}
__device__ __forceinline__ Acc acc_shfl_xor(Acc a, int o) {
  Acc r;
  r.bits = __shfl_xor_sync(0xffffffffu, a.bits, o);
  return r;
}
__device__ __forceinline__ Acc acc_warp_reduce(uint32_t kind, uint32_t dt, Acc a) {
#pragma unroll
  for (int o = kWarp / 2; o > 0; o >>= 1) a = acc_combine(kind, dt, a, acc_shfl_xor(a, o));
  return a;
}
// All threads of the lane call; every thread gets the result.
__device__ __forceinline__ Acc acc_block_reduce(const Lane &L, uint32_t kind, uint32_t dt, Acc a) {
  unsigned long long *red = reinterpret_cast<unsigned long long *>(L.smem + kSmemRed);
  a = acc_warp_reduce(kind, dt, a);
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = (L.nthr + kWarp - 1) / kWarp;
  __syncthreads();
  if (l == 0) red[w] = a.bits;
  __syncthreads();
  Acc r = acc_identity(kind, dt);
  if (l < nw) r.bits = red[l];
  return acc_warp_reduce(kind, dt, r);
}

// Combine functors over the 32-bit register representation.
struct RFSum { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return __float_as_uint(__uint_as_float(a) + __uint_as_float(b)); } };
struct RFProd { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return __float_as_uint(__uint_as_float(a) * __uint_as_float(b)); } };
struct RFMax { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return __float_as_uint(np_max(__uint_as_float(a), __uint_as_float(b))); } };
struct RFMin { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return __float_as_uint(np_min(__uint_as_float(a), __uint_as_float(b))); } };
// Sums whose stream is the 16-bit source of a convert: a 32-bit word holds two elements, folded on the way in.
struct RFSumBf {
  static __device__ __forceinline__ uint32_t pre(uint32_t w) { return __float_as_uint(__uint_as_float(w << 16) + __uint_as_float(w & 0xffff0000u)); }
  static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return __float_as_uint(__uint_as_float(a) + __uint_as_float(b)); }
};
struct RFSumF16 {
  static __device__ __forceinline__ uint32_t pre(uint32_t w) { return __float_as_uint(f16_bits_to_f32(w & 0xffffu) + f16_bits_to_f32(w >> 16)); }
  static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return __float_as_uint(__uint_as_float(a) + __uint_as_float(b)); }
};
struct RISum { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return a + b; } };
struct RIProd { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return a * b; } };
struct RIAnd { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return a & b; } };
struct RIOr { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return a | b; } };
struct RIXor { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return a ^ b; } };
struct RIMaxS { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return static_cast<uint32_t>(max(static_cast<int32_t>(a), static_cast<int32_t>(b))); } };
struct RIMinS { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return static_cast<uint32_t>(min(static_cast<int32_t>(a), static_cast<int32_t>(b))); } };
struct RIMaxU { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return max(a, b); } };
struct RIMinU { static __device__ __forceinline__ uint32_t pre(uint32_t w) { return w; } static __device__ __forceinline__ uint32_t f(uint32_t a, uint32_t b) { return min(a, b); } };

// Groups of 4 elements [g_lo, g_hi), strided over `nthreads`; DOT multiplies by
// the shared vector at element (4g - dbase) first (GEMV mode).
template <typename C, bool DOT>
__device__ __forceinline__ uint32_t reduce_vec32(const uint8_t *p, uint32_t dt, int64_t g_lo, int64_t g_hi,
                                                 uint32_t rank, uint32_t nthreads, uint32_t ident,
                                                 const uint8_t *dotvec, int64_t dbase) {
  constexpr int U = 8;   // 16-byte loads in flight per thread
  uint32_t acc[U];
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = ident;
  int64_t g = g_lo + rank;
  const int64_t step = nthreads;
  if (!DOT && dt_size(dt) == 4u && g + (U - 1) * step < g_hi) {
    // 4-byte elements: software-pipelined, the next trip's U loads are issued before
    // this trip's values are combined, so 2 U loads per thread are in flight
    const uint4 *q = reinterpret_cast<const uint4 *>(p);
    uint4 a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) a[u] = q[g + u * step];
    g += U * step;
    for (; g + (U - 1) * step < g_hi; g += U * step) {
#pragma unroll
      for (int u = 0; u < U; ++u) b[u] = q[g + u * step];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        acc[u] = C::f(C::f(acc[u], a[u].x), C::f(a[u].y, C::f(a[u].z, a[u].w)));
        a[u] = b[u];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u] = C::f(C::f(acc[u], a[u].x), C::f(a[u].y, C::f(a[u].z, a[u].w)));
  }
  for (; g + (U - 1) * step < g_hi; g += U * step) {
    uint32_t v[U][4], w[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) load4(p, dt, (g + u * step) << 2, v[u]);
    if (DOT) {
#pragma unroll
      for (int u = 0; u < U; ++u) load4(dotvec, dt, ((g + u * step) << 2) - dbase, w[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t x = DOT ? __float_as_uint(__uint_as_float(v[u][e]) * __uint_as_float(w[u][e])) : v[u][e];
        acc[u] = C::f(acc[u], x);
      }
  }
  for (; g < g_hi; g += step) {
    uint32_t v[4], w[4];
    load4(p, dt, g << 2, v);
    if (DOT) load4(dotvec, dt, (g << 2) - dbase, w);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t x = DOT ? __float_as_uint(__uint_as_float(v[e]) * __uint_as_float(w[e])) : v[e];
      acc[0] = C::f(acc[0], x);
    }
  }
  return C::f(C::f(C::f(acc[0], acc[1]), C::f(acc[2], acc[3])), C::f(C::f(acc[4], acc[5]), C::f(acc[6], acc[7])));
}

// Reduce elements [lo, hi) of `p`, strided over `nthreads` cooperating threads
// (this thread is `rank`); 16-byte loads when the run is 4-aligned f32-class.
__device__ __forceinline__ Acc reduce_run(const uint8_t *p, uint32_t dt, uint32_t kind, int64_t lo, int64_t hi,
                                          uint32_t rank, uint32_t nthreads, const uint8_t *dotvec, int64_t dot_off) {
  Acc acc = acc_identity(kind, dt);
  const uint32_t esz = dt_size(dt);
  const bool vec = esz <= 4 && (lo % 4 == 0) && (reinterpret_cast<uintptr_t>(p) % 16 == 0) &&
                   (!dotvec || ((dot_off % 4 == 0) && reinterpret_cast<uintptr_t>(dotvec) % 16 == 0));
  if (vec) {
    const int64_t g_lo = lo >> 2, g_hi = hi >> 2;
    // The streaming part runs in a loop specialised on the combine (no per-element
    // dispatch) with four 16-byte loads in flight per thread.
    const int64_t dbase = lo - dot_off;
    uint32_t r;
    const bool fl = is_float_dt(dt);
    const uint32_t ident = static_cast<uint32_t>(acc.bits);
    if (fl && dotvec) r = reduce_vec32<RFSum, true>(p, dt, g_lo, g_hi, rank, nthreads, ident, dotvec, dbase);
    else if (fl && kind == kSum) r = reduce_vec32<RFSum, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (fl && kind == kRMax) r = reduce_vec32<RFMax, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (fl && kind == kRMin) r = reduce_vec32<RFMin, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (fl) r = reduce_vec32<RFProd, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (kind == kSum) r = reduce_vec32<RISum, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (kind == kProd) r = reduce_vec32<RIProd, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (kind == kRAnd) r = reduce_vec32<RIAnd, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (kind == kROr) r = reduce_vec32<RIOr, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (kind == kRXor) r = reduce_vec32<RIXor, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (kind == kRMax && dt == kI32) r = reduce_vec32<RIMaxS, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (kind == kRMax) r = reduce_vec32<RIMaxU, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else if (dt == kI32) r = reduce_vec32<RIMinS, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    else r = reduce_vec32<RIMinU, false>(p, dt, g_lo, g_hi, rank, nthreads, ident, nullptr, 0);
    acc.bits = r;
    for (int64_t i = (g_hi << 2) + rank; i < hi; i += nthreads) {
      Acc x = acc_load(p, dt, i);
      if (dotvec) x.bits = __float_as_uint(__uint_as_float(static_cast<uint32_t>(x.bits)) * loadf(dotvec, dt, i - lo + dot_off));
      acc = acc_combine(kind, dt, acc, x);
    }
    return acc;
  }
  for (int64_t i = lo + rank; i < hi; i += nthreads) {
    Acc x = acc_load(p, dt, i);
    if (dotvec) x.bits = __float_as_uint(__uint_as_float(static_cast<uint32_t>(x.bits)) * loadf(dotvec, dt, i - lo + dot_off));
    acc = acc_combine(kind, dt, acc, x);
  }
  return acc;
}

// RED_PART for 4-byte elements, streamed: the lane's tiles are one contiguous byte range;
// it flows through a ring of kStreamBufs 16 KB shared-memory buffers filled by bulk
// asynchronous copies (one thread issues, mbarrier completion), so ~100 KB per SM are in
// flight independent of registers; every thread folds its 32 bytes of each buffer, and at
// each tile boundary the lane reduces and stores that tile's partial.
constexpr uint32_t kStreamChunk = 16384, kStreamBufs = 8;

template <typename C>
__device__ __forceinline__ bool red_part_stream(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi,
                                                uint32_t kind, uint32_t dt) {
  const KParams &P = *L.P;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *a = resolve(P, t.ptr[1]);
  const int64_t n = t.p[0], chunk = t.p[1];
  const int64_t lo = static_cast<int64_t>(tile_lo) * chunk, hi = min(static_cast<int64_t>(tile_hi) * chunk, n);
  if (lo >= hi) return true;
  const uint32_t tile_bytes = static_cast<uint32_t>(chunk) * 4u;
  if ((reinterpret_cast<uintptr_t>(a) & 15u) || tile_bytes % kStreamChunk || ((hi - lo) & 3) ||
      L.smem_bytes < kSmemSys + 1024u + kStreamBufs * kStreamChunk)
    return false;
  const uint8_t *src = a + lo * 4;
  const uint64_t total = static_cast<uint64_t>(hi - lo) * 4u;
  const uint32_t nchunks = static_cast<uint32_t>((total + kStreamChunk - 1) / kStreamChunk), per_tile = tile_bytes / kStreamChunk;
  uint64_t *bar = reinterpret_cast<uint64_t *>(L.smem + kSmemSys);
  uint8_t *bufs = L.smem + kSmemSys + 1024;
  auto bytes_of = [&](uint32_t c) {
    const uint64_t left = total - static_cast<uint64_t>(c) * kStreamChunk;
    return left < kStreamChunk ? static_cast<uint32_t>(left) : kStreamChunk;
  };
  __syncthreads();
  if (L.tid == 0) {
    for (uint32_t i = 0; i < kStreamBufs; ++i) mbar_init(&bar[i], 1);
    fence_mbar_init();
    for (uint32_t c = 0; c + 1 < kStreamBufs && c < nchunks; ++c) {
      mbar_arrive_expect_tx(&bar[c], bytes_of(c));
      bulk_g2s(bufs + c * kStreamChunk, src + static_cast<size_t>(c) * kStreamChunk, bytes_of(c), &bar[c]);
    }
  }
  __syncthreads();
  const uint32_t ident = static_cast<uint32_t>(acc_identity(kind, dt).bits);
  uint32_t acc = ident;
  bool fine = true;
  for (uint32_t c = 0; c < nchunks; ++c) {
    const uint32_t b = c % kStreamBufs;
    bool ok = mbar_wait_bounded(&bar[b], (c / kStreamBufs) & 1u, P.wait_budget_ns);
    if (!ok) set_status(P, kStTensorTimeout, L.lane, c, t.op);
    // lane-wide: nobody is still reading the buffer consumed last trip; a lost copy ends the op for all
    if (!__syncthreads_and(ok)) { fine = false; break; }
    const uint32_t nx = c + kStreamBufs - 1u;
    if (L.tid == 0 && nx < nchunks) {
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(&bar[nx % kStreamBufs], bytes_of(nx));
      bulk_g2s(bufs + (nx % kStreamBufs) * kStreamChunk, src + static_cast<size_t>(nx) * kStreamChunk, bytes_of(nx), &bar[nx % kStreamBufs]);
    }
    const uint32_t nb = bytes_of(c);
    const uint4 *q = reinterpret_cast<const uint4 *>(bufs + b * kStreamChunk);
    for (uint32_t o = L.tid; o < nb / 16u; o += L.nthr) {
      const uint4 v = q[o];
      acc = C::f(C::f(acc, v.x), C::f(v.y, C::f(v.z, v.w)));
    }
    if ((c + 1u) % per_tile == 0u || c + 1u == nchunks) {     // a tile is complete
      Acc r;
      r.bits = acc;
      r = acc_block_reduce(L, kind, dt, r);
      if (L.tid == 0) acc_store(dst, dt, tile_lo + c / per_tile, r);
      acc = ident;
    }
  }
  __syncthreads();
  if (L.tid == 0)
    for (uint32_t i = 0; i < kStreamBufs; ++i) mbar_inval(&bar[i]);
  __syncthreads();
  (void)fine;
  return true;
}

// One contiguous run of 16-byte words [w_lo, w_hi) of a 4-byte-element array, streamed
// through the ring of bulk copies (as red_part_stream) and folded by the whole lane;
// every thread returns the lane's total. Short runs are read directly.
template <typename C>
__device__ __forceinline__ uint32_t red_words_lane(const Lane &L, const uint8_t *a, uint64_t w_lo, uint64_t w_hi,
                                                   uint32_t kind, uint32_t dt, uint32_t ident) {
  const KParams &P = *L.P;
  uint32_t acc = ident;
  const uint8_t *src = a + w_lo * 16u;
  const uint64_t total = (w_hi - w_lo) * 16u;
  const bool stream = total >= 4u * kStreamChunk && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
                      L.smem_bytes >= kSmemSys + 1024u + kStreamBufs * kStreamChunk;
  if (stream) {
    // Ring of kStreamBufs buffers; per buffer a "full" barrier (the copy's bytes have landed) and an
    // "empty" barrier (every warp has read its share). Thread 0 issues the copies; nothing else in the
    // loop is lane-wide, so warps drift up to a ring's length apart instead of meeting at every buffer.
    const uint32_t nchunks = static_cast<uint32_t>((total + kStreamChunk - 1) / kStreamChunk);
    const uint32_t nwarps = L.nthr / kWarp, lane_id = L.tid % kWarp;
    uint64_t *full = reinterpret_cast<uint64_t *>(L.smem + kSmemSys);
    uint64_t *empty = full + kStreamBufs;
    uint8_t *bufs = L.smem + kSmemSys + 1024;
    auto bytes_of = [&](uint32_t c) {
      const uint64_t left = total - static_cast<uint64_t>(c) * kStreamChunk;
      return left < kStreamChunk ? static_cast<uint32_t>(left) : kStreamChunk;
    };
    auto refill = [&](uint32_t c) {
      const uint32_t bb = c % kStreamBufs;
      mbar_arrive_expect_tx(&full[bb], bytes_of(c));
      bulk_g2s(bufs + bb * kStreamChunk, src + static_cast<size_t>(c) * kStreamChunk, bytes_of(c), &full[bb]);
    };
    __syncthreads();
    if (L.tid == 0) {
      for (uint32_t i = 0; i < kStreamBufs; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], nwarps); }
      fence_mbar_init();
      for (uint32_t c = 0; c < kStreamBufs && c < nchunks; ++c) refill(c);
    }
    __syncthreads();
    uint32_t acc2 = ident;   // two chains per thread: the 16-byte words alternate between them
    bool ok = true;
    for (uint32_t c = 0; c < nchunks && ok; ++c) {
      const uint32_t b = c % kStreamBufs, par = (c / kStreamBufs) & 1u;
      if (L.tid == 0 && c >= 1u && c - 1u + kStreamBufs < nchunks) {
        // the buffer of chunk c - 1 goes to chunk c - 1 + kStreamBufs once every warp has left it
        const uint32_t pb = (c - 1u) % kStreamBufs;
        if (mbar_wait_bounded(&empty[pb], ((c - 1u) / kStreamBufs) & 1u, P.wait_budget_ns)) {
          fence_proxy_async_smem();
          refill(c - 1u + kStreamBufs);
        } else {
          set_status(P, kStTensorTimeout, L.lane, c, kTopRedPart);
        }
      }
      if (!mbar_wait_bounded(&full[b], par, P.wait_budget_ns)) {
        set_status(P, kStTensorTimeout, L.lane, c, kTopRedPart);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t nw = bytes_of(c) / 16u;
      const uint4 *q = reinterpret_cast<const uint4 *>(bufs + b * kStreamChunk);
      uint32_t o = L.tid;
      for (; o + L.nthr < nw; o += 2u * L.nthr) {
        const uint4 v = q[o], u = q[o + L.nthr];
        acc = C::f(C::f(acc, C::pre(v.x)), C::f(C::pre(v.y), C::f(C::pre(v.z), C::pre(v.w))));
        acc2 = C::f(C::f(acc2, C::pre(u.x)), C::f(C::pre(u.y), C::f(C::pre(u.z), C::pre(u.w))));
      }
      if (o < nw) {
        const uint4 v = q[o];
        acc = C::f(C::f(acc, C::pre(v.x)), C::f(C::pre(v.y), C::f(C::pre(v.z), C::pre(v.w))));
      }
      __syncwarp();
      if (lane_id == 0) mbar_arrive(&empty[b]);
    }
    acc = C::f(acc, acc2);
    __syncthreads();
    if (L.tid == 0 && ok)
      for (uint32_t i = 0; i < kStreamBufs; ++i) { mbar_inval(&full[i]); mbar_inval(&empty[i]); }
    __syncthreads();
  } else if (w_hi > w_lo) {
    const uint4 *q = reinterpret_cast<const uint4 *>(a);
    for (uint64_t o = w_lo + L.tid; o < w_hi; o += L.nthr) {
      const uint4 v = ldg_v4(q + o);
      acc = C::f(C::f(acc, C::pre(v.x)), C::f(C::pre(v.y), C::f(C::pre(v.z), C::pre(v.w))));
    }
  }
  Acc r;
  r.bits = acc;
  return static_cast<uint32_t>(acc_block_reduce(L, kind, dt, r).bits);
}

// A full reduction re-cut over all lanes by the loader (kRedFused): this lane folds the
// 16-byte words [w_lo, w_hi) of the input (the last lane also the ragged tail), leaves
// its total in the program's scratch and counts itself in; the lane that arrives last
// folds all lanes' totals in lane order and stores the result the RED_COMB would have.
template <typename C>
__device__ __forceinline__ void red_full_lane(const Lane &L, const DTask &t, uint32_t w_lo, uint32_t w_hi, uint32_t kind,
                                              uint32_t dt) {
  const KParams &P = *L.P;
  const uint8_t *a = resolve(P, t.ptr[1]);
  uint8_t *out = resolve(P, t.ptr[3]);
  const uint64_t n = t.p[0];
  RedScratch *sc = reinterpret_cast<RedScratch *>(P.scratch);
  const uint32_t ident = static_cast<uint32_t>(acc_identity(kind, dt).bits);
  const bool carried = (t.flags & kRedCarried) != 0u;   // the row op that wrote the input summed it on the way
  uint32_t total = carried ? ident : red_words_lane<C>(L, a, w_lo, w_hi, kind, dt, ident);
  uint32_t *flag = reinterpret_cast<uint32_t *>(L.smem + kSmemFlag);
  if (carried) __syncthreads();           // the flag word is the grid barrier's too: everybody has read its verdict
  if (L.tid == 0) {
    if (carried) {
      uint32_t *w = reinterpret_cast<uint32_t *>(&sc->total[P.n_lanes + L.lane]);
      total = *w;
      *w = 0u;                            // rest state for the next execute
    } else if (L.lane == P.n_lanes - 1u) {       // the elements past the last whole 16-byte word
      if (t.flags & (kRedSrcBf16 | kRedSrcF16)) {
        for (uint64_t i = (n / 8u) * 8u; i < n; ++i) {
          const uint32_t h = reinterpret_cast<const uint16_t *>(a)[i];
          total = C::f(total, __float_as_uint((t.flags & kRedSrcBf16) ? bf16_bits_to_f32(h) : f16_bits_to_f32(h)));
        }
      } else {
        for (uint64_t i = (n / 4u) * 4u; i < n; ++i) total = C::f(total, reinterpret_cast<const uint32_t *>(a)[i]);
      }
    }
    sc->total[L.lane] = total;
    __threadfence();
    *flag = atom_add_acq_rel_gpu(&sc->arrived, 1u) == P.n_lanes - 1u ? 1u : 0u;
  }
  __syncthreads();
  const bool last = *flag != 0u;
  __syncthreads();   // the flag word is the grid barrier's too
  if (!last) return;
  __threadfence();
  Acc acc;
  acc.bits = ident;
  for (uint32_t l = L.tid; l < P.n_lanes; l += L.nthr) {
    const unsigned long long v = *reinterpret_cast<volatile unsigned long long *>(&sc->total[l]);
    acc.bits = C::f(static_cast<uint32_t>(acc.bits), static_cast<uint32_t>(v));
  }
  acc = acc_block_reduce(L, kind, dt, acc);
  if (L.tid == 0) {
    acc_store(out, dt, 0, acc);
    st_relaxed_gpu(&sc->arrived, 0u);   // rest state for the next reduction of this program
  }
}

// RED_PART: tile t reduces in[t*chunk, min((t+1)*chunk, n)) into partials[t]. With
// kRedFused the entry names the 16-byte words [w_lo, w_hi) instead (see red_full_lane).
static __device__ __noinline__ void red_part_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi,
                                                   uint32_t w_lo, uint32_t w_hi) {
  const KParams &P = *L.P;
  if (t.flags & kRedFused) {
    const uint32_t kind = t.p[2], dt = t.dt;
    const bool fl = dt == kF32;
    if (fl && kind == kSum && (t.flags & kRedSrcBf16)) red_full_lane<RFSumBf>(L, t, w_lo, w_hi, kind, dt);
    else if (fl && kind == kSum && (t.flags & kRedSrcF16)) red_full_lane<RFSumF16>(L, t, w_lo, w_hi, kind, dt);
    else if (fl && kind == kSum) red_full_lane<RFSum>(L, t, w_lo, w_hi, kind, dt);
    else if (fl && kind == kRMax) red_full_lane<RFMax>(L, t, w_lo, w_hi, kind, dt);
    else if (fl && kind == kRMin) red_full_lane<RFMin>(L, t, w_lo, w_hi, kind, dt);
    else if (fl) red_full_lane<RFProd>(L, t, w_lo, w_hi, kind, dt);
    else if (kind == kSum) red_full_lane<RISum>(L, t, w_lo, w_hi, kind, dt);
    else if (kind == kProd) red_full_lane<RIProd>(L, t, w_lo, w_hi, kind, dt);
    else if (kind == kRAnd) red_full_lane<RIAnd>(L, t, w_lo, w_hi, kind, dt);
    else if (kind == kROr) red_full_lane<RIOr>(L, t, w_lo, w_hi, kind, dt);
    else if (kind == kRXor) red_full_lane<RIXor>(L, t, w_lo, w_hi, kind, dt);
    else if (kind == kRMax && dt == kI32) red_full_lane<RIMaxS>(L, t, w_lo, w_hi, kind, dt);
    else if (kind == kRMax) red_full_lane<RIMaxU>(L, t, w_lo, w_hi, kind, dt);
    else if (dt == kI32) red_full_lane<RIMinS>(L, t, w_lo, w_hi, kind, dt);
    else red_full_lane<RIMinU>(L, t, w_lo, w_hi, kind, dt);
    return;
  }
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *a = resolve(P, t.ptr[1]);
  const int64_t n = t.p[0], chunk = t.p[1];
  const uint32_t kind = t.p[2], dt = t.dt;
  if (dt == kF32 && kind == kSum && red_part_stream<RFSum>(L, t, tile_lo, tile_hi, kind, dt)) return;
  if (dt == kF32 && kind == kRMax && red_part_stream<RFMax>(L, t, tile_lo, tile_hi, kind, dt)) return;
  if (dt == kF32 && kind == kRMin && red_part_stream<RFMin>(L, t, tile_lo, tile_hi, kind, dt)) return;
  if ((dt == kI32 || dt == kU32) && kind == kSum && red_part_stream<RISum>(L, t, tile_lo, tile_hi, kind, dt)) return;
  for (uint32_t tile = tile_lo; tile < tile_hi; ++tile) {
    const int64_t lo = tile * chunk, hi = min(lo + chunk, n);
    if (lo >= hi) continue;
    if (tile + 1 < tile_hi) {
      // the lane's next tile is pulled into L2 while this one is reduced, so the load
      // pipeline that drains at the block reduction refills from L2 rather than HBM
      const uint32_t esz = dt_size(dt);
      const int64_t nb = (min(hi + chunk, n) - hi) * esz;
      const uint8_t *q = a + hi * esz;
      for (int64_t b = static_cast<int64_t>(L.tid) * 128; b < nb; b += static_cast<int64_t>(L.nthr) * 128) prefetch_l2(q + b);
    }
    Acc acc = reduce_run(a, dt, kind, lo, hi, L.tid, L.nthr, nullptr, 0);
    acc = acc_block_reduce(L, kind, dt, acc);
    if (L.tid == 0) acc_store(dst, dt, tile, acc);
  }
}

// RED_COMB: fold n_parts partials into dst[0] (single tile).
static __device__ __noinline__ void red_comb_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  if (!(tile_lo == 0 && tile_hi > 0)) return;
  const KParams &P = *L.P;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *a = resolve(P, t.ptr[1]);
  const uint32_t kind = t.p[1], dt = t.dt;
  Acc acc = reduce_run(a, dt, kind, 0, t.p[0], L.tid, L.nthr, nullptr, 0);
  acc = acc_block_reduce(L, kind, dt, acc);
  if (L.tid == 0) acc_store(dst, dt, 0, acc);
}


#if B2_SHORT
// RED_SEG on f32 with segments of 2..8 elements (a trailing axis of 3 in an
// (N, N, 3) tensor): a thread per segment reads 4 bytes at a stride of `seg`
// words and the load pipeline never fills. Here a warp takes 128 consecutive
// segments (128 * seg contiguous floats) with `seg` coalesced 16-byte loads per
// thread, parks them in its shared-memory slab, and each thread folds segments
// l, l+32, l+64, l+96 from there; results leave as 128-byte rows. Elements of a
// segment are folded in index order, like the per-thread loop.
// SEG > 0: the segment length as a constant (its loads sit in exactly SEG registers);
// SEG == 0: any length up to 8.
template <uint32_t KIND, uint32_t SEG>
__device__ __forceinline__ void red_seg_small_f32(const Lane &L, float *dst, const float *a, uint32_t lo, uint32_t hi,
                                                  uint32_t seg_rt) {
  constexpr uint32_t kSpan = 128, kMaxSeg = SEG ? SEG : 8;
  const uint32_t seg = SEG ? SEG : seg_rt;
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = L.nthr / kWarp;
  float *stage = reinterpret_cast<float *>(L.smem + kSmemSys) + static_cast<size_t>(w) * kSpan * kMaxSeg;
  auto one = [&](uint32_t o) {
    const float *p = a + static_cast<int64_t>(o) * seg;
    float r = p[0];
    for (uint32_t i = 1; i < seg; ++i) r = red_f(KIND, r, p[i]);
    dst[o] = r;
  };
  const uint32_t o_al = min(hi, (lo + 3u) & ~3u);          // 16-byte alignment of the first full span
  for (uint32_t o = lo + L.tid; o < o_al; o += L.nthr) one(o);
  const uint32_t nsteps = (hi - o_al) / kSpan;
  const uint32_t span_lines = (kSpan * seg * 4u + 127u) / 128u;
  for (uint32_t s = w; s < nsteps; s += nw) {
    const uint32_t o0 = o_al + s * kSpan;
    const float *p = a + static_cast<int64_t>(o0) * seg;
    uint4 v[kMaxSeg];
#pragma unroll
    for (uint32_t j = 0; j < kMaxSeg; ++j)
      if (j < seg) v[j] = ldg_v4(p + (j * kWarp + l) * 4u);
    if (s + nw < nsteps && l < span_lines)                   // the warp's next span, into L2
      prefetch_l2(reinterpret_cast<const uint8_t *>(p + static_cast<int64_t>(nw) * kSpan * seg) + l * 128u);
#pragma unroll
    for (uint32_t j = 0; j < kMaxSeg; ++j)
      if (j < seg) *reinterpret_cast<uint4 *>(stage + (j * kWarp + l) * 4u) = v[j];
    __syncwarp();
#pragma unroll
    for (uint32_t q = 0; q < kSpan / kWarp; ++q) {
      const uint32_t si = l + q * kWarp;
      const float *sp = stage + si * seg;
      float r = sp[0];
      for (uint32_t i = 1; i < seg; ++i) r = red_f(KIND, r, sp[i]);
      dst[o0 + si] = r;
    }
    __syncwarp();
  }
  for (uint32_t o = o_al + nsteps * kSpan + L.tid; o < hi; o += L.nthr) one(o);
}

#endif

// RED_SEG: out[o] = reduce(in[o*seg, (o+1)*seg)), one segment per tile index;
// p3 = 1: dot mode, out[o] = sum_j in[o*seg+j] * b[j].
static __device__ __noinline__ void red_seg_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *a = resolve(P, t.ptr[1]);
  const uint32_t n_out = t.p[0], kind = t.p[3] ? static_cast<uint32_t>(kSum) : t.p[2];
  const int64_t seg = t.p[1];
  const uint32_t dt = t.p[3] ? t.adt : t.dt;  // reduce keeps the input dtype; dot mode reads adt
  const uint8_t *vecb = t.p[3] ? resolve(P, t.ptr[2]) : nullptr;
  const uint32_t hi = min(tile_hi, n_out);
#if B2_SHORT
  if (!t.p[3] && dt == kF32 && t.dt == kF32 && seg >= 2 && seg <= 8 && hi > tile_lo &&
      (reinterpret_cast<uintptr_t>(a) & 15u) == 0 && (kind == kSum || kind == kRMax || kind == kRMin)) {
    float *d = reinterpret_cast<float *>(dst);
    const float *s = reinterpret_cast<const float *>(a);
    const uint32_t sg = static_cast<uint32_t>(seg);
    if (kind == kSum && sg == 3) red_seg_small_f32<kSum, 3>(L, d, s, tile_lo, hi, sg);
    else if (kind == kSum && sg == 2) red_seg_small_f32<kSum, 2>(L, d, s, tile_lo, hi, sg);
    else if (kind == kSum && sg == 4) red_seg_small_f32<kSum, 4>(L, d, s, tile_lo, hi, sg);
    else if (kind == kSum) red_seg_small_f32<kSum, 0>(L, d, s, tile_lo, hi, sg);
    else if (kind == kRMax) red_seg_small_f32<kRMax, 0>(L, d, s, tile_lo, hi, sg);
    else red_seg_small_f32<kRMin, 0>(L, d, s, tile_lo, hi, sg);
    return;
  }
#endif
  if (seg <= 16) {  // thread per segment
    for (uint32_t o = tile_lo + L.tid; o < hi; o += L.nthr) {
      Acc acc = reduce_run(a, dt, kind, o * seg, (o + 1) * seg, 0, 1, vecb, 0);
      acc_store(dst, t.dt, o, acc);
    }
  } else if (seg <= 16384) {  // warp per segment
    const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = L.nthr / kWarp;
    for (uint32_t o = tile_lo + w; o < hi; o += nw) {
      Acc acc = reduce_run(a, dt, kind, o * seg, (o + 1) * seg, l, kWarp, vecb, 0);
      acc = acc_warp_reduce(kind, dt, acc);
      if (l == 0) acc_store(dst, t.dt, o, acc);
    }
  } else {  // the whole lane per segment
    for (uint32_t o = tile_lo; o < hi; ++o) {
      Acc acc = reduce_run(a, dt, kind, o * seg, (o + 1) * seg, L.tid, L.nthr, vecb, 0);
      acc = acc_block_reduce(L, kind, dt, acc);
      if (L.tid == 0) acc_store(dst, t.dt, o, acc);
    }
  }
}

// RED_STRIDED on f32 with a short inner axis (2..4) and a long reduced axis:
// out[row*INNER + c] = reduce_r in[(row*red + r)*INNER + c]. A row's red*INNER
// elements are contiguous, so a warp streams one row with coalesced 16-byte
// loads. A step covers 32*INNER loads = 128*INNER elements, a multiple of INNER,
// so register (j, k) of a thread (load j of the step, element k of its 16 bytes)
// sees the same output column c = (128 j + 4 l + k) mod INNER in every step:
// the loop adds into INNER*4 fixed accumulators and the columns are sorted out
// once per row.
template <int INNER, uint32_t KIND>
__device__ __forceinline__ void red_strided_rows_f32(const Lane &L, float *dst, const float *a, const float *a_end,
                                                     int64_t row_lo, int64_t row_hi, int64_t red, int64_t out_lo,
                                                     int64_t out_hi) {
  const uint32_t w = L.tid / kWarp, l = L.tid % kWarp, nw = L.nthr / kWarp;
  const int64_t row_f4 = red * INNER / 4;                    // 16-byte words per row
  constexpr int64_t kStep = static_cast<int64_t>(kWarp) * INNER;
  const int64_t full = row_f4 / kStep;
  const float ident = red_f_identity(KIND);
  auto put = [&](float (&res)[INNER], int c, float x) {
#pragma unroll
    for (int cc = 0; cc < INNER; ++cc) res[cc] = (c == cc) ? red_f(KIND, res[cc], x) : res[cc];
  };
  for (int64_t row = row_lo + w; row < row_hi; row += nw) {
    const float *rp = a + row * red * INNER;
    float acc[INNER][4];
#pragma unroll
    for (int j = 0; j < INNER; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[j][k] = ident;
    int64_t s = 0;
    for (; s + 2 <= full; s += 2) {                          // two steps' loads in flight
      uint4 v[2][INNER];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < INNER; ++j) v[h][j] = ldg_v4(rp + ((s + h) * kStep + j * kWarp + l) * 4);
      const float *pf = rp + (s + 8) * kStep * 4 + l * 32;   // 2 steps = 24*INNER/3 lines of 128 B, 8 steps ahead
      if (l < (2 * kStep * 16 + 127) / 128 && pf < a_end) prefetch_l2(pf);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < INNER; ++j) {
          acc[j][0] = red_f(KIND, acc[j][0], __uint_as_float(v[h][j].x));
          acc[j][1] = red_f(KIND, acc[j][1], __uint_as_float(v[h][j].y));
          acc[j][2] = red_f(KIND, acc[j][2], __uint_as_float(v[h][j].z));
          acc[j][3] = red_f(KIND, acc[j][3], __uint_as_float(v[h][j].w));
        }
    }
    for (; s < full; ++s) {
#pragma unroll
      for (int j = 0; j < INNER; ++j) {
        const uint4 v = ldg_v4(rp + (s * kStep + j * kWarp + l) * 4);
        acc[j][0] = red_f(KIND, acc[j][0], __uint_as_float(v.x));
        acc[j][1] = red_f(KIND, acc[j][1], __uint_as_float(v.y));
        acc[j][2] = red_f(KIND, acc[j][2], __uint_as_float(v.z));
        acc[j][3] = red_f(KIND, acc[j][3], __uint_as_float(v.w));
      }
    }
    float res[INNER];
#pragma unroll
    for (int c = 0; c < INNER; ++c) res[c] = ident;
#pragma unroll
    for (int j = 0; j < INNER; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) put(res, static_cast<int>((128u * j + 4u * l + k) % INNER), acc[j][k]);
    for (int64_t f = full * kStep + l; f < row_f4; f += kWarp) {   // the row's ragged end
      const uint4 v = ldg_v4(rp + f * 4);
      const int c0 = static_cast<int>((f * 4) % INNER);
      put(res, c0 % INNER, __uint_as_float(v.x));
      put(res, (c0 + 1) % INNER, __uint_as_float(v.y));
      put(res, (c0 + 2) % INNER, __uint_as_float(v.z));
      put(res, (c0 + 3) % INNER, __uint_as_float(v.w));
    }
#pragma unroll
    for (int c = 0; c < INNER; ++c) {
#pragma unroll
      for (int o = kWarp / 2; o > 0; o >>= 1) res[c] = red_f(KIND, res[c], __shfl_xor_sync(0xffffffffu, res[c], o));
      const int64_t g = row * INNER + c;
      if (l == 0 && g >= out_lo && g < out_hi) dst[g] = res[c];
    }
  }
}

template <uint32_t KIND>
__device__ __forceinline__ void red_strided_rows_kind(const Lane &L, float *dst, const float *a, const float *a_end,
                                                      int64_t row_lo, int64_t row_hi, int64_t red, int64_t inner,
                                                      int64_t out_lo, int64_t out_hi) {
  if (inner == 2) red_strided_rows_f32<2, KIND>(L, dst, a, a_end, row_lo, row_hi, red, out_lo, out_hi);
  else if (inner == 3) red_strided_rows_f32<3, KIND>(L, dst, a, a_end, row_lo, row_hi, red, out_lo, out_hi);
  else red_strided_rows_f32<4, KIND>(L, dst, a, a_end, row_lo, row_hi, red, out_lo, out_hi);
}

// RED_STRIDED: out[o*inner + i] = reduce_r in[(o*red + r)*inner + i]; EW-style
// tiling of the outputs. An entry either names output tiles [tile_lo, tile_hi)
// or, when the loader spread a task with few tiles over all lanes, whole rows
// [row_lo, row_hi) (row_hi > row_lo; a row = the `inner` outputs of one o).
// General path: consecutive threads own consecutive outputs (coalesced along
// `inner`), each keeps kQ independent outputs in flight.
static __device__ __noinline__ void red_strided_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi,
                                               uint32_t row_lo, uint32_t row_hi) {
  const KParams &P = *L.P;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *a = resolve(P, t.ptr[1]);
  const int64_t n_out = t.p[0], red = t.p[1], inner = t.p[2];
  const uint32_t kind = t.p[3], dt = t.dt;
  const bool by_rows = row_hi > row_lo;
  const int64_t lo = by_rows ? static_cast<int64_t>(row_lo) * inner : static_cast<int64_t>(tile_lo) * kEwTs;
  const int64_t hi = min(by_rows ? static_cast<int64_t>(row_hi) * inner : static_cast<int64_t>(tile_hi) * kEwTs, n_out);
  if (lo >= hi) return;
  if (red_strided_rows_ok(dt, red, inner, kind) && (reinterpret_cast<uintptr_t>(a) & 15u) == 0) {
    // rows that intersect [lo, hi); a row cut by a tile boundary is reduced by both
    // neighbours and each stores its own outputs
    const int64_t r0 = lo / inner, r1 = (hi + inner - 1) / inner;
    float *d = reinterpret_cast<float *>(dst);
    const float *s = reinterpret_cast<const float *>(a);
    const float *s_end = s + (n_out / inner) * red * inner;
    red_strided_rows_kind<kSum>(L, d, s, s_end, r0, r1, red, inner, lo, hi);
    return;
  }
  constexpr int kQ = 8;
  for (int64_t g0 = lo + L.tid; g0 < hi; g0 += static_cast<int64_t>(L.nthr) * kQ) {
    Acc acc[kQ];
    int64_t base[kQ];
#pragma unroll
    for (int q = 0; q < kQ; ++q) {
      const int64_t g = g0 + static_cast<int64_t>(q) * L.nthr;
      acc[q] = acc_identity(kind, dt);
      base[q] = g < hi ? (g / inner) * red * inner + (g % inner) : -1;
    }
    for (int64_t r = 0; r < red; ++r) {
#pragma unroll
      for (int q = 0; q < kQ; ++q)
        if (base[q] >= 0) acc[q] = acc_combine(kind, dt, acc[q], acc_load(a, dt, base[q] + r * inner));
    }
#pragma unroll
    for (int q = 0; q < kQ; ++q)
      if (base[q] >= 0) acc_store(dst, dt, g0 + static_cast<int64_t>(q) * L.nthr, acc[q]);
  }
}

}  // namespace b2
#endif
