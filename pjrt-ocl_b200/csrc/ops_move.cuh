// Data-movement tile ops: strided GATHER, strided SCATTER, IOTA_DIM, and the
// dynamic-offset gather/scatter behind dynamic_slice / dynamic_update_slice.
//
// Replaces vmo_gather_tile (pjrt_plugin/kernels/ops/gather.cl:9-82),
// vmo_scatter_tile (ops/scatter.cl:9-50), vmo_iota_tile (ops/iota.cl:4-29) and
// vmo_dyn_gather_tile / vmo_dyn_scatter_tile (ops/dynslice.cl:28-166).
// Semantics: python/pjrt_ocl/ops/shape.py:196-217, ops/concat.py:214-236,
// ops/making.py:85-117, ops/dynslice.py:134-190.
//
// The loader collapses each access map to <= 4 dims and marks the ones whose
// innermost run is contiguous on both sides and a whole number of 16-byte
// chunks; those move as 16-byte vectors (one index computation per chunk),
// coalesced on the contiguous side. Everything else moves element by element,
// coalesced on the side that is walked linearly.
#ifndef B2VM_OPS_MOVE_CUH_
#define B2VM_OPS_MOVE_CUH_

#include "dev_common.cuh"

namespace b2 {


__device__ __forceinline__ void copy_elem(uint8_t *d, int64_t di, const uint8_t *s, int64_t si, uint32_t esz) {
  switch (esz) {
    case 1: d[di] = s[si]; break;
    case 2: reinterpret_cast<uint16_t *>(d)[di] = reinterpret_cast<const uint16_t *>(s)[si]; break;
    case 4: reinterpret_cast<uint32_t *>(d)[di] = reinterpret_cast<const uint32_t *>(s)[si]; break;
    default: reinterpret_cast<unsigned long long *>(d)[di] = reinterpret_cast<const unsigned long long *>(s)[si]; break;
  }
}

// Runtime base offset of a dynamic slice: sum_d clamp(start_d, 0, max_d) * stride_d.
__device__ __forceinline__ int64_t dyn_base(const KParams &P, const DMove &m) {
  int64_t base = 0;
  for (uint32_t d = 0; d < m.n_idx; ++d) {
    const uint8_t *ip = resolve(P, m.idx_ptr[d]);
    long long s = m.is64 ? *reinterpret_cast<const long long *>(ip) : *reinterpret_cast<const int32_t *>(ip);
    s = s < 0 ? 0 : (s > m.clamp_max[d] ? m.clamp_max[d] : s);
    base += s * m.idx_stride[d];
  }
  return base;
}

// A transposing gather: dst rows (length cc = dim[rank-1]) walk the source with stride
// ld, while consecutive dst rows are adjacent in the source. Element by element every
// read would touch its own 32-byte sector. Here whole dst rows [row_a, row_b) move
// through shared-memory tiles of up to 32 rows x 64 columns: read along the source's
// contiguous direction (rows), write along dst's (columns), both coalesced.
template <typename E>
__device__ __forceinline__ void transpose_rows(const Lane &L, const DMove &m, E *dst, const E *src, int64_t row_a,
                                               int64_t row_b) {
  constexpr int TR = 64, TC = 256;   // 16K elements per tile: 32 independent loads per thread in flight
  const DView &v = m.view;
  const int64_t cc = v.dim[v.rank - 1], rr = v.dim[v.rank - 2], ld = v.stride[v.rank - 1];
  E *tile = reinterpret_cast<E *>(L.smem + kSmemSys);             // [TC][TR + 1]
  for (int64_t row0 = row_a; row0 < row_b;) {
    // rows of one segment share every outer coordinate: their source addresses are consecutive
    const int64_t r_in = row0 % rr;
    const int nr = static_cast<int>(min(min(static_cast<int64_t>(TR), rr - r_in), row_b - row0));
    const int64_t sbase = view_index(v, static_cast<uint32_t>(row0 * cc));
    for (int64_t c0 = 0; c0 < cc; c0 += TC) {
      const int nc = static_cast<int>(min(static_cast<int64_t>(TC), cc - c0));
      __syncthreads();
      const E *sp = src + sbase + c0 * ld;
      // loads first, into registers, then the shared-memory stores: written as one loop the
      // compiler must assume the two pointers alias and would wait out each load in turn
      constexpr int U = 8;
      for (int i0 = L.tid; i0 < nc * TR; i0 += U * static_cast<int>(L.nthr)) {
        E val[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = i0 + u * static_cast<int>(L.nthr);
          const int r = i % TR, c = i / TR;
          val[u] = (i < nc * TR && r < nr) ? sp[static_cast<int64_t>(c) * ld + r] : E(0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = i0 + u * static_cast<int>(L.nthr);
          if (i < nc * TR) tile[(i / TR) * (TR + 1) + i % TR] = val[u];
        }
      }
      __syncthreads();
      E *dp = dst + row0 * cc + c0;
#pragma unroll 8
      for (int i = L.tid; i < nr * TC; i += L.nthr) {
        const int c = i % TC, r = i / TC;
        if (c < nc) dp[static_cast<int64_t>(r) * cc + c] = tile[c * (TR + 1) + r];
      }
    }
    row0 += nr;
  }
  __syncthreads();
}

// gather: dst[i] = a[base + view(i)];  scatter: dst[base + view(i)] = a[i]
static __device__ __noinline__ void move_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi, bool scatter) {
  const KParams &P = *L.P;
  const DMove &m = *reinterpret_cast<const DMove *>(P.desc + t.desc);
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *src = resolve(P, t.ptr[1]);
  const uint32_t n = t.p[1];
  const uint64_t lo64 = static_cast<uint64_t>(tile_lo) * kEwTs;
  uint64_t hi64 = static_cast<uint64_t>(tile_hi) * kEwTs;
  if (hi64 > n) hi64 = n;
  if (lo64 >= hi64) return;
  const uint32_t lo = static_cast<uint32_t>(lo64), hi = static_cast<uint32_t>(hi64);
  const int64_t base = m.n_idx ? dyn_base(P, m) : 0;
  const uint32_t esz = m.esz;
  const bool vec = m.chunk && (base % m.chunk == 0);
  if (m.transposed && !scatter) {
    const int64_t cc = m.view.dim[m.view.rank - 1];
    const int64_t row_a = (static_cast<int64_t>(lo) + cc - 1) / cc, row_b = static_cast<int64_t>(hi) / cc;
    if (row_b > row_a) {
      // ragged ends of the range element by element, whole rows through the tiles
      for (uint32_t i = lo + L.tid; i < row_a * cc; i += L.nthr) copy_elem(dst, i, src, view_index(m.view, i), esz);
      for (uint32_t i = static_cast<uint32_t>(row_b * cc) + L.tid; i < hi; i += L.nthr)
        copy_elem(dst, i, src, view_index(m.view, i), esz);
      if (esz == 2) transpose_rows(L, m, reinterpret_cast<uint16_t *>(dst), reinterpret_cast<const uint16_t *>(src), row_a, row_b);
      else transpose_rows(L, m, reinterpret_cast<uint32_t *>(dst), reinterpret_cast<const uint32_t *>(src), row_a, row_b);
      return;
    }
  }
  if (vec) {
    // lo is a multiple of 4096 and chunk divides 16, so chunks never straddle lo.
    const uint32_t c = m.chunk, c_lo = lo / c, c_hi = hi / c;
    // four chunks per thread per trip: the four loads are independent and in flight together
    constexpr uint32_t U = 4;
    uint32_t k = c_lo + L.tid;
    for (; k + (U - 1) * L.nthr < c_hi; k += U * L.nthr) {
      int64_t s[U];
      uint4 w[U];
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) s[u] = base + view_index(m.view, (k + u * L.nthr) * c);
#pragma unroll
      for (uint32_t u = 0; u < U; ++u)
        w[u] = scatter ? *reinterpret_cast<const uint4 *>(src + static_cast<int64_t>(k + u * L.nthr) * 16)
                       : *reinterpret_cast<const uint4 *>(src + s[u] * esz);
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) {
        if (scatter) *reinterpret_cast<uint4 *>(dst + s[u] * esz) = w[u];
        else *reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(k + u * L.nthr) * 16) = w[u];
      }
    }
    for (; k < c_hi; k += L.nthr) {
      const int64_t s = base + view_index(m.view, k * c);
      if (scatter)
        *reinterpret_cast<uint4 *>(dst + s * esz) = *reinterpret_cast<const uint4 *>(src + static_cast<int64_t>(k) * 16);
      else
        *reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(k) * 16) = *reinterpret_cast<const uint4 *>(src + s * esz);
    }
    for (uint32_t i = c_hi * c + L.tid; i < hi; i += L.nthr) {  // ragged tail of the range
      const int64_t s = base + view_index(m.view, i);
      if (scatter) copy_elem(dst, s, src, i, esz); else copy_elem(dst, i, src, s, esz);
    }
    return;
  }
  uint32_t i = lo + L.tid;
#if B2_SHORT
  if (!scatter && esz == 4 && m.view.rank >= 1 && m.view.rank <= 3 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
    // A gather whose source runs are shorter than 16 bytes (an (N, 3) table repeated
    // along a middle axis): a thread owns whole 16-byte chunks of dst, finds the source
    // coordinates of a chunk's first element once and walks to the next three; two
    // chunks (8 loads) are in flight per trip. lo is a multiple of the 4096-element tile.
    const ViewWalk w = view_walk(m.view);
    const uint32_t *s32 = reinterpret_cast<const uint32_t *>(src);
    constexpr uint32_t U = 2;
    const uint32_t c_hi = hi / 4u;
    uint32_t k = lo / 4u + L.tid;
    for (; k < c_hi; k += U * L.nthr) {
      uint32_t v[U][4];
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) {
        const uint32_t kk = k + u * L.nthr;
        if (kk < c_hi) {
          uint32_t cA, cB, cO;
          view_walk_seek(w, kk * 4u, cA, cB, cO);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[u][e] = s32[base + view_walk_index(w, cA, cB, cO)];
            view_walk_next(w, cA, cB, cO);
          }
        }
      }
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) {
        const uint32_t kk = k + u * L.nthr;
        if (kk < c_hi) *reinterpret_cast<uint4 *>(dst + static_cast<size_t>(kk) * 16) = make_uint4(v[u][0], v[u][1], v[u][2], v[u][3]);
      }
    }
    i = c_hi * 4u + L.tid;      // the ragged end of the range, below
  }
#endif
  for (; i < hi; i += L.nthr) {
    const int64_t s = base + view_index(m.view, i);
    if (scatter) copy_elem(dst, s, src, i, esz); else copy_elem(dst, i, src, s, esz);
  }
}

// iota: dst[i] = coordinate of i along `dim` (aux {rank, dims[rank], dim}); the
// loader stores {dim_size, inner} = sizes such that coord = (i / inner) % dim_size.
static __device__ __noinline__ void iota_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const uint32_t *d = reinterpret_cast<const uint32_t *>(P.desc + t.desc);
  const uint32_t dim_size = d[0], inner = d[1];
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint32_t n = t.p[1], dt = t.dt;
  const uint64_t lo64 = static_cast<uint64_t>(tile_lo) * kEwTs;
  uint64_t hi64 = static_cast<uint64_t>(tile_hi) * kEwTs;
  if (hi64 > n) hi64 = n;
  for (uint64_t i = lo64 + L.tid; i < hi64; i += L.nthr) {
    const uint32_t c = dim_size ? (static_cast<uint32_t>(i) / inner) % dim_size : 0u;
    if (is_float_dt(dt)) storef(dst, dt, i, static_cast<float>(c));
    else if (dt == kF64) reinterpret_cast<double *>(dst)[i] = static_cast<double>(c);
    else if (dt == kI64) reinterpret_cast<long long *>(dst)[i] = c;
    else store1(dst, dt, i, c);
  }
}

}  // namespace b2
#endif
