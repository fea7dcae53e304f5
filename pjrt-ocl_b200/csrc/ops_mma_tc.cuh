// TILE_MMA on the 5th-generation tensor cores (tcgen05), bf16 / f16 operands, f32
// accumulation in tensor memory.
//
// Same contract as the CUDA-core path (ops_mma.cuh; pjrt_plugin/kernels/ops/mma.cl:
// 74-96,136-434; python/pjrt_ocl/ops/dot.py:206-293): C[g] = A[g] . B[g] on 128x128
// output tiles numbered batch x tiles_m x tiles_n, optional operand views, optional
// store epilogue. Taken when the loader proved both operands affine with a unit
// stride along k or along the row / column index (DMma::tc_mode).
//
// One lane (CTA, 16 warps) works through its tile range in "super-tiles" of one or
// two horizontally adjacent 128x128 tiles, i.e. a 128 x (128|256) accumulator, so a
// block of A is fetched once for both:
//   warps 0-7   producers: 16-byte asynchronous copies global -> shared straight into
//               the 128-byte-swizzled operand layout the tensor core reads, 64 k per
//               stage, kTcStages stages in flight, zero-filling rows / k beyond the edge;
//   warp 8      lane 0 issues the tcgen05.mma instructions (4 per stage, K = 16 each)
//               and commits them to the stage's "empty" barrier;
//   warps 8-15  epilogue: tcgen05.ld the accumulator (each warp its 32 lanes x 64 or
//               128 columns), micro-epilogue, convert, store.
// Every barrier wait is bounded by the launch's wait budget and watches a lane-wide
// failure flag; on failure the lane records a status, drains its copies, frees its
// tensor memory and returns.
#ifndef B2VM_OPS_MMA_TC_CUH_
#define B2VM_OPS_MMA_TC_CUH_

#include "ops_mma.cuh"

namespace b2 {

#if B2_HAS_TC

constexpr int kTcBK = 64;                    // k per stage: 128 bytes, one swizzle row
constexpr int kTcStages = 4;
constexpr int kTcABytes = 128 * 128;         // 128 rows x 128 B
constexpr int kTcBBytes = 256 * 128;         // up to 256 rows x 128 B
constexpr int kTcStageBytes = kTcABytes + kTcBBytes;
constexpr int kTcProducers = 256;
constexpr uint32_t kTcCols = 256;            // tensor-memory columns held (f32 accumulator 128 x 256)

struct TcShared {                            // lives in the reduction scratch of the system area
  uint64_t full[kTcStages];
  uint64_t empty[kTcStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};
static_assert(sizeof(TcShared) <= 512, "fits the scratch slot");

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
         (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Bounded wait that also gives up when another role of the lane failed.
// `backoff_ns`: sleep between polls - for waits that are expected to be long (the
// epilogue warps during the main loop), so they leave the issue slots to the producers.
__device__ __forceinline__ bool tc_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *failed,
                                        unsigned long long budget_ns, uint32_t backoff_ns = 0) {
  if (mbar_try_wait_parity(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait_parity(bar, parity)) return true;
      if (backoff_ns) nanosleep_ns(backoff_ns);
    }
    if (*failed) return false;
    if (globaltimer_ns() - t0 > budget_ns) { *failed = 1u; return false; }
  }
}

// A whole warp waits, but only lane 0 polls: the other lanes sit at the warp
// barrier without taking issue slots from the warps that have work. Every lane
// gets lane 0's outcome (so the warp stays together when a wait ran out), and the
// warp barrier orders lane 0's acquire before the other lanes' later accesses.
__device__ __forceinline__ bool tc_wait_warp(uint64_t *bar, uint32_t parity, volatile uint32_t *failed,
                                             unsigned long long budget_ns, uint32_t backoff_ns = 0) {
  uint32_t ok = 1u;
  if ((threadIdx.x & 31u) == 0u) ok = tc_wait(bar, parity, failed, budget_ns, backoff_ns) ? 1u : 0u;
  return __shfl_sync(0xffffffffu, ok, 0) != 0u;
}

// A producer thread's share of one operand block (ROWS x 64 k), fixed for a whole
// super-tile: NCH 16-byte chunks, each with a shared-memory offset inside the stage,
// a source pointer that advances by `step` elements per k block, and the bytes of
// the chunk that exist (rows / columns beyond the matrix edge are zero-filled).
//   K-major operand (element (row, k) at src[row * ld + k]): row at 128 B pitch, its
//   16-byte chunks XORed with row % 8.
//   MN-major operand (element (row, k) at src[k * ld + row]): 64-row blocks 8192 B
//   apart, 8-k groups 1024 B apart, inside a group one k per 128 B line with its
//   chunks XORed with k % 8.
template <int ROWS>
struct TcPlan {
  static constexpr int NCH = ROWS / 32;
  const uint16_t *src[NCH];
  uint32_t dst[NCH];
  uint32_t bytes[NCH];      // K-major: 16 or 0 by row; MN-major: bytes of the row chunk
  uint32_t koff[NCH];       // k of the chunk inside the block (its validity in the last, partial block)
  int64_t step;
  bool mn;
};

template <int ROWS>
__device__ __forceinline__ void tc_plan(TcPlan<ROWS> &p, bool mn, const uint16_t *src, int64_t ld, int64_t rows_valid,
                                        uint32_t ptid) {
  p.mn = mn;
  if (!mn) {
    const uint32_t c = ptid & 7u, r = ptid >> 3;                // 32 rows per pass
    p.step = kTcBK;
#pragma unroll
    for (int i = 0; i < TcPlan<ROWS>::NCH; ++i) {
      const int64_t row = r + 32 * i;
      p.dst[i] = r * 128u + ((c ^ (r & 7u)) << 4) + static_cast<uint32_t>(i) * 4096u;
      p.bytes[i] = row < rows_valid ? 16u : 0u;
      p.src[i] = src + (row < rows_valid ? row : 0) * ld + 8 * c;
      p.koff[i] = 8u * c;
    }
  } else {
    constexpr uint32_t CPR = ROWS / 8;                          // chunks per k line
    constexpr uint32_t KPP = kTcProducers / CPR;                // k lines per pass
    const uint32_t cm = ptid % CPR, kr = ptid / CPR;
    const int64_t m = 8 * static_cast<int64_t>(cm);
    const uint32_t mbytes = m < rows_valid ? static_cast<uint32_t>(min(static_cast<int64_t>(16), 2 * (rows_valid - m))) : 0u;
    p.step = kTcBK * ld;
#pragma unroll
    for (int i = 0; i < TcPlan<ROWS>::NCH; ++i) {
      const uint32_t kk = kr + KPP * static_cast<uint32_t>(i);
      p.dst[i] = (cm >> 3) * 8192u + (kk >> 3) * 1024u + (kk & 7u) * 128u + (((cm & 7u) ^ (kk & 7u)) << 4);
      p.bytes[i] = mbytes;
      p.src[i] = src + kk * ld + (mbytes ? m : 0);
      p.koff[i] = kk;
    }
  }
}

// Issue the thread's chunks of k block `kb` into the stage at `sbase`.
template <int ROWS>
__device__ __forceinline__ void tc_issue(const TcPlan<ROWS> &p, uint32_t sbase, int64_t kb, int64_t K,
                                         const uint16_t *safe) {
  const int64_t k0 = kb * kTcBK;
  if (k0 + kTcBK <= K) {                 // a full k block: validity is the row's alone
#pragma unroll
    for (int i = 0; i < TcPlan<ROWS>::NCH; ++i)
      cp_async_16_zfill(sbase + p.dst[i], p.src[i] + kb * p.step, p.bytes[i]);
    return;
  }
#pragma unroll
  for (int i = 0; i < TcPlan<ROWS>::NCH; ++i) {
    const int64_t k = k0 + p.koff[i];
    uint32_t b = p.bytes[i];
    if (k >= K) b = 0u;
    else if (!p.mn) b = min(b, static_cast<uint32_t>(2 * (K - k)));
    cp_async_16_zfill(sbase + p.dst[i], b ? p.src[i] + kb * p.step : safe, b);
  }
}

__device__ __forceinline__ void tc_store_row32(uint8_t *dst, uint32_t dt, int64_t idx, const float (&v)[32], int64_t ncols,
                                               bool vec) {
  if (vec && ncols >= 32) {
    if (dt == kF32) {
      float4 *q = reinterpret_cast<float4 *>(dst + idx * 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
      uint4 *q = reinterpret_cast<uint4 *>(dst + idx * 2);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = v[8 * j + 2 * e], hi = v[8 * j + 2 * e + 1];
          w[e] = dt == kBF16 ? cvt_bf16x2(hi, lo) : (f32_to_f16_bits(lo) | (f32_to_f16_bits(hi) << 16));
        }
        q[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j < ncols) storef(dst, dt, idx + j, v[j]);
}

// Returns false (nothing done) when this launch cannot use the path (misaligned
// operand base); the caller then runs the CUDA-core path.
static __device__ __noinline__ bool mma_tc_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const DMma &dm = *reinterpret_cast<const DMma *>(P.desc + t.desc);
  const int64_t M = t.p[0], N = t.p[1], K = t.p[2], G = t.p[3] ? t.p[3] : 1;
  const uint32_t adt = t.adt, dt = t.dt;
  uint8_t *dst = resolve(P, t.ptr[0]);
  const uint8_t *Ab = resolve(P, t.ptr[1]);
  const uint8_t *Bb = resolve(P, t.ptr[2]);
  const uint8_t *res = t.p[6] ? resolve(P, t.ptr[3]) : nullptr;
  if ((reinterpret_cast<uintptr_t>(Ab) | reinterpret_cast<uintptr_t>(Bb)) & 15u) return false;
  if (!(dt == kF32 || dt == kBF16 || dt == kF16)) return false;
  const uint16_t *A = reinterpret_cast<const uint16_t *>(Ab) + dm.a_off;
  const uint16_t *B = reinterpret_cast<const uint16_t *>(Bb) + dm.b_off;
  const bool amn = dm.tc_mode & kTcAmn, bmn = dm.tc_mode & kTcBmn;
  const int64_t tn = (N + kMmaT - 1) / kMmaT, tm = (M + kMmaT - 1) / kMmaT, per = tm * tn;
  const int64_t nkb = (K + kTcBK - 1) / kTcBK;
  const bool vec_store = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && N % 8 == 0;
  const bool use_tma = dm.tmap >= 0;     // operands fetched by the TMA unit (else per-thread asynchronous copies)
  const DTmap *tm_a = use_tma ? P.tmaps + dm.tmap : nullptr, *tm_b = use_tma ? tm_a + 1 : nullptr;

  B2_DYN_SMEM(sm);
  TcShared *S = reinterpret_cast<TcShared *>(sm + kSmemRed);
  volatile uint32_t *failed = &S->failed;
  const uint32_t stage0 = (smem_addr(sm + kSmemSys) + 1023u) & ~1023u;
  const uint32_t w = L.tid / kWarp, lane = L.tid % kWarp;
  const unsigned long long budget = P.wait_budget_ns;

  __syncthreads();   // the scratch slot is free
  if (L.tid == 0) {
    for (int s = 0; s < kTcStages; ++s) { mbar_init(&S->full[s], use_tma ? 1u : static_cast<uint32_t>(kTcProducers)); mbar_init(&S->empty[s], 1); }
    // epilogue threads: warps 4-15 with TMA producers (twelve warps, three per lane quarter), else warps 8-15
    for (int b = 0; b < 2; ++b) { mbar_init(&S->acc_full[b], 1); mbar_init(&S->acc_empty[b], use_tma ? 384u : 256u); }
    S->failed = 0u;
    fence_mbar_init();
  }
  const uint32_t tcols = use_tma ? 2u * kTcCols : kTcCols;
  if (w == 8) {
    __syncwarp();
    tmem_alloc(&S->tmem_base, tcols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = S->tmem_base;

  // Rasterisation. The scheduler hands every lane a contiguous range of tile
  // *positions* (balanced split of [0, tiles) over the lanes), and the lanes walk
  // their ranges in step. Executing position p as tile p would make the lanes'
  // concurrent tiles a sparse scatter over the whole matrix (every block of A and
  // B live at once: far more than L2 holds, so the operands stream from HBM once
  // per use). Instead positions are mapped to tiles by a bijection chosen so that
  // what the lanes execute at the same time is a compact 2-D block of the output:
  // positions pair up (2u, 2u+1) -> the two halves of a 128 x 256 "wide tile", and
  // pair u of chunk j at step s gets rank s * k + j (wave-major), ranks filling the
  // wide-tile grid in groups of kRasterRows rows, column-major inside a group. Any
  // bijection keeps the result exact - every tile is still computed exactly once
  // within the task's barrier phase; only the locality depends on the guess k.
  constexpr int64_t kRasterRows = 16;
  const int64_t total_tiles = G * per;
  const int64_t U = per / 2, kch = min(static_cast<int64_t>(P.n_lanes), U);
  const bool raster = G == 1 && tn % 2 == 0 && U >= 2 * static_cast<int64_t>(P.n_lanes);
  const int64_t tnw = tn / 2;
  auto tile_of = [&](int64_t pos) -> int64_t {
    if (!raster) return pos;
    const int64_t u = pos >> 1, h = pos & 1;
    const int64_t j = ((u + 1) * kch - 1) / U;            // chunk of pair u under a balanced split
    const int64_t lo_j = U * j / kch, st = u - lo_j, c_lo = U / kch;
    const int64_t rank = st < c_lo ? st * kch + j : c_lo * kch + (lo_j - j * c_lo);
    const int64_t grp = rank / (kRasterRows * tnw), o = rank % (kRasterRows * tnw);
    const int64_t rows = min(kRasterRows, tm - grp * kRasterRows);
    const int64_t row = grp * kRasterRows + o % rows, pc = o / rows;
    return row * tn + 2 * pc + h;
  };
  // Enumerate the lane's super-tiles; every role walks the same sequence.
  auto next_super = [&](uint32_t &pos, int64_t &g, int64_t &r0, int64_t &c0, int &nt) -> bool {
    if (pos >= tile_hi || pos >= total_tiles) { pos = tile_hi; return false; }
    const int64_t tile = tile_of(pos);
    g = tile / per;
    const int64_t loc = tile % per, ti = loc / tn, tj = loc % tn;
    r0 = ti * kMmaT; c0 = tj * kMmaT;
    const bool pair = raster ? ((pos & 1u) == 0u) : (tj + 1 < tn);
    nt = (pair && pos + 1 < tile_hi && static_cast<int64_t>(pos) + 1 < total_tiles) ? 2 : 1;
    pos += nt;
    return true;
  };

  if (w < 8 && use_tma) {
    // ---------------- producer: one thread drives the TMA unit ----------------
    // Per stage: the A block (one 128-row box, or two 64-row-wide boxes when the rows
    // are the unit-stride dimension) and the B block likewise, each box landing as
    // one 128-byte-swizzled [rows][64] image - exactly the layout of the per-thread
    // path below. Boxes past the matrix edge arrive zero-filled.
    if (L.tid == 0) {
      uint32_t it = 0;
      uint32_t tile = tile_lo; int64_t g, r0, c0; int nt;
      bool ok = true;
      while (ok && next_super(tile, g, r0, c0, nt)) {
        const int32_t gi = static_cast<int32_t>(g), ri = static_cast<int32_t>(r0), ci = static_cast<int32_t>(c0);
        for (int64_t kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % kTcStages;
          if (!tc_wait(&S->empty[s], ((it / kTcStages) & 1u) ^ 1u, failed, budget)) { ok = false; break; }
          const uint32_t sa = stage0 + s * kTcStageBytes, sb = sa + kTcABytes;
          const int32_t k0 = static_cast<int32_t>(kb * kTcBK);
          if (amn) {
            tma_load_3d(sa, tm_a, ri, k0, gi, &S->full[s]);
            tma_load_3d(sa + 8192u, tm_a, ri + 64, k0, gi, &S->full[s]);
          } else {
            tma_load_3d(sa, tm_a, k0, ri, gi, &S->full[s]);
          }
          if (bmn) {
            for (int b = 0; b < 2 * nt; ++b) tma_load_3d(sb + 8192u * b, tm_b, ci + 64 * b, k0, gi, &S->full[s]);
          } else {
            for (int b = 0; b < nt; ++b) tma_load_3d(sb + 16384u * b, tm_b, k0, ci + 128 * b, gi, &S->full[s]);
          }
          mbar_arrive_tx(&S->full[s], static_cast<uint32_t>(kTcABytes + 16384 * nt));
        }
      }
    }
  } else if (w < 8) {
    // ---------------- producers: per-thread asynchronous copies ----------------
    const uint32_t ptid = L.tid;
    uint32_t it = 0;                              // stages issued
    uint32_t tile = tile_lo; int64_t g, r0, c0; int nt;
    bool ok = true;
    while (ok && next_super(tile, g, r0, c0, nt)) {
      const uint16_t *Ag = A + g * dm.a_gs + (amn ? r0 : r0 * dm.a_ld);
      const uint16_t *Bg = B + g * dm.b_gs + (bmn ? c0 : c0 * dm.b_ld);
      const int64_t a_rows = min(static_cast<int64_t>(kMmaT), M - r0);
      const int64_t b_rows = min(static_cast<int64_t>(kMmaT) * nt, N - c0);
      TcPlan<128> pa;
      tc_plan(pa, amn, Ag, dm.a_ld, a_rows, ptid);
      // The copies of a stage are asynchronous and so is their arrival on the stage's
      // "full" barrier: a producer never waits for data, only for a free stage, so
      // every free stage is in flight at once.
      auto run = [&](auto &pb) {
        for (int64_t kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % kTcStages;
          if (!tc_wait_warp(&S->empty[s], ((it / kTcStages) & 1u) ^ 1u, failed, budget)) { ok = false; break; }
          const uint32_t sa = stage0 + s * kTcStageBytes;
          tc_issue(pa, sa, kb, K, A);
          tc_issue(pb, sa + kTcABytes, kb, K, B);
          cp_async_mbar_arrive(&S->full[s]);
        }
      };
      if (nt == 2) {
        TcPlan<256> pb;
        tc_plan(pb, bmn, Bg, dm.b_ld, b_rows, ptid);
        run(pb);
      } else {
        TcPlan<128> pb;
        tc_plan(pb, bmn, Bg, dm.b_ld, b_rows, ptid);
        run(pb);
      }
    }
    cp_async_wait_all();                          // nothing of this thread is still in flight
  }
  // ---------------- MMA issue ----------------
  // With TMA producers (one thread) warp 1 is free to issue, so the accumulator is
  // double-buffered in tensor memory (columns 0 and 256) and the epilogue of one
  // super-tile runs under the main loop of the next. With per-thread producers the
  // issuing thread sits in epilogue warp 8 and there is one accumulator.
  const uint32_t nbuf = use_tma ? 2u : 1u;
  const uint32_t fmt = adt == kBF16 ? 1u : 0u;
  uint32_t mma_it = 0;                               // k blocks consumed so far (issuing thread only)
  auto issue_tile = [&](uint32_t n, int nt) -> bool {   // super-tile number n of this lane
    const uint32_t buf = n % nbuf, use = n / nbuf, ninst = 128u * nt;
    // the epilogue warps have drained this accumulator's previous contents
    if (!tc_wait(&S->acc_empty[buf], (use & 1u) ^ 1u, failed, budget)) return false;
    tc_fence_after_sync();
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((amn ? 1u : 0u) << 15) | ((bmn ? 1u : 0u) << 16) |
                           ((ninst >> 3) << 17) | ((128u >> 4) << 24);
    for (int64_t kb = 0; kb < nkb; ++kb, ++mma_it) {
      const uint32_t s = mma_it % kTcStages;
      if (!tc_wait(&S->full[s], (mma_it / kTcStages) & 1u, failed, budget)) return false;
      if (!use_tma) fence_proxy_async_smem();       // per-thread (generic-proxy) writes -> the MMA's async-proxy reads
      tc_fence_after_sync();
      const uint32_t sa = stage0 + s * kTcStageBytes, sb = sa + kTcABytes;
      const uint64_t da = amn ? tc_desc(sa, 8192u, 1024u) : tc_desc(sa, 16u, 1024u);
      const uint64_t db = bmn ? tc_desc(sb, 8192u, 1024u) : tc_desc(sb, 16u, 1024u);
      const uint64_t adv_a = amn ? (2048u >> 4) : (32u >> 4), adv_b = bmn ? (2048u >> 4) : (32u >> 4);
#pragma unroll
      for (uint32_t j = 0; j < kTcBK / 16; ++j)
        tc_mma_f16(tmem + buf * 256u, da + j * adv_a, db + j * adv_b, idesc, (kb > 0 || j > 0) ? 1u : 0u);
      tc_commit(&S->empty[s]);                    // frees the stage when these MMAs have read it
    }
    tc_commit(&S->acc_full[buf]);
    return true;
  };
  if (use_tma && w == 1 && lane == 0) {
    uint32_t n = 0;
    uint32_t tile = tile_lo; int64_t g, r0, c0; int nt;
    while (next_super(tile, g, r0, c0, nt) && issue_tile(n, nt)) ++n;
  }
  const uint32_t epi_first = use_tma ? 4u : 8u;      // first epilogue warp
  if (w >= epi_first) {
    // ---------------- epilogue ----------------
    // warp w reads tensor-memory lanes 32 (w % 4) .. +31; the warps sharing a lane quarter
    // split the accumulator's 32-column chunks round-robin
    const uint32_t ew = w - epi_first, q = w & 3u, slot = ew >> 2, nslots = (16u - epi_first) >> 2;
    // the store epilogue, decoded once: up to kEpiMax micro-ops {kind, operand source, s, t}
    constexpr int kEpiMax = 4;
    int epi_n = 0;
    uint32_t epi_kind[kEpiMax], epi_src[kEpiMax];
    float epi_s[kEpiMax], epi_t[kEpiMax];
    bool epi_generic = false;
    if (t.p[6]) {
      const int32_t *e = P.aux + (t.p[6] - 1u);
      epi_n = e[0];
      if (epi_n > kEpiMax) { epi_generic = true; epi_n = 0; }
#pragma unroll
      for (int mi = 0; mi < kEpiMax; ++mi) {
        const bool on = mi < epi_n;
        epi_kind[mi] = on ? static_cast<uint32_t>(e[1 + 4 * mi]) : 0u;
        epi_src[mi] = on ? static_cast<uint32_t>(e[2 + 4 * mi]) : 0u;
        epi_s[mi] = on ? __int_as_float(e[3 + 4 * mi]) : 0.0f;
        epi_t[mi] = on ? __int_as_float(e[4 + 4 * mi]) : 0.0f;
      }
    }
    // staging slab of this warp for coalesced stores (32 rows x 16 words, pitch 17), after the stages
    const uint32_t stg_off = stage0 - smem_addr(sm) + kTcStages * kTcStageBytes + ew * (32u * 17u * 4u);
    uint32_t *stg = reinterpret_cast<uint32_t *>(sm + stg_off);
    const bool coalesce = vec_store && stg_off + 32u * 17u * 4u <= L.smem_bytes;
    const uint32_t cdt = t.cdt;
    const bool vec_res = res && (reinterpret_cast<uintptr_t>(res) & 15u) == 0 && N % 8 == 0 && (cdt == kBF16 || cdt == kF32);
    uint32_t n = 0;
    uint32_t tile = tile_lo; int64_t g, r0, c0; int nt;
    bool ok = true;
    while (ok && next_super(tile, g, r0, c0, nt)) {
      const uint32_t buf = n % nbuf, use = n / nbuf, ninst = 128u * nt;
      if (!use_tma) {
        if (w == 8 && lane == 0) ok = issue_tile(n, nt);
        __syncwarp();
      }
      // wait for the accumulator (voted: the whole warp leaves together if the wait ran out)
      if (!tc_wait_warp(&S->acc_full[buf], use & 1u, failed, budget, 64u)) { ok = false; break; }
      ++n;
      tc_fence_after_sync();
      const int64_t r = r0 + 32 * q + lane;
#pragma unroll 1
      for (uint32_t col = 32u * slot; col < ninst; col += 32u * nslots) {
        uint32_t raw[32];
        __syncwarp();   // the warp-wide tensor-memory load needs all 32 lanes back together
                        // (rows beyond M leave the store below divergent)
        tc_ld32(tmem + ((32u * q) << 16) + buf * 256u + col, raw);
        tc_wait_ld();
        const int64_t c = c0 + col;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
        if (r < M && c < N) {
          const int64_t ncols = min(static_cast<int64_t>(32), N - c);
          // v[] and y[] are only ever indexed by constants, so they stay in registers; the rare paths that walk
          // columns in a rolled loop do it on copies of their own (which live in local memory).
          if (epi_generic) {
            float tv[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) tv[j] = v[j];
#pragma unroll 1
            for (int j = 0; j < 32; ++j)
              if (j < ncols) tv[j] = mma_epilogue(P, t, res, tv[j], g, r, c + j, M, N);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = tv[j];
          }
#pragma unroll
          for (int mi = 0; mi < kEpiMax; ++mi) {
            if (mi >= epi_n) break;
            const float es = epi_s[mi], et = epi_t[mi];
            const uint32_t kind = epi_kind[mi];
            // one-operand micro-ops never materialise a second operand (32 more live registers)
            if (kind == kGelu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
              continue;
            }
            if (kind == kAffine) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = affine2(v[j], es, et);
              continue;
            }
            float y[32];
            if (epi_src[mi]) {      // 1: the residual's element, 2: the per-column vector's
              const int64_t yi = epi_src[mi] == 1u ? (g * M + r) * N + c : c;
              if (vec_res && ncols == 32) {
                if (cdt == kF32) {
                  const float4 *yp = reinterpret_cast<const float4 *>(res + yi * 4);
#pragma unroll
                  for (int j = 0; j < 8; ++j) { const float4 f = yp[j]; y[4 * j] = f.x; y[4 * j + 1] = f.y; y[4 * j + 2] = f.z; y[4 * j + 3] = f.w; }
                } else {
                  const uint4 *yp = reinterpret_cast<const uint4 *>(res + yi * 2);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const uint4 u = yp[j];
                    y[8 * j] = bf16_bits_to_f32(u.x & 0xffffu); y[8 * j + 1] = __uint_as_float(u.x & 0xffff0000u);
                    y[8 * j + 2] = bf16_bits_to_f32(u.y & 0xffffu); y[8 * j + 3] = __uint_as_float(u.y & 0xffff0000u);
                    y[8 * j + 4] = bf16_bits_to_f32(u.z & 0xffffu); y[8 * j + 5] = __uint_as_float(u.z & 0xffff0000u);
                    y[8 * j + 6] = bf16_bits_to_f32(u.w & 0xffffu); y[8 * j + 7] = __uint_as_float(u.w & 0xffff0000u);
                  }
                }
              } else {
                float ty[32];
#pragma unroll 1
                for (int j = 0; j < 32; ++j) ty[j] = j < ncols ? loadf(res, cdt, yi + j) : 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) y[j] = ty[j];
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) y[j] = v[j];
            }
            switch (kind) {     // one dispatch, the 32 evaluations inside
              case kAdd: _Pragma("unroll") for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(v[j], y[j]); break;
              case kMul: _Pragma("unroll") for (int j = 0; j < 32; ++j) v[j] = __fmul_rn(v[j], y[j]); break;
              case kSubt: _Pragma("unroll") for (int j = 0; j < 32; ++j) v[j] = __fsub_rn(v[j], y[j]); break;
              case kMax: _Pragma("unroll") for (int j = 0; j < 32; ++j) v[j] = np_max(v[j], y[j]); break;
              default: {
                float tv[32], ty[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) { tv[j] = v[j]; ty[j] = y[j]; }
#pragma unroll 1
                for (int j = 0; j < 32; ++j) tv[j] = micro_alu(kind, tv[j], ty[j], es, et);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = tv[j];
                break;
              }
            }
          }
          if (!(coalesce && c + 32 <= N)) tc_store_row32(dst, dt, (g * M + r) * N + c, v, ncols, vec_store);
        }
        if (coalesce && c + 32 <= N) {
          // Each thread holds 32 consecutive columns of ONE row: stored directly, a warp
          // instruction would touch 32 rows with 16 bytes each (half-filled sectors). The
          // warp's 32 x 32 block goes through its staging slab instead and leaves as
          // 64-byte row segments, 4 lanes per row, 8 rows per instruction.
          const uint32_t esz = dt == kF32 ? 4u : 2u;
#pragma unroll
          for (uint32_t h = 0; h < 2; ++h) {          // f32: two 16-column halves; 2-byte types: one pass
            if (h == 1 && esz == 2u) break;
            __syncwarp();
            if (esz == 4u) {
#pragma unroll
              for (int j = 0; j < 16; ++j) stg[lane * 17u + j] = __float_as_uint(v[16 * h + j]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float lo = v[2 * j], hi = v[2 * j + 1];
                stg[lane * 17u + j] = dt == kBF16 ? cvt_bf16x2(hi, lo) : (f32_to_f16_bits(lo) | (f32_to_f16_bits(hi) << 16));
              }
            }
            __syncwarp();
#pragma unroll
            for (uint32_t pass = 0; pass < 4; ++pass) {
              const uint32_t row = pass * 8u + (lane >> 2), ch = lane & 3u;
              const int64_t rr = r0 + 32 * q + row;
              if (rr < M) {
                const uint32_t *sp = stg + row * 17u + ch * 4u;
                uint8_t *gp = dst + ((g * M + rr) * N + c) * esz + h * 64u + ch * 16u;
                *reinterpret_cast<uint4 *>(gp) = make_uint4(sp[0], sp[1], sp[2], sp[3]);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&S->acc_empty[buf]);            // this thread is done with the accumulator
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  // A wait that ran out leaves copies and MMAs of other roles possibly still in flight
  // towards the stages, their barriers and the accumulator. They all complete within
  // microseconds on their own (nothing they wait for is outstanding), so the failed
  // path gives them that time before tensor memory goes back, and leaves the barriers
  // valid instead of invalidating words a late completion may still signal.
  const bool gave_up = S->failed != 0u;
  if (gave_up) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 50000ull) nanosleep_ns(1000);
  }
  if (w == 8) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, tcols);
  }
  if (L.tid == 0) {
    if (gave_up) set_status(P, kStTensorTimeout, L.lane, tile_lo, kTopMma);
    if (!gave_up) {
      for (int s = 0; s < kTcStages; ++s) { mbar_inval(&S->full[s]); mbar_inval(&S->empty[s]); }
      for (int b = 0; b < 2; ++b) { mbar_inval(&S->acc_full[b]); mbar_inval(&S->acc_empty[b]); }
    }
  }
  __syncthreads();
  return true;
}

#else   // no tensor-core instructions in this build

__device__ __forceinline__ bool mma_tc_tiles(const Lane &, const DTask &, uint32_t, uint32_t) { return false; }

#endif

}  // namespace b2
#endif
