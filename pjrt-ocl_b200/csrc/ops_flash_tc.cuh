// TILE_FLASH_ATTN on the tensor cores: S = Q K^T and O = P V as tcgen05.mma with the
// accumulators in tensor memory, online softmax in between.
//
// Same contract as the CUDA-core path (ops_flash.cuh; pjrt_plugin/kernels/ops/
// attention.cl:49-159; python/pjrt_ocl/ops/attention.py:52-66): tile = one query row
// (head g, position m) of out[H,T,hd]; Q [H,T,hd], K given as the QK^T matmul's B
// operand [H,hd,C], V [H,C,hd], each possibly through a view; with `causal` key c is
// masked when c > m + C - T. Taken for bf16 / f16 operands with head_dim 64 whose
// (viewed) layouts three rank-4 TMA tensor maps can describe (DFlash::tc_mode; the
// loader decides), so a [batch, seq, heads, hd] projection is attended in place.
//
// Work unit: 256 consecutive query rows of one head = two 128-row tiles ("slots" A and
// B) that share one stream of 128-key K / V blocks. Units are handed out heaviest first
// from a counter in the program's scratch when the loader allowed it (causal units
// differ 10 x in cost), else a lane takes the units that start inside its row range.
// Per unit, over the key blocks j:
//   warp 0   one thread drives TMA: Q tiles once, then K(j) / V(j) through a 3-stage ring
//            (operands land in the 128-byte-swizzled layouts the tensor core reads);
//   warp 1   one thread issues the MMAs: S_s(j) = Q_s K(j)^T (128 x 128 x 64) into the
//            slot's score columns, O_s (+)= P_s(j) V(j) (128 x 64 x 128) into the slot's
//            output columns, ordered PV_A(j), S_A(j+1), PV_B(j), S_B(j+1) so one slot's
//            matmuls run under the other slot's softmax;
//   warps 4-7 / 8-11   softmax of slot A / B, one thread per query row: pass 1 reads the
//            row's 128 scores from tensor memory for the maximum, pass 2 reads them again,
//            exponentiates (log2 domain, one ex2 each), and writes P as 16-bit values into
//            shared memory for the second matmul. O stays in tensor memory for the whole
//            unit; it is rescaled in place (tcgen05.ld / st) only when a row's maximum grew
//            by more than 2^8 since the maximum in use was set - P then stays below 256 and
//            the result is mathematically unchanged. Finally out = O / (row sum).
// Every wait is bounded; a wait that runs out ends the task with a status.
#ifndef B2VM_OPS_FLASH_TC_CUH_
#define B2VM_OPS_FLASH_TC_CUH_

#include "ops_flash.cuh"
#include "ops_mma_tc.cuh"

namespace b2 {

#if B2_HAS_TC

constexpr int kFaStages = 3;
constexpr uint32_t kFaTile = 128 * 128;        // bytes of a Q tile, a K block or a V block (128 x 64 x 2)
constexpr uint32_t kFaPBytes = 2 * 128 * 128;  // P of one slot: 128 rows x 128 keys = two 64-key sub-tiles
constexpr uint32_t kFaCols = 512;              // S_A 0, S_B 128, O_A 256, O_B 320
constexpr float kFaRescale = 8.0f;             // log2 of the growth of a row maximum that forces a rescale

struct FaShared {
  uint64_t q_full;
  uint64_t kv_full[kFaStages];
  uint64_t kv_empty[kFaStages];
  uint64_t s_full[2];       // MMA -> softmax: the slot's scores are in tensor memory
  uint64_t s_free[2];       // softmax -> MMA: the scores have been read (4 warp arrivals)
  uint64_t p_full[2];       // softmax -> MMA: P is in shared memory, O is rescaled (4 warp arrivals)
  uint64_t pv_done[2];      // MMA -> softmax: O_s holds block j, P's buffer is free
  uint32_t tmem_base;
  uint32_t failed;
  uint32_t unit;            // the unit all roles work on next, or 0xffffffff
  uint32_t pad;
};
static_assert(sizeof(FaShared) <= 512, "fits the scratch slot");

template <typename Lane>
static __device__ __noinline__ bool flash_tc_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const DFlash &df = *reinterpret_cast<const DFlash *>(P.desc + t.desc);
  const int32_t *x = P.aux + t.p[3];
  const int64_t H = x[0], T = x[1], C = x[2];
  constexpr int64_t hd = 64;
  const float sl2 = __int_as_float(x[4]) * 1.4426950408889634f;   // scores in the log2 domain
  const bool causal = x[5] != 0;
  uint8_t *out = resolve(P, t.ptr[0]);
  if (df.tmap < 0 || (reinterpret_cast<uintptr_t>(out) & 15u)) return false;
  const DTmap *tm_q = P.tmaps + df.tmap, *tm_k = tm_q + 1, *tm_v = tm_q + 2;
  const uint32_t adt = t.adt, dt = t.dt;
  const int64_t rows_end = min(static_cast<int64_t>(tile_hi), H * T);
  if (static_cast<int64_t>(tile_lo) >= rows_end && df.work_slot == kNoWorkSlot) return true;

  B2_DYN_SMEM(sm);
  FaShared *S = reinterpret_cast<FaShared *>(sm + kSmemRed);
  volatile uint32_t *failed = &S->failed;
  const uint32_t base0 = (smem_addr(sm + kSmemSys) + 1023u) & ~1023u;
  const uint32_t q_s = base0, kv_s = q_s + 2u * kFaTile, p_s = kv_s + kFaStages * 2u * kFaTile;
  const uint32_t w = __shfl_sync(0xffffffffu, L.tid / kWarp, 0), lane = L.tid % kWarp;   // the warp index, provably uniform
  const unsigned long long budget = P.wait_budget_ns;
  const bool k_mn = df.k_mn != 0;

  __syncthreads();   // the scratch slot and the workspace are free
  if (L.tid == 0) {
    mbar_init(&S->q_full, 1);
    for (int s = 0; s < kFaStages; ++s) { mbar_init(&S->kv_full[s], 1); mbar_init(&S->kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&S->s_full[b], 1); mbar_init(&S->s_free[b], 4); mbar_init(&S->p_full[b], 4); mbar_init(&S->pv_done[b], 1);
    }
    S->failed = 0u;
    fence_mbar_init();
  }
  if (w == 1) {
    __syncwarp();
    tmem_alloc(&S->tmem_base, kFaCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = S->tmem_base;

  // ---- units: 256-row blocks aligned inside a head ----
  const int64_t upm = (T + 255) / 256;                 // units per head
  const int64_t n_units = H * upm;
  const bool dynamic = df.work_slot != kNoWorkSlot;
  uint32_t *work = dynamic ? reinterpret_cast<RedScratch *>(P.scratch)->work + 2u * df.work_slot : nullptr;
  // static mode: the units whose first row lies in [tile_lo, rows_end)
  int64_t u_next = 0, u_stop = 0;
  if (!dynamic) {
    const int64_t first = static_cast<int64_t>(tile_lo);
    auto unit_at_or_after = [&](int64_t row) {       // index of the first unit starting at a row >= `row`
      const int64_t g = row / T, m = row % T;
      return g * upm + (m + 255) / 256;
    };
    u_next = unit_at_or_after(first);
    u_stop = unit_at_or_after(rows_end);
  }
  // ring / phase positions, carried across units by every role that uses them
  uint32_t kvpos = 0, qn = 0, cnt[2] = {0u, 0u};

  for (;;) {
    // ---- next unit (one thread decides, everybody reads it after the barrier) ----
    if (L.tid == 0) {
      uint32_t u = 0xffffffffu;
      if (dynamic) {
        const uint32_t tk = atomicAdd(&work[0], 1u);
        if (static_cast<int64_t>(tk) < n_units) {
          // heaviest first: with a causal mask the last 256 rows of a head see the most keys
          const int64_t lvl = tk / H, g = tk % H;
          u = static_cast<uint32_t>(g * upm + (causal ? upm - 1 - lvl : lvl));
        }
      } else if (u_next < u_stop) {
        u = static_cast<uint32_t>(u_next++);
      }
      S->unit = u;
    }
    tc_fence_before_sync();
    __syncthreads();       // also: every role is done with the previous unit (Q, P, the rings, tensor memory)
    tc_fence_after_sync();
    const uint32_t unit = __shfl_sync(0xffffffffu, S->unit, 0);
    if (unit == 0xffffffffu || S->failed) break;
    const int64_t g = unit / upm, m0 = (unit % upm) * 256;
    const int32_t h0c = static_cast<int32_t>(g % df.h0_size), h1c = static_cast<int32_t>(g / df.h0_size);
    // key blocks each slot needs
    int64_t nkb[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int64_t ms = m0 + 128 * s, rows_q = min(static_cast<int64_t>(128), T - ms);
      const int64_t c_max = rows_q <= 0 ? 0 : (causal ? min(C, ms + rows_q + (C - T)) : C);
      nkb[s] = c_max <= 0 ? 0 : (c_max + 127) / 128;
    }
    const int64_t nmax = max(nkb[0], nkb[1]);

    if (w == 0) {
      // ---------------- producer: one thread drives TMA ----------------
      if (lane == 0) {
        tma_load_4d(q_s, tm_q, 0, static_cast<int32_t>(m0), h0c, h1c, &S->q_full);        // rows past T arrive as zeros
        tma_load_4d(q_s + kFaTile, tm_q, 0, static_cast<int32_t>(m0 + 128), h0c, h1c, &S->q_full);
        mbar_arrive_tx(&S->q_full, 2u * kFaTile);
        for (int64_t j = 0; j < nmax; ++j) {
          const uint32_t pos = kvpos + static_cast<uint32_t>(j), st = pos % kFaStages;
          if (!tc_wait(&S->kv_empty[st], ((pos / kFaStages) & 1u) ^ 1u, failed, budget, 32u)) break;
          const uint32_t ks = kv_s + st * 2u * kFaTile, vs = ks + kFaTile;
          const int32_t c0 = static_cast<int32_t>(j * 128);
          if (k_mn) {       // K as [d][keys]: two boxes of 64 keys x 64 d
            tma_load_4d(ks, tm_k, c0, 0, h0c, h1c, &S->kv_full[st]);
            tma_load_4d(ks + 8192u, tm_k, c0 + 64, 0, h0c, h1c, &S->kv_full[st]);
          } else {          // K as [keys][d]: one box of 128 keys x 64 d
            tma_load_4d(ks, tm_k, 0, c0, h0c, h1c, &S->kv_full[st]);
          }
          tma_load_4d(vs, tm_v, 0, c0, h0c, h1c, &S->kv_full[st]);
          mbar_arrive_tx(&S->kv_full[st], 2u * kFaTile);
        }
      }
      __syncwarp();
    } else if (w == 1) {
      // ---------------- MMA issue ----------------
      // The whole warp walks the loop with warp-uniform control (votes, shuffles from lane 0) and one
      // elected lane issues: operands that the compiler can prove uniform stay in uniform registers,
      // which is what makes a tcgen05.mma cheap to issue (measured: ~95 cycles each from a thread inside
      // a lane == 0 branch, where every operand has to be moved over first).
      {
        const uint32_t fmt = adt == kBF16 ? 1u : 0u;
        // S: A = Q (K-major), B = K block; O: A = P (K-major), B = V (d is the unit-stride "MN" dimension)
        const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((k_mn ? 1u : 0u) << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
        bool ok = tc_wait_warp(&S->q_full, qn & 1u, failed, budget);
        tc_fence_after_sync();
        // Descriptors of stage 0 / slot 0; the others differ in the 16-byte-unit address field only.
        const uint64_t dq0 = tc_desc(q_s, 16u, 1024u), dp0 = tc_desc(p_s, 16u, 1024u);
        const uint64_t dk0 = k_mn ? tc_desc(kv_s, 8192u, 1024u) : tc_desc(kv_s, 16u, 1024u);
        const uint64_t dv0 = tc_desc(kv_s + kFaTile, 16384u, 1024u);
        const uint64_t adv_b = k_mn ? (2048u >> 4) : (32u >> 4);
        const bool issuer = elect_one_sync();
        // The issuer is an event loop over both slots: S(j+1) of a slot goes out as soon as the slot's
        // scores are in registers (s_free) and the keys have landed; P.V(j) when the slot's P is written.
        // S is tried first, so the next scores are ready when the softmax warps finish a block.
        uint32_t ns[2] = {0u, 0u}, npv[2] = {0u, 0u}, released = 0u;
        const uint32_t nk0 = static_cast<uint32_t>(nkb[0]), nk1 = static_cast<uint32_t>(nkb[1]), nmx = static_cast<uint32_t>(nmax);
        uint32_t kv_seen = 0, idle = 0;
        unsigned long long t_idle = 0;
        while (ok) {
          bool progressed = false, done = true;
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t nk = s ? nk1 : nk0;
            if (ns[s] < nk) {
              done = false;
              const uint32_t j = ns[s];
              if (kv_seen <= j) {
                const uint32_t pos = kvpos + kv_seen;
                if (__all_sync(0xffffffffu, mbar_test_wait_parity(&S->kv_full[pos % kFaStages], (pos / kFaStages) & 1u))) ++kv_seen;
              }
              if (kv_seen > j && (j == 0u || __all_sync(0xffffffffu, mbar_test_wait_parity(&S->s_free[s], (cnt[s] + j - 1u) & 1u)))) {
                tc_fence_after_sync();
                const uint32_t st = (kvpos + j) % kFaStages;
                const uint64_t da = dq0 + static_cast<uint32_t>(s) * (kFaTile >> 4);
                const uint64_t db = dk0 + st * ((2u * kFaTile) >> 4);
                if (issuer) {
#pragma unroll
                  for (uint32_t kk = 0; kk < 4; ++kk)
                    tc_mma_f16(tmem + static_cast<uint32_t>(s) * 128u, da + kk * (32u >> 4), db + kk * adv_b, idesc_s, kk ? 1u : 0u);
                  tc_commit(&S->s_full[s]);
                }
                __syncwarp();
                ++ns[s];
                progressed = true;
              }
            }
            if (npv[s] < nk) {
              done = false;
              const uint32_t j = npv[s];
              if (ns[s] > j && __all_sync(0xffffffffu, mbar_test_wait_parity(&S->p_full[s], (cnt[s] + j) & 1u))) {
                tc_fence_after_sync();
                const uint32_t st = (kvpos + j) % kFaStages;
                const uint64_t dp = dp0 + static_cast<uint32_t>(s) * (kFaPBytes >> 4);
                const uint64_t dv = dv0 + st * ((2u * kFaTile) >> 4);
                if (issuer) {
#pragma unroll
                  for (uint32_t kk = 0; kk < 8; ++kk)
                    tc_mma_f16(tmem + 256u + static_cast<uint32_t>(s) * 64u, dp + ((kk >> 2) * 16384u + (kk & 3u) * 32u) / 16u,
                               dv + kk * (2048u >> 4), idesc_o, (j > 0u || kk > 0u) ? 1u : 0u);
                  tc_commit(&S->pv_done[s]);
                }
                __syncwarp();
                ++npv[s];
                progressed = true;
              }
            }
          }
          // a stage is free when the matmuls of both slots that read it have completed
          while (released < nmx && (released >= nk0 || npv[0] > released) && (released >= nk1 || npv[1] > released)) {
            if (issuer) tc_commit(&S->kv_empty[(kvpos + released) % kFaStages]);
            __syncwarp();
            ++released;
          }
          if (done) break;
          if (progressed) {
            idle = 0;
            continue;
          }
          nanosleep_ns(32);      // leave the issue slots to the softmax warps of this scheduler
          if ((++idle & 1023u) == 0u) {
            uint32_t give_up = 0u;
            if (lane == 0) {
              if (*failed) give_up = 1u;
              const unsigned long long now = globaltimer_ns();
              if (idle == 1024u) t_idle = now;
              else if (now - t_idle > budget) { *failed = 1u; give_up = 1u; }
            }
            if (__shfl_sync(0xffffffffu, give_up, 0)) { ok = false; break; }
          }
        }
      }
      __syncwarp();
    } else if (w >= 4 && w < 12) {
      // ---------------- softmax + output: one thread per query row ----------------
      const int s = w >= 8 ? 1 : 0;
      const uint32_t q4 = w & 3u, r = 32u * q4 + lane;
      const int64_t m = m0 + 128 * s + r, grow = g * T + m;
      const bool row_ok = m < T;
      const int64_t c_end = causal ? min(C, m + (C - T) + 1) : C;    // keys this row may see
      const uint32_t s_addr = tmem + ((32u * q4) << 16) + static_cast<uint32_t>(s) * 128u;
      const uint32_t o_addr = tmem + ((32u * q4) << 16) + 256u + static_cast<uint32_t>(s) * 64u;
      const uint32_t prow = p_s + static_cast<uint32_t>(s) * kFaPBytes + r * 128u;
      const bool bf = adt == kBF16;
      float m_used = -INFINITY, l_run = 0.0f;
      bool ok = true;
      const int64_t nb = nkb[s];
      for (int64_t j = 0; ok && j < nb; ++j) {
        const uint32_t use = cnt[s] + static_cast<uint32_t>(j);
        if (!tc_wait_warp(&S->s_full[s], use & 1u, failed, budget)) { ok = false; break; }
        tc_fence_after_sync();
        const int lim = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(128), c_end - j * 128)));
        // pass 1: the row's maximum over this block
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four independent chains
#pragma unroll 1
        for (int cb = 0; cb < 128; cb += 32) {
          uint32_t raw[32];
          __syncwarp();
          tc_ld32(s_addr + cb, raw);
          tc_wait_ld();
          if (cb + 32 <= lim) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cb + i < lim) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[i]));
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        mx *= sl2;     // sl2 > 0 for every softmax scale in use; a non-positive scale takes the CUDA-core path
        // the maximum in use moves only when the row's true maximum outgrew it by 2^8
        const bool grow_m = mx > m_used + kFaRescale;
        const float alpha = !grow_m ? 1.0f : (m_used == -INFINITY ? 0.0f : fast_ex2(m_used - mx));
        // O(j-1) complete, P's buffer free
        if (j > 0 && !tc_wait_warp(&S->pv_done[s], (use - 1u) & 1u, failed, budget)) { ok = false; break; }
        tc_fence_after_sync();
        if (j > 0 && __any_sync(0xffffffffu, grow_m)) {
#pragma unroll 1
          for (int cb = 0; cb < 64; cb += 32) {
            uint32_t raw[32];
            __syncwarp();
            tc_ld32(o_addr + cb, raw);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
            tc_st32(o_addr + cb, raw);
          }
          tc_wait_st();
        }
        if (grow_m) { l_run *= alpha; m_used = mx; }
        const float neg_m = m_used == -INFINITY ? 0.0f : -m_used;
        // pass 2: p = 2^(s - m_used), written as the 16-bit A operand of the second matmul
        float ps4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
        for (int cb = 0; cb < 128; cb += 32) {
          uint32_t raw[32];
          __syncwarp();
          tc_ld32(s_addr + cb, raw);
          tc_wait_ld();
          if (cb == 96) {            // the scores are in registers: the slot's next S may be written
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S->s_free[s]);
          }
          float pv[32];
          if (cb + 32 <= lim) {
#pragma unroll
            for (int i = 0; i < 32; ++i) pv[i] = fast_ex2(fmaf(__uint_as_float(raw[i]), sl2, neg_m));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) pv[i] = cb + i < lim ? fast_ex2(fmaf(__uint_as_float(raw[i]), sl2, neg_m)) : 0.0f;
          }
          uint32_t pk[16];
          if (bf) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = cvt_bf16x2(pv[2 * i + 1], pv[2 * i]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = f32_to_f16_bits(pv[2 * i]) | (f32_to_f16_bits(pv[2 * i + 1]) << 16);
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) ps4[i & 3] += pv[i];
          // 32 keys = 4 chunks of 8 in the row's 128-byte line of sub-tile cb / 64
          const uint32_t sub = prow + (static_cast<uint32_t>(cb) >> 6) * 16384u;
#pragma unroll
          for (uint32_t q = 0; q < 4; ++q) {
            const uint32_t ch = ((static_cast<uint32_t>(cb) & 63u) >> 3) + q;
            uint4 *dstp = reinterpret_cast<uint4 *>(sm + (sub + ((ch ^ (r & 7u)) << 4) - smem_addr(sm)));
            *dstp = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
          }
        }
        l_run += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        tc_fence_before_sync();
        fence_proxy_async_smem();               // P (generic-proxy stores) -> the MMA's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&S->p_full[s]);
      }
      // ---- output: O / l ----
      if (ok && nb > 0) {
        const uint32_t use = cnt[s] + static_cast<uint32_t>(nb) - 1u;
        if (!tc_wait_warp(&S->pv_done[s], use & 1u, failed, budget)) ok = false;
        tc_fence_after_sync();
        if (ok) {
          const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll 1
          for (int cb = 0; cb < 64; cb += 32) {
            uint32_t raw[32];
            __syncwarp();
            tc_ld32(o_addr + cb, raw);
            tc_wait_ld();
            if (row_ok) {
              float v[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]) * inv;
              tc_store_row32(out, dt, grow * hd + cb, v, 32, true);
            }
          }
        }
      }
    }
    kvpos += static_cast<uint32_t>(nmax);
    cnt[0] += static_cast<uint32_t>(nkb[0]);
    cnt[1] += static_cast<uint32_t>(nkb[1]);
    ++qn;
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  const bool gave_up = S->failed != 0u;
  if (gave_up) {     // copies / matmuls of other roles may still be landing: give them time (see ops_mma_tc.cuh)
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 50000ull) nanosleep_ns(1000);
  }
  if (w == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, kFaCols);
  }
  if (L.tid == 0) {
    if (gave_up) {
      set_status(P, kStTensorTimeout, L.lane, tile_lo, kTopFlashAttn);
    } else {
      mbar_inval(&S->q_full);
      for (int s = 0; s < kFaStages; ++s) { mbar_inval(&S->kv_full[s]); mbar_inval(&S->kv_empty[s]); }
      for (int b = 0; b < 2; ++b) {
        mbar_inval(&S->s_full[b]); mbar_inval(&S->s_free[b]); mbar_inval(&S->p_full[b]); mbar_inval(&S->pv_done[b]);
      }
    }
    if (dynamic) {
      // the last lane to finish puts the counters back to rest for the task's next run
      __threadfence();
      if (atomicAdd(&work[1], 1u) == df.n_owner_lanes - 1u) { st_relaxed_gpu(&work[0], 0u); st_relaxed_gpu(&work[1], 0u); }
    }
  }
  __syncthreads();
  return true;
}

#else

__device__ __forceinline__ bool flash_tc_tiles(const Lane &, const DTask &, uint32_t, uint32_t) { return false; }

#endif

}  // namespace b2
#endif
