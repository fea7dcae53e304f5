// TILE_FLASH_ATTN on the tensor cores: S = Q K^T and O = P V as tcgen05.mma with the
// accumulators in tensor memory, online softmax in between.
//
// Same contract as the CUDA-core path (ops_flash.cuh; pjrt_plugin/kernels/ops/
// attention.cl:49-159; python/pjrt_ocl/ops/attention.py:52-66): tile = one query row
// (head g, position m) of out[H,T,hd]; Q [H,T,hd], K given as the QK^T matmul's B
// operand [H,hd,C], V [H,C,hd]; with `causal` key c is masked when c > m + C - T.
// Taken for bf16 / f16 operands without views and head_dim 64 (DFlash::tc_mode).
//
// A lane's range of query rows is covered by 128-row blocks aligned inside a head
// (rows outside the lane's range are computed and dropped: a block that straddles
// two lanes' ranges is computed by both). Per block, over 128-key blocks:
//   warps 0-3   producers: Q once, then K^T / V blocks through a 3-stage ring,
//               16-byte asynchronous copies into the swizzled operand layouts;
//   warp 4      lane 0 issues S(j) = Q K(j)^T  (M 128, N 128, K 64) into one of two
//               S buffers, and O(j) = P(j) V(j) (M 128, N 64, K 128) into one of two O
//               buffers, S(j+1) being issued ahead of O(j);
//   warps 8-15  softmax: two threads per query row (row = tensor-memory lane, the pair
//               splits the 128 key columns and the 64 output columns): read S(j), mask,
//               exchange the half-row maxima through shared memory, write P(j) as
//               16-bit values into shared memory for the second matmul, then fold
//               O(j-1) into the register accumulator with the rescale factor; finally
//               out = acc / (sum of the two half-row sums).
// Scores are handled in the log2 domain (one ex2 per score). Every wait is bounded.
#ifndef B2VM_OPS_FLASH_TC_CUH_
#define B2VM_OPS_FLASH_TC_CUH_

#include "ops_flash.cuh"
#include "ops_mma_tc.cuh"

namespace b2 {

#if B2_HAS_TC

constexpr int kFaStages = 3;
constexpr int kFaQBytes = 128 * 128;          // Q block: 128 rows x 64 d
constexpr int kFaKvBytes = 2 * 128 * 128;     // K^T block (64 d x 128 keys) + V block (128 keys x 64 d)
constexpr int kFaPBytes = 2 * 128 * 128;      // P block: 128 rows x 128 keys = two 64-key sub-tiles
constexpr uint32_t kFaCols = 512;             // S0 S1 at columns 0 / 128, O0 O1 at 256 / 320

struct FaShared {
  uint64_t q_full;
  uint64_t kv_full[kFaStages];
  uint64_t kv_empty[kFaStages];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_full[2];
  uint64_t mx_full[2];      // both halves of every row have published their block maximum
  uint64_t l_full;          // ... their final row sums
  uint32_t tmem_base;
  uint32_t failed;
};
static_assert(sizeof(FaShared) <= 512, "fits the scratch slot");

__device__ __noinline__ bool flash_tc_tiles(const Lane &L, const DTask &t, uint32_t tile_lo, uint32_t tile_hi) {
  const KParams &P = *L.P;
  const int32_t *x = P.aux + t.p[3];
  const int64_t H = x[0], T = x[1], C = x[2];
  constexpr int64_t hd = 64;
  const float sl2 = __int_as_float(x[4]) * 1.4426950408889634f;   // scores in the log2 domain
  const bool causal = x[5] != 0;
  uint8_t *out = resolve(P, t.ptr[0]);
  const uint8_t *Qb = resolve(P, t.ptr[1]);
  const uint8_t *Kb = resolve(P, t.ptr[2]);
  const uint8_t *Vb = resolve(P, t.ptr[3]);
  if ((reinterpret_cast<uintptr_t>(Qb) | reinterpret_cast<uintptr_t>(Kb) | reinterpret_cast<uintptr_t>(Vb) |
       reinterpret_cast<uintptr_t>(out)) & 15u)
    return false;
  const uint16_t *Q = reinterpret_cast<const uint16_t *>(Qb);
  const uint16_t *KT = reinterpret_cast<const uint16_t *>(Kb);
  const uint16_t *V = reinterpret_cast<const uint16_t *>(Vb);
  const uint32_t adt = t.adt, dt = t.dt;
  const int64_t rows_end = min(static_cast<int64_t>(tile_hi), H * T);
  if (static_cast<int64_t>(tile_lo) >= rows_end) return true;

  B2_DYN_SMEM(sm);
  FaShared *S = reinterpret_cast<FaShared *>(sm + kSmemRed);
  volatile uint32_t *failed = &S->failed;
  const uint32_t base0 = (smem_addr(sm + kSmemSys) + 1023u) & ~1023u;
  const uint32_t q_s = base0, kv_s = q_s + kFaQBytes, p_s = kv_s + kFaStages * kFaKvBytes;
  const uint32_t w = L.tid / kWarp, lane = L.tid % kWarp;
  const unsigned long long budget = P.wait_budget_ns;

  __syncthreads();   // the scratch slot and the workspace are free
  if (L.tid == 0) {
    mbar_init(&S->q_full, 128);
    for (int s = 0; s < kFaStages; ++s) { mbar_init(&S->kv_full[s], 128); mbar_init(&S->kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&S->s_full[b], 1); mbar_init(&S->p_full[b], 256); mbar_init(&S->o_full[b], 1); mbar_init(&S->mx_full[b], 256);
    }
    mbar_init(&S->l_full, 256);
    S->failed = 0u;
    fence_mbar_init();
  }
  if (w == 4) {
    __syncwarp();
    tmem_alloc(&S->tmem_base, kFaCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = S->tmem_base;

  // blocks of 128 query rows, aligned inside a head, that intersect [tile_lo, rows_end)
  const int64_t nblk = (T + 127) / 128;
  const int64_t first = static_cast<int64_t>(tile_lo), last = rows_end - 1;
  const int64_t b_lo = (first / T) * nblk + (first % T) / 128, b_hi = (last / T) * nblk + (last % T) / 128;
  uint32_t kvit = 0, jt = 0, qn = 0;     // ring positions, carried across blocks by every role

  for (int64_t blk = b_lo; blk <= b_hi; ++blk) {
    const int64_t g = blk / nblk, m0 = (blk % nblk) * 128;
    const int64_t rows_q = min(static_cast<int64_t>(128), T - m0);
    // keys any row of the block may see
    const int64_t c_max = causal ? min(C, m0 + rows_q - 1 + (C - T) + 1) : C;
    const int64_t nkb = (c_max + 127) / 128;

    if (w < 4) {
      // ---------------- producers (128 threads) ----------------
      const uint32_t ptid = L.tid;
      {   // Q block, K-major: row (query) at 128 B pitch, chunks XORed with row % 8
        const uint32_t c = ptid & 7u, r = ptid >> 3;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int64_t row = r + 16 * i;
          const bool okr = row < rows_q;
          cp_async_16_zfill(q_s + static_cast<uint32_t>(row) * 128u + ((c ^ (static_cast<uint32_t>(row) & 7u)) << 4),
                            okr ? Q + ((g * T + m0 + row) * hd + 8 * c) : Q, okr ? 16u : 0u);
        }
        cp_async_mbar_arrive(&S->q_full);
      }
      for (int64_t j = 0; j < nkb; ++j) {
        const uint32_t kvpos = kvit + static_cast<uint32_t>(j), s = kvpos % kFaStages;
        if (!tc_wait_warp(&S->kv_empty[s], ((kvpos / kFaStages) & 1u) ^ 1u, failed, budget, 64u)) break;
        const uint32_t ks = kv_s + s * kFaKvBytes, vs = ks + 128 * 128;
        const int64_t n0 = j * 128;
        {   // K^T block: element (d, key) at KT[(g*hd + d)*C + key]: keys are the unit-stride ("MN") dimension
          const uint32_t cm = ptid & 15u, dr = ptid >> 4;            // 16 key chunks x 8 d lines per pass
          const int64_t key = n0 + 8 * cm;
          const uint32_t kbytes = key < C ? static_cast<uint32_t>(min(static_cast<int64_t>(16), 2 * (C - key))) : 0u;
#pragma unroll
          for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t d = dr + 8u * i;
            const uint32_t dst = ks + (cm >> 3) * 8192u + (d >> 3) * 1024u + (d & 7u) * 128u + (((cm & 7u) ^ (d & 7u)) << 4);
            cp_async_16_zfill(dst, kbytes ? KT + ((g * hd + d) * C + key) : KT, kbytes);
          }
        }
        {   // V block: element (key, d) at V[(g*C + key)*hd + d]: d is the unit-stride ("MN") dimension, keys are k
          const uint32_t cd = ptid & 7u, kr = ptid >> 3;             // 8 d chunks x 16 keys per pass
#pragma unroll
          for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t kk = kr + 16u * i;
            const int64_t key = n0 + kk;
            const uint32_t dst = vs + (kk >> 3) * 1024u + (kk & 7u) * 128u + ((cd ^ (kk & 7u)) << 4);
            cp_async_16_zfill(dst, key < C ? V + ((g * C + key) * hd + 8 * cd) : V, key < C ? 16u : 0u);
          }
        }
        cp_async_mbar_arrive(&S->kv_full[s]);
      }
      cp_async_wait_all();
    } else if (w == 4) {
      // ---------------- MMA issue ----------------
      if (lane == 0) {
        const uint32_t fmt = adt == kBF16 ? 1u : 0u;
        // S: A = Q K-major, B = K^T MN-major, N = 128.  O: A = P K-major, B = V MN-major, N = 64.
        const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
        bool ok = tc_wait(&S->q_full, qn & 1u, failed, budget);
        auto issue_s = [&](uint32_t jj, uint32_t kvpos) {   // S(jj) into buffer jj % 2 from ring stage kvpos
          const uint32_t s = kvpos % kFaStages;
          if (!tc_wait(&S->kv_full[s], (kvpos / kFaStages) & 1u, failed, budget)) { ok = false; return; }
          fence_proxy_async_smem();
          tc_fence_after_sync();
          const uint64_t da = tc_desc(q_s, 16u, 1024u);
          const uint64_t db = tc_desc(kv_s + s * kFaKvBytes, 8192u, 1024u);
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk)
            tc_mma_f16(tmem + (jj & 1u) * 128u, da + kk * (32u >> 4), db + kk * (2048u >> 4), idesc_s, kk ? 1u : 0u);
          tc_commit(&S->s_full[jj & 1u]);
        };
        if (ok && nkb > 0) issue_s(jt, kvit);
        for (int64_t j = 0; ok && j < nkb; ++j) {
          const uint32_t jj = jt + static_cast<uint32_t>(j), kvpos = kvit + static_cast<uint32_t>(j);
          if (j + 1 < nkb) issue_s(jj + 1, kvpos + 1);
          if (!ok) break;
          if (!tc_wait(&S->p_full[jj & 1u], (jj >> 1) & 1u, failed, budget)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t s = kvpos % kFaStages;
          const uint32_t pb = p_s + (jj & 1u) * kFaPBytes;
          const uint64_t dv = tc_desc(kv_s + s * kFaKvBytes + 128 * 128, 16384u, 1024u);
#pragma unroll
          for (uint32_t kk = 0; kk < 8; ++kk) {
            const uint64_t dp = tc_desc(pb + (kk >> 2) * 16384u + (kk & 3u) * 32u, 16u, 1024u);
            tc_mma_f16(tmem + 256u + (jj & 1u) * 64u, dp, dv + kk * (2048u >> 4), idesc_o, kk ? 1u : 0u);
          }
          tc_commit(&S->kv_empty[s]);
          tc_commit(&S->o_full[jj & 1u]);
        }
      }
      __syncwarp();
    } else if (w >= 8) {
      // ---------------- softmax + output: two threads per query row ----------------
      const uint32_t q4 = w & 3u, hf = (w - 8u) >> 2, r = 32u * q4 + lane;
      float *xch = reinterpret_cast<float *>(sm + kSmemChain);          // [2 parities][2 halves][128 rows], then [2][128] sums
      const int64_t m = m0 + r, grow = g * T + m;
      const bool row_ok = m < T && grow >= first && grow < rows_end;
      const int64_t c_end = causal ? min(C, m + (C - T) + 1) : C;   // keys this row may see
      float m_run = -INFINITY, l_run = 0.0f;
      float acc[32];                                                  // output columns 32 hf .. 32 hf + 31
#pragma unroll
      for (int d = 0; d < 32; ++d) acc[d] = 0.0f;
      bool ok = true;
      for (int64_t j = 0; ok && j <= nkb; ++j) {
        const uint32_t jj = jt + static_cast<uint32_t>(j);
        float alpha = 1.0f;
        if (j < nkb) {
          if (!tc_wait_warp(&S->s_full[jj & 1u], (jj >> 1) & 1u, failed, budget)) { ok = false; break; }
          tc_fence_after_sync();
          // valid columns of this thread's half (keys n0 + 64 hf .. + lim - 1)
          const int lim = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(64), c_end - j * 128 - 64 * hf)));
          const uint32_t s_addr = tmem + ((32u * q4) << 16) + (jj & 1u) * 128u + 64u * hf;
          // pass 1: the half row's maximum over this block, then the row's through shared memory
          float mx = -INFINITY;
#pragma unroll 1
          for (int cb = 0; cb < 64; cb += 32) {
            uint32_t raw[32];
            __syncwarp();
            tc_ld32(s_addr + cb, raw);
            tc_wait_ld();
            if (cb + 32 <= lim) {
#pragma unroll
              for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(raw[i]) * sl2);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (cb + i < lim) mx = fmaxf(mx, __uint_as_float(raw[i]) * sl2);
            }
          }
          xch[((jj & 1u) * 2u + hf) * 128u + r] = mx;
          mbar_arrive(&S->mx_full[jj & 1u]);
          if (!tc_wait_warp(&S->mx_full[jj & 1u], (jj >> 1) & 1u, failed, budget)) { ok = false; break; }
          mx = fmaxf(mx, xch[((jj & 1u) * 2u + (hf ^ 1u)) * 128u + r]);
          const float m_new = fmaxf(m_run, mx);
          alpha = m_run == -INFINITY ? (m_new == -INFINITY ? 1.0f : 0.0f) : fast_ex2(m_run - m_new);
          const float neg_m = m_new == -INFINITY ? 0.0f : -m_new;
          // pass 2: p = 2^(s - m_new), written as the 16-bit A operand of the second matmul
          float psum = 0.0f;
          const uint32_t prow = p_s + (jj & 1u) * kFaPBytes + hf * 16384u + r * 128u;   // 64 keys = one sub-tile
          const bool bf = adt == kBF16;
#pragma unroll 1
          for (int cb = 0; cb < 64; cb += 16) {
            uint32_t raw[16];
            __syncwarp();
            tc_ld16(s_addr + cb, raw);
            tc_wait_ld();
            float pv[16];
            if (cb + 16 <= lim) {
#pragma unroll
              for (int i = 0; i < 16; ++i) pv[i] = fast_ex2(fmaf(__uint_as_float(raw[i]), sl2, neg_m));
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) pv[i] = cb + i < lim ? fast_ex2(fmaf(__uint_as_float(raw[i]), sl2, neg_m)) : 0.0f;
            }
            uint32_t pk[8];
            if (bf) {
#pragma unroll
              for (int i = 0; i < 8; ++i) pk[i] = cvt_bf16x2(pv[2 * i + 1], pv[2 * i]);
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) pk[i] = f32_to_f16_bits(pv[2 * i]) | (f32_to_f16_bits(pv[2 * i + 1]) << 16);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) psum += pv[i];
#pragma unroll
            for (uint32_t q = 0; q < 2; ++q) {                      // 16 keys = 2 chunks of 8
              const uint32_t ch = (static_cast<uint32_t>(cb) >> 3) + q;
              uint4 *dstp = reinterpret_cast<uint4 *>(sm + (prow + ((ch ^ (r & 7u)) << 4) - smem_addr(sm)));
              *dstp = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            }
          }
          l_run = l_run * alpha + psum;
          m_run = m_new;
          tc_fence_before_sync();
          fence_proxy_async_smem();               // P (generic-proxy stores) -> the MMA's reads
          mbar_arrive(&S->p_full[jj & 1u]);
        }
        if (j > 0) {
          // fold O(j-1) in: acc = (acc + O(j-1)) * alpha(j)
          const uint32_t pj = jj - 1u;
          if (!tc_wait_warp(&S->o_full[pj & 1u], (pj >> 1) & 1u, failed, budget)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t raw[32];
          __syncwarp();
          tc_ld32(tmem + ((32u * q4) << 16) + 256u + (pj & 1u) * 64u + 32u * hf, raw);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = (acc[i] + __uint_as_float(raw[i])) * alpha;
        } else {
#pragma unroll
          for (int d = 0; d < 32; ++d) acc[d] *= alpha;
        }
      }
      // the row's sum is the two halves' (they share the running maximum)
      float *lx = xch + 512;
      lx[hf * 128u + r] = l_run;
      mbar_arrive(&S->l_full);
      if (ok && !tc_wait_warp(&S->l_full, qn & 1u, failed, budget)) ok = false;
      if (ok && row_ok) {
        const float inv = 1.0f / (l_run + lx[(hf ^ 1u) * 128u + r]);
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = acc[i] * inv;
        tc_store_row32(out, dt, grow * hd + 32 * hf, v, 32, true);
      }
    }
    kvit += static_cast<uint32_t>(nkb);
    jt += static_cast<uint32_t>(nkb);
    ++qn;
    // Every role is done with the block: Q, the rings and tensor memory are free again.
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (S->failed) break;
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (w == 4) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, kFaCols);
  }
  if (L.tid == 0) {
    if (S->failed) set_status(P, kStTensorTimeout, L.lane, tile_lo, kTopFlashAttn);
    mbar_inval(&S->q_full);
    for (int s = 0; s < kFaStages; ++s) { mbar_inval(&S->kv_full[s]); mbar_inval(&S->kv_empty[s]); }
    for (int b = 0; b < 2; ++b) {
      mbar_inval(&S->s_full[b]); mbar_inval(&S->p_full[b]); mbar_inval(&S->o_full[b]); mbar_inval(&S->mx_full[b]);
    }
    mbar_inval(&S->l_full);
  }
  __syncthreads();
  return true;
}

#else

__device__ __forceinline__ bool flash_tc_tiles(const Lane &, const DTask &, uint32_t, uint32_t) { return false; }

#endif

}  // namespace b2
#endif
