// The persistent megakernel: one CTA per scheduler lane interprets its lane's
// entry stream - tile entries, scheduler-placed global barriers, and the
// WHILE / IF / FOR frame stack - exactly as the reference's `vm2` does
// (pjrt_plugin/kernels/vm_main.cl:107-258; control semantics mirrored by
// python/pjrt_ocl/vmreader.py:655-773).
//
// Differences from the reference that the bytecode cannot see:
//  - the grid barrier is one release-add plus an acquire-polled generation word
//    (vm_common.cl:284-300 uses the same two words), every wait is bounded: when
//    the budget runs out the lane records {code, lane, barrier index}, raises an
//    abort flag all other waits poll, and every lane leaves the kernel normally;
//  - consecutive lane-local elementwise entries run as one fused pass (ops_ew.cuh);
//  - frame-stack overflow and unknown tile ops set a status instead of corrupting state.
#include <cuda_runtime.h>

// This file is compiled once per entry of variants.h, with
//   -DB2_VARIANT=<name> -DB2_FAMILIES=<mask>
// and then holds only the tile-op families in the mask. The kernel and its launch
// glue carry the variant's name; the runtime picks the build per program.
#ifndef B2_FAMILIES
#define B2_FAMILIES 0xFFFFFFFFu
#define B2_VARIANT all
#endif
#define B2_HAS(fam) (((B2_FAMILIES) & (fam)) != 0u)
#define B2_PASTE2(a, b) a##b
#define B2_PASTE(a, b) B2_PASTE2(a, b)

#include <cstring>
#define B2_SHORT B2_HAS(0x100u)   // kFamShort
#include "dev_common.cuh"
#include "ops_ew.cuh"
#include "ops_ew_steps.cuh"
#if B2_HAS(0x20u)   // kFamMma
#include "ops_mma.cuh"
#include "ops_mma_tc.cuh"
#endif
#if B2_HAS(0x40u)   // kFamFlash
#include "ops_flash_tc.cuh"
#include "ops_flash.cuh"
#endif
#if B2_HAS(0x02u)   // kFamMove
#include "ops_move.cuh"
#endif
#if B2_HAS(0x04u)   // kFamRed
#include "ops_reduce.cuh"
#endif
#if B2_HAS(0x10u)   // kFamRegion
#include "ops_region.cuh"
#endif
#if B2_HAS(0x08u)   // kFamRows
#include "ops_rows.cuh"
#endif
#if B2_HAS(0x80u)   // kFamIndex
#include "ops_index.cuh"
#endif

namespace b2 {
static_assert(kFamMove == 0x02u && kFamRed == 0x04u && kFamRows == 0x08u && kFamRegion == 0x10u && kFamMma == 0x20u &&
              kFamFlash == 0x40u && kFamIndex == 0x80u && kFamShort == 0x100u, "the literals in the #if lines above");

constexpr int kVmThreads = 512;   // threads per lane: the one instantiation the library carries
struct Frame { uint32_t pc, end, widx, phase; };  // phase: 0 while-cond, 1 while-body, 2 if, FOR: trips left
constexpr uint32_t kRoot = 0xFFFFFFFFu;

// Grid-wide barrier over the n_lanes co-resident CTAs. Returns false when the
// wait was abandoned (budget exhausted here or abort raised by another lane).
// `gen` is the generation this lane expects (thread 0's copy, read once at kernel
// entry: every lane passes every barrier, so it advances by one per call).
// Ordering: the CTA barrier makes the lane's stores visible to thread 0, whose
// acq_rel arrival publishes them (release is cumulative); the last arriver's release
// on `gen` and the waiters' acquire loads of it carry them to every other lane, and
// the closing CTA barrier to that lane's other threads.
__device__ __forceinline__ bool grid_barrier(const Lane &L, uint32_t barrier_index, unsigned long long t_start, uint32_t &gen) {
  const KParams &P = *L.P;
  volatile uint32_t &ok_flag = *reinterpret_cast<volatile uint32_t *>(L.smem + kSmemFlag);
  __syncthreads();
  if (L.tid == 0) {
    bool ok = true;
    DSync *s = P.sync;
    if (P.lane_ts && barrier_index < kPhaseSlots) P.lane_ts[L.lane * kLaneTsSlots + 2u + barrier_index] = globaltimer_ns();
    const uint32_t prev = atom_add_acq_rel_gpu(&s->arrive, 1u);
    if (prev == P.n_lanes - 1u) {
      st_relaxed_gpu(&s->arrive, 0u);
      red_release_gpu_add(&s->gen, 1u);
      if (ld_relaxed_gpu(&s->abort)) ok = false;
    } else {
      const unsigned long long t0 = globaltimer_ns();
      uint32_t spins = 0;
      for (;;) {
        const unsigned long long v = ld_acquire_gpu_u64(&s->gen);      // {gen, abort}
        if (static_cast<uint32_t>(v >> 32)) { ok = false; break; }
        if (static_cast<uint32_t>(v) != gen) break;
        if (++spins > 32u) {
          nanosleep_ns(64);
          if ((spins & 255u) == 0u && globaltimer_ns() - t0 > P.wait_budget_ns) {
            set_status(P, kStBarrierTimeout, L.lane, barrier_index, 0u);
            ok = false;
            break;
          }
        }
      }
    }
    ++gen;
    // when the phase ended for everybody: the barrier's release as lane 0 sees it
    if (L.lane == 0 && barrier_index < kPhaseSlots) s->phase_ns[barrier_index] = globaltimer_ns() - t_start;
    ok_flag = ok ? 1u : 0u;
  }
  __syncthreads();
  return ok_flag != 0u;
}

template <int NT>
__device__ __forceinline__ void exec_entry(const Lane &L, const DEntry &en) {
  const KParams &P = *L.P;
  const DTask &t = P.tasks[en.task];
  switch (t.op) {
#if B2_HAS(0x20u)
    case kTopMma: {
      const DMma &dm = *reinterpret_cast<const DMma *>(P.desc + t.desc);
      const bool tc = NT == 512 && B2_HAS_TC && (dm.tc_mode & kTcOk) && mma_tc_tiles(L, t, en.tile_lo, en.tile_hi);
      if (!tc) mma_simt_tiles<NT>(L, t, en.tile_lo, en.tile_hi);
      break;
    }
#endif
#if B2_HAS(0x02u)
    case kTopGather: case kTopDynGather: move_tiles(L, t, en.tile_lo, en.tile_hi, false); break;
    case kTopScatter: case kTopDynScatter: move_tiles(L, t, en.tile_lo, en.tile_hi, true); break;
    case kTopIotaDim: iota_tiles(L, t, en.tile_lo, en.tile_hi); break;
#endif
#if B2_HAS(0x04u)
    case kTopRedPart: red_part_tiles(L, t, en.tile_lo, en.tile_hi, en.a, en.b); break;
    case kTopRedComb: red_comb_tiles(L, t, en.tile_lo, en.tile_hi); break;
    case kTopRedSeg: red_seg_tiles(L, t, en.tile_lo, en.tile_hi); break;
    case kTopRedStrided: red_strided_tiles(L, t, en.tile_lo, en.tile_hi, en.a, en.b); break;
#endif
#if B2_HAS(0x08u)
    case kTopSoftmaxSeg: rows_tiles(L, t, en.tile_lo, en.tile_hi, true); break;
    case kTopLayernormSeg: rows_tiles(L, t, en.tile_lo, en.tile_hi, false); break;
    case kTopRmsRows: rms_rows_tiles(L, t, en.tile_lo, en.tile_hi); break;
#endif
#if B2_HAS(0x10u)
    case kTopMapRegion: region_tiles(L, t, en.tile_lo, en.tile_hi); break;
#endif
#if B2_HAS(0x40u)
    case kTopFlashAttn: {
      const DFlash &df = *reinterpret_cast<const DFlash *>(P.desc + t.desc);
      const bool tc = NT == 512 && B2_HAS_TC && df.tc_mode && flash_tc_tiles(L, t, en.tile_lo, en.tile_hi);
      if (!tc) flash_simt_tiles(L, t, en.tile_lo, en.tile_hi);
      break;
    }
#endif
#if B2_HAS(0x80u)
    case kTopRedWindow: red_window_tiles(L, t, en.tile_lo, en.tile_hi); break;
    case kTopGatherIndex: indexed_tiles(L, t, en.tile_lo, en.tile_hi, false); break;
    case kTopScatterIndex: indexed_tiles(L, t, en.tile_lo, en.tile_hi, true); break;
    case kTopConv: conv_tiles(L, t, en.tile_lo, en.tile_hi); break;
#endif
    default:   // a tile op this build does not hold (the host picks the build, so: a host bug) or an unknown one
      if (L.tid == 0) set_status(P, kStBadOp, L.lane, en.task, t.op);
      break;
  }
}

#define B2_VM_KERNEL B2_PASTE(b2_vm_, B2_VARIANT)
template <int NT>
__global__ void __launch_bounds__(NT, 1) B2_VM_KERNEL(const __grid_constant__ KParams P, const uint32_t smem_bytes) {
  B2_DYN_SMEM(smem);
  Lane L;
  L.P = &P;
  L.smem = smem;
  L.smem_bytes = smem_bytes;
  L.lane = blockIdx.x;
  L.tid = threadIdx.x;
  L.nthr = NT;
  const VmLane span = P.lanes[L.lane];
  const DEntry *stream = P.entries + span.off;
  const unsigned long long t_start = globaltimer_ns();
  if (P.lane_ts && L.tid == 0) P.lane_ts[L.lane * kLaneTsSlots] = t_start;

  Frame st[kMaxDepth + 1];
  int sp = 0;
  st[0].pc = 0; st[0].end = span.root_len; st[0].widx = kRoot; st[0].phase = 0;
  uint32_t barrier_i = 0;
  uint32_t gen = L.tid == 0 ? ld_relaxed_gpu(&P.sync->gen) : 0u;   // thread 0's copy of the barrier generation
  bool pub = false;   // a tile entry ran since the last barrier (vm_main.cl:82-100)
  bool alive = true;

  while (alive) {
    Frame &f = st[sp];
    if (f.pc >= f.end) {
      if (f.widx == kRoot) break;
      const DEntry w = stream[f.widx];
      if (w.task == kEntIf) {                    // branch done: no closing barrier
        sp--;
        st[sp].pc++;
        continue;
      }
      alive = grid_barrier(L, barrier_i++, t_start, gen);
      pub = false;
      if (!alive) break;
      if (w.task == kEntFor) {                   // one iteration done
        if (--f.phase != 0u) { f.pc = w.tile_lo; f.end = w.tile_lo + w.tile_hi; }
        else { sp--; st[sp].pc++; }
      } else if (f.phase == 0u) {                // while-cond range done: read the flag
        const uint32_t cbits = ld_relaxed_gpu(reinterpret_cast<const uint32_t *>(resolve(P, w.cond)));
        if (cbits != 0u) { f.pc = w.a; f.end = w.a + w.b; f.phase = 1u; }
        else { sp--; st[sp].pc++; }
      } else {                                   // while-body done: re-run the cond range
        f.pc = w.tile_lo; f.end = w.tile_lo + w.tile_hi; f.phase = 0u;
      }
      continue;
    }
    const uint32_t epc = f.pc;
    const DEntry en = stream[epc];
    if (en.task == kEntBarrier) {
      alive = grid_barrier(L, barrier_i++, t_start, gen);
      pub = false;
      f.pc++;
      continue;
    }
    if (en.task == kEntWhile || en.task == kEntFor || en.task == kEntIf) {
      uint32_t start, len, phase;
      if (en.task == kEntWhile) {
        start = en.tile_lo; len = en.tile_hi; phase = 0u;
      } else if (en.task == kEntFor) {
        if (en.a == 0u) { f.pc++; continue; }    // trip 0: skip the loop
        start = en.tile_lo; len = en.tile_hi; phase = en.a;
      } else {
        const uint32_t cbits = ld_relaxed_gpu(reinterpret_cast<const uint32_t *>(resolve(P, en.cond)));
        start = cbits ? en.tile_lo : en.a;
        len = cbits ? en.tile_hi : en.b;
        phase = 2u;
        if (len == 0u) { f.pc++; continue; }
      }
      if (sp + 1 > kMaxDepth) {
        if (L.tid == 0) set_status(P, kStStackOverflow, L.lane, epc, 0u);
        break;
      }
      sp++;
      st[sp].pc = start; st[sp].end = start + len; st[sp].widx = epc; st[sp].phase = phase;
      continue;
    }
    if (en.task != kEntNop) {
      // Publish the previous tile entry's stores to the whole lane: consecutive
      // entries map elements to threads differently.
      if (pub) { __threadfence_block(); __syncthreads(); }
      pub = true;
      const uint32_t chain = en.chain > 1u ? en.chain : 1u;
      if (P.tasks[en.task].op == kTopEw) {
        ew_entries(L, stream + epc, chain);
        f.pc += chain;
        continue;
      }
      exec_entry<NT>(L, en);
    }
    f.pc++;
  }
  if (P.lane_ts && L.tid == 0) P.lane_ts[L.lane * kLaneTsSlots + 1u] = globaltimer_ns();
  if (L.lane == 0 && L.tid == 0) {
    P.sync->barriers = barrier_i;
    P.sync->device_ns = globaltimer_ns() - t_start;
  }
}

// ---- host-side launch glue (called from runtime.cc through the table in variants.h) ----
cudaError_t B2_PASTE(LaunchVm_, B2_VARIANT)(const KParams &params, uint32_t n_lanes, int threads, uint32_t smem_bytes,
                                            cudaStream_t stream, const void *keep_base, size_t keep_bytes) {
  void *args[2] = {const_cast<KParams *>(&params), &smem_bytes};
  if (threads != kVmThreads) return cudaErrorInvalidValue;
  const void *fn = reinterpret_cast<const void *>(&B2_VM_KERNEL<kVmThreads>);
  cudaLaunchAttribute attr[2];
  std::memset(attr, 0, sizeof(attr));
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  unsigned n_attr = 1;
  if (keep_base && keep_bytes) {        // the program's tables stay in the L2 set-aside between the phases
    attr[1].id = cudaLaunchAttributeAccessPolicyWindow;
    attr[1].val.accessPolicyWindow.base_ptr = const_cast<void *>(keep_base);
    attr[1].val.accessPolicyWindow.num_bytes = keep_bytes;
    attr[1].val.accessPolicyWindow.hitRatio = 1.0f;
    attr[1].val.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
    attr[1].val.accessPolicyWindow.missProp = cudaAccessPropertyNormal;
    n_attr = 2;
  }
  // {grid, block, dynamic shared memory, stream, attributes, their count}
  cudaLaunchConfig_t cfg = {dim3(n_lanes), dim3(static_cast<unsigned>(threads)), smem_bytes, stream, attr, n_attr};
  return cudaLaunchKernelExC(&cfg, fn, args);
}

// Co-resident CTAs of this build at `threads` per lane and `smem_bytes` of dynamic shared memory.
cudaError_t B2_PASTE(VmResidency_, B2_VARIANT)(int device, int threads, uint32_t smem_bytes, int *max_lanes) {
  if (threads != kVmThreads) return cudaErrorInvalidValue;
  const void *fn = reinterpret_cast<const void *>(&B2_VM_KERNEL<kVmThreads>);
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes));
  if (e != cudaSuccess) return e;
  int per_sm = 0, sms = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, smem_bytes);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return e;
  *max_lanes = per_sm * sms;
  return cudaSuccess;
}

}  // namespace b2
