// CUDA runtime side of the backend and its C ABI (include/b2vm.h).
//
// Mirrors, for the execution path only, the reference's OclRuntime and
// LoadedProgram (pjrt_plugin/src/runtime.h:120-435; runtime.cc:255-662 Create,
// :735-1074 Load, :1103-1218 Execute/LaunchKernel, :2107-2277 ExecuteDevice and
// the buffer pool): one device, one stream, one mutex per runtime; an arena per
// loaded program with constants uploaded once; <= 64 zero-copy I/O ports;
// synchronous execute; size-keyed pool for result buffers.
#include <cuda_runtime.h>
#include <cuda.h>   // CUtensorMap types only; the encoder is reached through the runtime's driver entry point

#include <cstdarg>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/b2vm.h"
#include "format.h"
#include "loader.h"
#include "variants.h"
#include "vmprog.h"

namespace b2 {
// One pair of launch glue per build of the megakernel (vm_kernel.cu, variants.h).
#define B2_DECLARE_VARIANT(name, fams)                                                                              \
  cudaError_t LaunchVm_##name(const KParams &params, uint32_t n_lanes, int threads, uint32_t smem_bytes,           \
                              cudaStream_t stream, const void *keep_base, size_t keep_bytes);                     \
  cudaError_t VmResidency_##name(int device, int threads, uint32_t smem_bytes, int *max_lanes);
B2_VARIANT_LIST(B2_DECLARE_VARIANT)
#undef B2_DECLARE_VARIANT

struct VmVariant {
  const char *name;
  uint32_t families;
  cudaError_t (*launch)(const KParams &, uint32_t, int, uint32_t, cudaStream_t, const void *, size_t);
  cudaError_t (*residency)(int, int, uint32_t, int *);
};
#define B2_VARIANT_ROW(name, fams) {#name, static_cast<uint32_t>(fams), &LaunchVm_##name, &VmResidency_##name},
const VmVariant kVariants[] = {B2_VARIANT_LIST(B2_VARIANT_ROW)};
#undef B2_VARIANT_ROW
constexpr int kNumVariants = static_cast<int>(sizeof(kVariants) / sizeof(kVariants[0]));
}  // namespace b2

namespace {

void SetErr(char *err, size_t cap, const std::string &m) {
  if (err && cap) {
    std::snprintf(err, cap, "%s", m.c_str());
  }
}
std::string CudaMsg(const char *what, cudaError_t e) {
  return std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
}

constexpr size_t kPoolPerSize = 4;  // runtime.h:304

// Encode one TMA tensor map (loader.h: TmapSpec) at operand address `base`: 16-bit
// elements, 128-byte swizzle, elements beyond the tensor's edge read as zero. Returns
// false when the tensor cannot be described (the task then loads with per-thread
// copies, or falls back to its CUDA-core path).
bool EncodeTmap(const b2::TmapSpec &s, const void *base, b2::DTmap *out) {
  if (!s.valid || reinterpret_cast<uintptr_t>(base) % 16) return false;
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1u, 1u, 1u, 1u};
  for (uint32_t k = 0; k < s.rank; ++k) { dims[k] = s.dims[k]; box[k] = s.box[k]; }
  for (uint32_t k = 0; k + 1 < s.rank; ++k) {
    if (s.strides[k] <= 0) return false;
    strides[k] = static_cast<cuuint64_t>(s.strides[k]) * 2;
    if (strides[k] % 16 || strides[k] >= (1ull << 40)) return false;
  }
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode) return false;
  static_assert(sizeof(CUtensorMap) == sizeof(b2::DTmap), "tensor map size");
  const CUresult r = encode(reinterpret_cast<CUtensorMap *>(out),
                            s.dtype == b2::kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, s.rank,
                            const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

struct b2_program {
  b2::VmProgram prog;
};

struct b2_runtime {
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaDeviceProp prop{};
  int threads = 512;
  uint32_t smem_bytes = 0;
  int max_lanes = 0;
  size_t l2_keep_bytes = 0;   // L2 set aside for persisting lines (the loaded programs' tables), 0 = unavailable
  std::mutex mu;        // serialises execute and host<->device copies (runtime.h:301)
  std::mutex pool_mu;   // runtime.h:302
  std::unordered_map<size_t, std::vector<void *>> pool;

  cudaError_t Bind() const { return cudaSetDevice(device); }

  void *PoolAlloc(size_t bytes, std::string *err) {
    const size_t key = bytes ? bytes : 8;
    {
      std::lock_guard<std::mutex> g(pool_mu);
      auto it = pool.find(key);
      if (it != pool.end() && !it->second.empty()) {
        void *p = it->second.back();
        it->second.pop_back();
        return p;
      }
    }
    void *p = nullptr;
    const cudaError_t e = cudaMalloc(&p, key);
    if (e != cudaSuccess) {
      *err = CudaMsg("device allocation", e) + " for " + std::to_string(key) + " bytes";
      cudaGetLastError();
      return nullptr;
    }
    return p;
  }
  void PoolFree(void *p, size_t bytes) {
    if (!p) return;
    const size_t key = bytes ? bytes : 8;
    {
      std::lock_guard<std::mutex> g(pool_mu);
      auto &v = pool[key];
      if (v.size() < kPoolPerSize) {
        v.push_back(p);
        return;
      }
    }
    cudaFree(p);
  }
};

struct b2_loaded {
  b2_runtime *rt = nullptr;
  b2::VmProgram prog;
  b2::DeviceTables tab;
  uint8_t *arena = nullptr;
  uint8_t *d_tables = nullptr;   // one allocation holding the tensor maps, tasks, entries, lane table, aux and descriptor pools
  size_t tables_bytes = 0;
  b2::DTask *d_tasks = nullptr;
  b2::DEntry *d_entries = nullptr;
  b2::VmLane *d_lanes = nullptr;
  int32_t *d_aux = nullptr;
  uint64_t *d_desc = nullptr;
  b2::DTmap *d_tmaps = nullptr;          // tensor maps of the tensor-core matmul operands
  std::vector<b2::DTmap> h_tmaps;
  std::vector<const void *> tmap_base;   // the operand address each map was encoded for
  std::vector<char> tmap_off;            // the owning matmul could not be described at load: per-thread copies instead
  b2::DSync *d_sync = nullptr;
  b2::DSync *h_sync = nullptr;  // pinned mirror
  unsigned long long *d_lane_ts = nullptr;   // per-lane timing buffer (b2_loaded_lane_timing), else null
  uint8_t *d_scratch = nullptr; // lane totals of re-cut full reductions (RedScratch), when the program has one
  size_t scratch_bytes = 0;
  int variant = b2::kNumVariants - 1;   // which build of the megakernel runs this program
  uint64_t launches = 0;
  bool sync_dirty = true;       // the device sync block must be cleared before the next launch
  uint64_t wait_budget_ns = 2000000000ull;
  cudaStream_t last_stream = nullptr;

  ~b2_loaded() {
    if (rt) rt->Bind();
    cudaFree(arena); cudaFree(d_tables);      // the tables are carved out of d_tables
    cudaFree(d_sync); cudaFree(d_scratch); cudaFree(d_lane_ts);
    if (h_sync) cudaFreeHost(h_sync);
  }
};

namespace {

// The device tables of a loaded program live in ONE allocation, each table at a 256-byte boundary: every
// launch names that range as an L2 persistence window, so that the few KB a lane reads at the start of each
// phase (entry, task, descriptors: a chain of dependent loads) are not evicted by the gigabytes the phases
// stream through the cache in between.
size_t TableBytes(size_t n) { return (std::max<size_t>(n, 16) + 255) & ~static_cast<size_t>(255); }
template <typename T>
cudaError_t Carve(uint8_t *pool, size_t *off, T **dptr, const std::vector<T> &v) {
  *dptr = reinterpret_cast<T *>(pool + *off);
  *off += TableBytes(v.size() * sizeof(T));
  return v.empty() ? cudaSuccess : cudaMemcpy(*dptr, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
}

// Enqueue one execution on `stream`: reset the sync block, launch the megakernel,
// copy the sync block back to its pinned mirror. `io` holds the port addresses.
b2_status Enqueue(b2_loaded *lp, const b2::IoTable &io, cudaStream_t stream, std::string *err) {
  // The barrier words return to their rest state after every complete run and
  // the status words are only written on failure, so the block is cleared only
  // at first use and after a failed run.
  cudaError_t e = cudaSuccess;
  if (lp->sync_dirty) {
    if (lp->d_scratch) cudaMemsetAsync(lp->d_scratch, 0, lp->scratch_bytes, stream);   // an aborted run may leave arrivals
    e = cudaMemsetAsync(lp->d_sync, 0, sizeof(b2::DSync), stream);
    if (e != cudaSuccess) { *err = CudaMsg("sync reset", e); return B2_INTERNAL; }
    lp->sync_dirty = false;
  }
  // Tensor maps carry the operand's address: the ones over I/O ports follow the
  // addresses bound for this launch.
  for (size_t i = 0; i < lp->tab.tmaps.size(); ++i) {
    const b2::TmapSpec &sp = lp->tab.tmaps[i];
    if (!(sp.base & b2::kPortBit) || lp->tmap_off[i]) continue;   // fixed address, or the task loads without tensor maps
    const uint8_t *base = static_cast<const uint8_t *>(io.p[sp.base & (b2::kMaxIoPorts - 1)]) + sp.off * 2;
    if (base == lp->tmap_base[i]) continue;
    if (!EncodeTmap(sp, base, &lp->h_tmaps[i])) {
      *err = "matmul operand bound at an address the tensor map cannot describe (needs 16-byte alignment)";
      return B2_INVALID_ARGUMENT;
    }
    lp->tmap_base[i] = base;
    e = cudaMemcpyAsync(lp->d_tmaps + i, &lp->h_tmaps[i], sizeof(b2::DTmap), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) { *err = CudaMsg("tensor map upload", e); return B2_INTERNAL; }
  }
  b2::KParams kp;
  std::memset(&kp, 0, sizeof(kp));
  kp.tmaps = lp->d_tmaps;
  kp.tasks = lp->d_tasks;
  kp.entries = lp->d_entries;
  kp.lanes = lp->d_lanes;
  kp.aux = lp->d_aux;
  kp.desc = lp->d_desc;
  kp.sync = lp->d_sync;
  kp.scratch = lp->d_scratch;
  kp.lane_ts = lp->d_lane_ts;
  kp.n_lanes = lp->prog.n_lanes;
  kp.wait_budget_ns = lp->wait_budget_ns;
  kp.io = io;
  e = b2::kVariants[lp->variant].launch(kp, lp->prog.n_lanes, lp->rt->threads, lp->rt->smem_bytes, stream, lp->d_tables,
                                        std::min(lp->tables_bytes, lp->rt->l2_keep_bytes));
  if (e != cudaSuccess) {          // whatever was queued before the failure may have run: start clean next time
    *err = CudaMsg("megakernel launch", e);
    cudaGetLastError();
    lp->sync_dirty = true;
    return B2_INTERNAL;
  }
  lp->launches++;
  lp->last_stream = stream;
  return B2_OK;
}

// Enqueue the copy of the device sync block to its pinned mirror.
b2_status FetchStatus(b2_loaded *lp, cudaStream_t stream, std::string *err) {
  const cudaError_t e = cudaMemcpyAsync(lp->h_sync, lp->d_sync, sizeof(b2::DSync), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) { *err = CudaMsg("status readback", e); return B2_INTERNAL; }
  return B2_OK;
}

b2_status CheckDeviceStatus(b2_loaded *lp, std::string *err) {
  const b2::DSync &s = *lp->h_sync;
  if (s.status[0] != b2::kStOk) lp->sync_dirty = true;
  switch (s.status[0]) {
    case b2::kStOk: return B2_OK;
    case b2::kStBarrierTimeout:
      *err = "device wait ran out: lane " + std::to_string(s.status[1]) + " at grid barrier " +
             std::to_string(s.status[2]) + " (are all " + std::to_string(lp->prog.n_lanes) + " lanes co-resident?)";
      return B2_DEADLINE_EXCEEDED;
    case b2::kStTensorTimeout:
      *err = "device wait ran out: lane " + std::to_string(s.status[1]) + " asynchronous copy / tensor-core wait in tile op " +
             std::to_string(s.status[3]);
      return B2_DEADLINE_EXCEEDED;
    case b2::kStStackOverflow:
      *err = "control nesting exceeds " + std::to_string(b2::kMaxDepth) + " on lane " + std::to_string(s.status[1]);
      return B2_INVALID_ARGUMENT;
    case b2::kStBadOp:
      *err = "tile op " + std::to_string(s.status[3]) + " reached on device but not implemented";
      return B2_UNIMPLEMENTED;
    default:
      *err = "unknown device status " + std::to_string(s.status[0]);
      return B2_INTERNAL;
  }
}

}  // namespace

extern "C" {

b2_status b2_runtime_create(int device_ordinal, b2_runtime **out, char *err, size_t err_cap) {
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    SetErr(err, err_cap, e != cudaSuccess ? CudaMsg("no CUDA device", e) : "no CUDA device");
    cudaGetLastError();
    return B2_FAILED_PRECONDITION;
  }
  if (device_ordinal < 0 || device_ordinal >= n) {
    SetErr(err, err_cap, "device ordinal " + std::to_string(device_ordinal) + " out of range (" + std::to_string(n) + " devices)");
    return B2_INVALID_ARGUMENT;
  }
  auto rt = std::make_unique<b2_runtime>();
  rt->device = device_ordinal;
  if ((e = rt->Bind()) != cudaSuccess || (e = cudaGetDeviceProperties(&rt->prop, device_ordinal)) != cudaSuccess) {
    SetErr(err, err_cap, CudaMsg("device query", e));
    return B2_INTERNAL;
  }
  if (rt->prop.major < 10) {
    SetErr(err, err_cap, std::string("device ") + rt->prop.name + " is sm_" + std::to_string(rt->prop.major) +
                             std::to_string(rt->prop.minor) + "; this backend is built for sm_100a only");
    return B2_FAILED_PRECONDITION;
  }
  // All of the opt-in shared memory of one CTA per SM, minus a margin for the
  // runtime's own reservation.
  size_t optin = rt->prop.sharedMemPerBlockOptin;
  rt->smem_bytes = static_cast<uint32_t>(std::min<size_t>(optin, 227 * 1024) - 1024);
  // every build of the megakernel must be launchable with the same lane count
  rt->max_lanes = 1 << 30;
  for (const b2::VmVariant &v : b2::kVariants) {
    int lanes = 0;
    if ((e = v.residency(device_ordinal, rt->threads, rt->smem_bytes, &lanes)) != cudaSuccess) {
      SetErr(err, err_cap, CudaMsg("megakernel occupancy query", e) + " (build '" + v.name + "')");
      cudaGetLastError();
      return B2_INTERNAL;
    }
    rt->max_lanes = std::min(rt->max_lanes, lanes);
  }
  // A few MB of L2 for lines marked persisting (context-scoped; released with the context). Failure only means
  // the tables compete for L2 like everything else.
  {
    const size_t want = std::min<size_t>(static_cast<size_t>(std::max(rt->prop.persistingL2CacheMaxSize, 0)), 4u << 20);
    if (want && !std::getenv("B2VM_NO_L2_KEEP") && cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, want) == cudaSuccess)
      rt->l2_keep_bytes = std::min<size_t>(want, static_cast<size_t>(std::max(rt->prop.accessPolicyMaxWindowSize, 0)));
    cudaGetLastError();
  }
  if ((e = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking)) != cudaSuccess) {
    SetErr(err, err_cap, CudaMsg("stream create", e));
    return B2_INTERNAL;
  }
  *out = rt.release();
  return B2_OK;
}

void b2_runtime_destroy(b2_runtime *rt) {
  if (!rt) return;
  rt->Bind();
  for (auto &kv : rt->pool)
    for (void *p : kv.second) cudaFree(p);
  if (rt->stream) cudaStreamDestroy(rt->stream);
  delete rt;
}

b2_status b2_runtime_info(const b2_runtime *rt, b2_device_info *out) {
  if (!rt || !out) return B2_INVALID_ARGUMENT;
  std::memset(out, 0, sizeof(*out));
  std::snprintf(out->device_name, sizeof(out->device_name), "%s", rt->prop.name);
  out->device_ordinal = rt->device;
  out->sm_count = rt->prop.multiProcessorCount;
  out->cc_major = rt->prop.major;
  out->cc_minor = rt->prop.minor;
  out->total_mem_bytes = rt->prop.totalGlobalMem;
  out->lanes = static_cast<uint32_t>(rt->max_lanes);
  out->ew_ts = b2::kEwTs;
  out->mma_t = b2::kMmaT;
  out->threads_per_lane = static_cast<uint32_t>(rt->threads);
  return B2_OK;
}

b2_status b2_alloc(b2_runtime *rt, size_t bytes, void **dev_ptr, char *err, size_t err_cap) {
  if (!rt || !dev_ptr) return B2_INVALID_ARGUMENT;
  rt->Bind();
  std::string m;
  *dev_ptr = rt->PoolAlloc(bytes, &m);
  if (!*dev_ptr) { SetErr(err, err_cap, m); return B2_RESOURCE_EXHAUSTED; }
  return B2_OK;
}

b2_status b2_free(b2_runtime *rt, void *dev_ptr, size_t bytes) {
  if (!rt) return B2_INVALID_ARGUMENT;
  rt->Bind();
  rt->PoolFree(dev_ptr, bytes);
  return B2_OK;
}

b2_status b2_h2d(b2_runtime *rt, void *dev_dst, const void *host_src, size_t bytes, char *err, size_t err_cap) {
  if (!rt) return B2_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(rt->mu);
  rt->Bind();
  cudaError_t e = cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, rt->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
  if (e != cudaSuccess) { SetErr(err, err_cap, CudaMsg("host to device copy", e)); return B2_INTERNAL; }
  return B2_OK;
}

b2_status b2_d2h(b2_runtime *rt, void *host_dst, const void *dev_src, size_t bytes, char *err, size_t err_cap) {
  if (!rt) return B2_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(rt->mu);
  rt->Bind();
  cudaError_t e = cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, rt->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
  if (e != cudaSuccess) { SetErr(err, err_cap, CudaMsg("device to host copy", e)); return B2_INTERNAL; }
  return B2_OK;
}

// ---- program ------------------------------------------------------------------------
b2_status b2_program_parse(const uint8_t *blob, size_t len, b2_program **out, char *err, size_t err_cap) {
  if (!out) return B2_INVALID_ARGUMENT;
  *out = nullptr;
  auto p = std::make_unique<b2_program>();
  std::string m;
  if (!blob || !b2::VmProgram::Parse(blob, len, &p->prog, &m)) {
    SetErr(err, err_cap, blob ? m : "null blob");
    return B2_INVALID_ARGUMENT;
  }
  *out = p.release();
  return B2_OK;
}
void b2_program_destroy(b2_program *prog) { delete prog; }
uint32_t b2_program_num_inputs(const b2_program *p) { return static_cast<uint32_t>(p->prog.args.ids.size()); }
uint32_t b2_program_num_outputs(const b2_program *p) { return static_cast<uint32_t>(p->prog.results.ids.size()); }
uint32_t b2_program_num_lanes(const b2_program *p) { return p->prog.n_lanes; }
uint32_t b2_program_num_tasks(const b2_program *p) { return static_cast<uint32_t>(p->prog.tasks.size()); }
uint64_t b2_program_arena_bytes(const b2_program *p) { return p->prog.arena_bytes; }
static const b2::BufferSlot *IoBuf(const b2_program *p, int is_output, uint32_t i) {
  const auto &ids = is_output ? p->prog.results.ids : p->prog.args.ids;
  return i < ids.size() ? &p->prog.buffers[ids[i]] : nullptr;
}
uint64_t b2_program_io_bytes(const b2_program *p, int is_output, uint32_t i) {
  const b2::BufferSlot *b = IoBuf(p, is_output, i);
  return b ? b->bytes : 0;
}
uint32_t b2_program_io_dtype(const b2_program *p, int is_output, uint32_t i) {
  const b2::BufferSlot *b = IoBuf(p, is_output, i);
  return b ? b->dtype : 0;
}
uint32_t b2_program_io_rank(const b2_program *p, int is_output, uint32_t i) {
  const auto &d = is_output ? p->prog.results.dims : p->prog.args.dims;
  return i < d.size() ? static_cast<uint32_t>(d[i].size()) : 0;
}
int64_t b2_program_io_dim(const b2_program *p, int is_output, uint32_t i, uint32_t k) {
  const auto &d = is_output ? p->prog.results.dims : p->prog.args.dims;
  return (i < d.size() && k < d[i].size()) ? d[i][k] : 0;
}

// ---- load ---------------------------------------------------------------------------------
b2_status b2_program_load(b2_runtime *rt, b2_program *prog, b2_loaded **out, char *err, size_t err_cap) {
  if (!rt || !prog || !out) return B2_INVALID_ARGUMENT;
  *out = nullptr;
  const b2::VmProgram &p = prog->prog;
  rt->Bind();
  // The grid barrier needs every lane resident at once: refuse rather than launch.
  if (static_cast<int>(p.n_lanes) > rt->max_lanes) {
    SetErr(err, err_cap, "program is scheduled for " + std::to_string(p.n_lanes) + " lanes but only " +
                             std::to_string(rt->max_lanes) + " megakernel CTAs are co-resident on " + rt->prop.name);
    return B2_FAILED_PRECONDITION;
  }
  auto lp = std::make_unique<b2_loaded>();
  lp->rt = rt;
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&lp->arena), std::max<uint64_t>(p.arena_bytes, 256));
  if (e != cudaSuccess) {
    SetErr(err, err_cap, CudaMsg("arena allocation", e) + " for " + std::to_string(p.arena_bytes) + " bytes");
    cudaGetLastError();
    return B2_RESOURCE_EXHAUSTED;
  }
  std::string m;
  bool unimpl = false;
  if (!b2::BuildDeviceTables(p, reinterpret_cast<uint64_t>(lp->arena), &lp->tab, &m, &unimpl)) {
    SetErr(err, err_cap, "load: " + m);
    return unimpl ? B2_UNIMPLEMENTED : B2_INVALID_ARGUMENT;
  }
  // The smallest build of the megakernel that holds every tile-op family the program uses.
  for (int v = 0; v < b2::kNumVariants; ++v)
    if ((lp->tab.families & ~b2::kVariants[v].families) == 0u) { lp->variant = v; break; }
  if (const char *force = std::getenv("B2VM_VARIANT")) {   // measurement aid: run on a named (larger) build
    for (int v = 0; v < b2::kNumVariants; ++v)
      if (!std::strcmp(force, b2::kVariants[v].name) && (lp->tab.families & ~b2::kVariants[v].families) == 0u) lp->variant = v;
  }
  // Tensor maps of the tensor-core matmul operands. Arena operands are final here;
  // port operands get a placeholder (the arena) and are re-encoded at bind. A task
  // whose operand cannot be described keeps the per-thread copy path.
  lp->h_tmaps.resize(lp->tab.tmaps.size());
  lp->tmap_base.assign(lp->tab.tmaps.size(), nullptr);
  lp->tmap_off.assign(lp->tab.tmaps.size(), 0);
  for (size_t i = 0; i < lp->tab.tmaps.size();) {
    const size_t group = lp->tab.tmaps[i].owner_is_flash ? 3 : 2;   // Q K V, or A B
    bool ok = i + group <= lp->tab.tmaps.size();
    for (size_t j = i; ok && j < i + group; ++j) {
      const b2::TmapSpec &sp = lp->tab.tmaps[j];
      const bool port = (sp.base & b2::kPortBit) != 0;
      const uint8_t *base = port ? lp->arena : reinterpret_cast<const uint8_t *>(static_cast<uintptr_t>(sp.base)) + sp.off * 2;
      ok = ok && EncodeTmap(sp, base, &lp->h_tmaps[j]);
      lp->tmap_base[j] = port ? nullptr : base;
    }
    if (!ok) {
      // the task keeps its other path: per-thread copies (matmul) or the CUDA-core kernel (attention)
      uint64_t *dw = &lp->tab.desc[lp->tab.tmaps[i].desc_word];
      if (lp->tab.tmaps[i].owner_is_flash) {
        b2::DFlash *f = reinterpret_cast<b2::DFlash *>(dw);
        f->tmap = -1;
        f->tc_mode = 0;
      } else {
        reinterpret_cast<b2::DMma *>(dw)->tmap = -1;
      }
      for (size_t j = i; j < std::min(i + group, lp->tab.tmaps.size()); ++j) lp->tmap_off[j] = 1;
    }
    i += group;
  }
  std::vector<int32_t> aux = p.aux;
  lp->tables_bytes = TableBytes(lp->h_tmaps.size() * sizeof(lp->h_tmaps[0])) + TableBytes(lp->tab.tasks.size() * sizeof(lp->tab.tasks[0])) +
                     TableBytes(lp->tab.entries.size() * sizeof(lp->tab.entries[0])) + TableBytes(lp->tab.lanes.size() * sizeof(lp->tab.lanes[0])) +
                     TableBytes(aux.size() * sizeof(aux[0])) + TableBytes(lp->tab.desc.size() * sizeof(lp->tab.desc[0]));
  size_t toff = 0;
  if ((e = cudaMalloc(reinterpret_cast<void **>(&lp->d_tables), lp->tables_bytes)) != cudaSuccess ||
      (e = Carve(lp->d_tables, &toff, &lp->d_tmaps, lp->h_tmaps)) != cudaSuccess || (e = Carve(lp->d_tables, &toff, &lp->d_tasks, lp->tab.tasks)) != cudaSuccess ||
      (e = Carve(lp->d_tables, &toff, &lp->d_entries, lp->tab.entries)) != cudaSuccess ||
      (e = Carve(lp->d_tables, &toff, &lp->d_lanes, lp->tab.lanes)) != cudaSuccess || (e = Carve(lp->d_tables, &toff, &lp->d_aux, aux)) != cudaSuccess ||
      (e = Carve(lp->d_tables, &toff, &lp->d_desc, lp->tab.desc)) != cudaSuccess ||
      (e = cudaMalloc(reinterpret_cast<void **>(&lp->d_sync), sizeof(b2::DSync))) != cudaSuccess ||
      (e = cudaMallocHost(reinterpret_cast<void **>(&lp->h_sync), sizeof(b2::DSync))) != cudaSuccess) {
    SetErr(err, err_cap, CudaMsg("device table upload", e));
    cudaGetLastError();
    return B2_RESOURCE_EXHAUSTED;
  }
  std::memset(lp->h_sync, 0, sizeof(b2::DSync));
  if (lp->tab.needs_scratch) {
    lp->scratch_bytes = sizeof(b2::RedScratch) + sizeof(unsigned long long) * 2u * p.n_lanes;   // zero = rest state of every counter
    if ((e = cudaMalloc(reinterpret_cast<void **>(&lp->d_scratch), lp->scratch_bytes)) != cudaSuccess ||
        (e = cudaMemset(lp->d_scratch, 0, lp->scratch_bytes)) != cudaSuccess) {
      SetErr(err, err_cap, CudaMsg("reduction scratch allocation", e));
      cudaGetLastError();
      return B2_RESOURCE_EXHAUSTED;
    }
  }
  for (const auto &k : p.consts) {  // constants are uploaded once (runtime.cc:1064-1072)
    if (k.data.empty()) continue;
    e = cudaMemcpy(lp->arena + p.buffers[k.buffer].offset, k.data.data(), k.data.size(), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { SetErr(err, err_cap, CudaMsg("constant upload", e)); return B2_INTERNAL; }
  }
  lp->prog = std::move(prog->prog);
  delete prog;
  *out = lp.release();
  return B2_OK;
}

void b2_loaded_destroy(b2_loaded *lp) { delete lp; }

const b2_program *b2_loaded_program(const b2_loaded *lp) {
  // b2_program is a thin wrapper around VmProgram: same address.
  static_assert(offsetof(b2_program, prog) == 0, "wrapper layout");
  return reinterpret_cast<const b2_program *>(&lp->prog);
}

uint64_t b2_loaded_launch_count(const b2_loaded *lp) { return lp->launches; }
int b2_loaded_in_out_result(const b2_loaded *lp, uint32_t input) {
  return lp && input < lp->tab.inout_result.size() ? lp->tab.inout_result[input] : -1;
}
uint64_t b2_loaded_stat(const b2_loaded *lp, int which) {
  if (!lp) return 0;
  switch (which) {
    case 0: return lp->tab.n_chains;
    case 1: return lp->tab.n_forwarded;
    case 2: return lp->tab.n_dead_stores;
    case 3: return lp->tab.n_mma;
    case 4: return lp->tab.n_mma_tc;
    case 5: return lp->tab.mma_flops;
    case 6: return lp->tab.n_flash;
    case 7: return lp->tab.n_flash_tc;
    case 8: return lp->tab.n_spread;
    case 9: return static_cast<uint64_t>(lp->variant);
    case 11: return lp->tab.n_fused_reduce;
    case 10: return lp->tab.families;
    case 12: return lp->tab.n_flash_decode;
    case 14: return lp->tab.n_rebalanced;
    case 15: return lp->tab.n_row_pipelines;
    case 16: return lp->tab.n_folded_converts;
    case 17: return lp->tab.n_carried_sums;
    case 18: return lp->tab.n_carried_barriers_removed;
    case 19: return lp->tab.n_rms_rows;
    case 20: return lp->tab.n_empty_phases_dropped;
    case 13: return static_cast<uint64_t>(std::count_if(lp->tab.inout_result.begin(), lp->tab.inout_result.end(), [](int o) { return o >= 0; }));
    default: return 0;
  }
}
void b2_loaded_set_wait_budget_ns(b2_loaded *lp, uint64_t ns) { lp->wait_budget_ns = ns; }
size_t b2_loaded_phase_ns(const b2_loaded *lp, uint64_t *out, size_t cap) {
  if (!lp || !out) return 0;
  std::lock_guard<std::mutex> g(lp->rt->mu);
  size_t n = std::min<size_t>(std::min<size_t>(lp->h_sync->barriers, b2::kPhaseSlots), cap);
  for (size_t i = 0; i < n; ++i) out[i] = lp->h_sync->phase_ns[i];
  return n;
}

b2_status b2_loaded_lane_timing(b2_loaded *lp, int on, char *err, size_t err_cap) {
  if (!lp) return B2_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(lp->rt->mu);
  lp->rt->Bind();
  if (!on) {
    if (lp->last_stream) cudaStreamSynchronize(lp->last_stream);
    cudaFree(lp->d_lane_ts);
    lp->d_lane_ts = nullptr;
    return B2_OK;
  }
  if (lp->d_lane_ts) return B2_OK;
  const size_t bytes = sizeof(unsigned long long) * b2::kLaneTsSlots * lp->prog.n_lanes;
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&lp->d_lane_ts), bytes);
  if (e == cudaSuccess) e = cudaMemset(lp->d_lane_ts, 0, bytes);
  if (e != cudaSuccess) {
    SetErr(err, err_cap, CudaMsg("lane timing buffer", e));
    cudaGetLastError();
    return B2_RESOURCE_EXHAUSTED;
  }
  return B2_OK;
}

size_t b2_loaded_lane_times(b2_loaded *lp, uint64_t *out, size_t cap) {
  if (!lp || !out || !lp->d_lane_ts) return 0;
  std::lock_guard<std::mutex> g(lp->rt->mu);
  lp->rt->Bind();
  const size_t n = std::min<size_t>(cap, static_cast<size_t>(b2::kLaneTsSlots) * lp->prog.n_lanes);
  cudaStream_t stream = lp->last_stream ? lp->last_stream : lp->rt->stream;
  if (cudaStreamSynchronize(stream) != cudaSuccess ||
      cudaMemcpy(out, lp->d_lane_ts, n * sizeof(uint64_t), cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

b2_status b2_loaded_status(b2_loaded *lp, b2_exec_status *out, char *err, size_t err_cap) {
  if (!lp || !out) return B2_INVALID_ARGUMENT;
  std::string m;
  {
    std::lock_guard<std::mutex> g(lp->rt->mu);
    lp->rt->Bind();
    cudaStream_t stream = lp->last_stream ? lp->last_stream : lp->rt->stream;
    b2_status fs = FetchStatus(lp, stream, &m);
    if (fs == B2_OK && cudaStreamSynchronize(stream) != cudaSuccess) {
      m = "status readback: stream synchronize failed";
      cudaGetLastError();
      fs = B2_INTERNAL;
    }
    if (fs != B2_OK) { SetErr(err, err_cap, m); return fs; }
  }
  const b2::DSync &s = *lp->h_sync;
  out->code = s.status[0]; out->lane = s.status[1]; out->where = s.status[2]; out->detail = s.status[3];
  out->barriers = s.barriers; out->device_ns = s.device_ns;
  const b2_status st = CheckDeviceStatus(lp, &m);
  if (st != B2_OK) SetErr(err, err_cap, m);
  return st;
}

// ---- execute ---------------------------------------------------------------------------------
static b2_status BindAndRun(b2_loaded *lp, void *const *dev_in, void *const *dev_out, cudaStream_t stream,
                            bool synchronous, std::string *err) {
  const b2::VmProgram &p = lp->prog;
  b2::IoTable io;
  std::memset(&io, 0, sizeof(io));
  cudaError_t e;
  for (size_t i = 0; i < p.args.ids.size(); ++i) {
    const auto &b = p.buffers[p.args.ids[i]];
    if (!b.bytes) continue;
    if (lp->tab.input_port[i] >= 0) {
      if (reinterpret_cast<uintptr_t>(dev_in[i]) % 16) { *err = "argument " + std::to_string(i) + " is not 16-byte aligned"; return B2_INVALID_ARGUMENT; }
      io.p[lp->tab.input_port[i]] = dev_in[i];
      // an in/out buffer: the kernel updates the result's memory (bound below), which starts as the argument
      const int o = lp->tab.inout_result[i];
      if (o >= 0 && dev_out[o] != dev_in[i] &&
          (e = cudaMemcpyAsync(dev_out[o], dev_in[i], b.bytes, cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) {
        *err = CudaMsg("in/out argument copy into its result", e);
        return B2_INTERNAL;
      }
    } else if ((e = cudaMemcpyAsync(lp->arena + b.offset, dev_in[i], b.bytes, cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) {
      *err = CudaMsg("argument copy into the arena", e);
      return B2_INTERNAL;
    }
  }
  for (size_t o = 0; o < p.results.ids.size(); ++o) {
    if (lp->tab.output_port[o] < 0 || !p.buffers[p.results.ids[o]].bytes) continue;
    if (reinterpret_cast<uintptr_t>(dev_out[o]) % 16) { *err = "result " + std::to_string(o) + " is not 16-byte aligned"; return B2_INVALID_ARGUMENT; }
    io.p[lp->tab.output_port[o]] = dev_out[o];
  }
  const b2_status st = Enqueue(lp, io, stream, err);
  if (st != B2_OK) { lp->sync_dirty = true; return st; }
  for (size_t o = 0; o < p.results.ids.size(); ++o) {
    const auto &b = p.buffers[p.results.ids[o]];
    if (lp->tab.output_port[o] >= 0 || !b.bytes) continue;
    if ((e = cudaMemcpyAsync(dev_out[o], lp->arena + b.offset, b.bytes, cudaMemcpyDeviceToDevice, stream)) != cudaSuccess) {
      *err = CudaMsg("result copy out of the arena", e);
      lp->sync_dirty = true;
      return B2_INTERNAL;
    }
  }
  if (!synchronous) return B2_OK;
  if (FetchStatus(lp, stream, err) != B2_OK) { lp->sync_dirty = true; return B2_INTERNAL; }
  if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) {
    *err = CudaMsg("execute", e);
    cudaGetLastError();
    lp->sync_dirty = true;
    return B2_INTERNAL;
  }
  return CheckDeviceStatus(lp, err);
}

b2_status b2_execute_device_async(b2_loaded *lp, void *const *dev_inputs, size_t n_inputs, void *const *dev_outputs,
                                  size_t n_outputs, void *cuda_stream, char *err, size_t err_cap) {
  if (!lp) return B2_INVALID_ARGUMENT;
  const b2::VmProgram &p = lp->prog;
  if (n_inputs != p.args.ids.size() || n_outputs != p.results.ids.size()) {
    SetErr(err, err_cap, "execute: got " + std::to_string(n_inputs) + " args / " + std::to_string(n_outputs) +
                             " results, want " + std::to_string(p.args.ids.size()) + " / " + std::to_string(p.results.ids.size()));
    return B2_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> g(lp->rt->mu);
  lp->rt->Bind();
  std::string m;
  const b2_status st = BindAndRun(lp, dev_inputs, dev_outputs,
                                  cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : lp->rt->stream, false, &m);
  if (st != B2_OK) SetErr(err, err_cap, m);
  return st;
}

b2_status b2_execute_device(b2_loaded *lp, void *const *dev_inputs, size_t n_inputs, void **dev_outputs,
                            size_t n_outputs, char *err, size_t err_cap) {
  if (!lp) return B2_INVALID_ARGUMENT;
  const b2::VmProgram &p = lp->prog;
  if (n_inputs != p.args.ids.size() || n_outputs != p.results.ids.size()) {
    SetErr(err, err_cap, "execute: got " + std::to_string(n_inputs) + " args / " + std::to_string(n_outputs) +
                             " results, want " + std::to_string(p.args.ids.size()) + " / " + std::to_string(p.results.ids.size()));
    return B2_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> g(lp->rt->mu);
  lp->rt->Bind();
  std::string m;
  for (size_t o = 0; o < n_outputs; ++o) dev_outputs[o] = nullptr;
  for (size_t o = 0; o < n_outputs; ++o) {
    dev_outputs[o] = lp->rt->PoolAlloc(p.buffers[p.results.ids[o]].bytes, &m);
    if (!dev_outputs[o]) {
      for (size_t k = 0; k < o; ++k) lp->rt->PoolFree(dev_outputs[k], p.buffers[p.results.ids[k]].bytes);
      SetErr(err, err_cap, m);
      return B2_RESOURCE_EXHAUSTED;
    }
  }
  const b2_status st = BindAndRun(lp, dev_inputs, dev_outputs, lp->rt->stream, true, &m);
  if (st != B2_OK) {
    for (size_t o = 0; o < n_outputs; ++o) {
      lp->rt->PoolFree(dev_outputs[o], p.buffers[p.results.ids[o]].bytes);
      dev_outputs[o] = nullptr;
    }
    SetErr(err, err_cap, m);
  }
  return st;
}

b2_status b2_execute_host(b2_loaded *lp, const void *const *inputs, size_t n_inputs, void *const *outputs,
                          size_t n_outputs, char *err, size_t err_cap) {
  if (!lp) return B2_INVALID_ARGUMENT;
  const b2::VmProgram &p = lp->prog;
  if (n_inputs != p.args.ids.size() || n_outputs != p.results.ids.size()) {
    SetErr(err, err_cap, "Execute: got " + std::to_string(n_inputs) + " args, want " + std::to_string(p.args.ids.size()));
    return B2_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> g(lp->rt->mu);
  b2_runtime *rt = lp->rt;
  rt->Bind();
  std::string m;
  std::vector<void *> din(n_inputs, nullptr), dout(n_outputs, nullptr);
  auto cleanup = [&] {
    for (size_t i = 0; i < n_inputs; ++i) rt->PoolFree(din[i], p.buffers[p.args.ids[i]].bytes);
    for (size_t o = 0; o < n_outputs; ++o) rt->PoolFree(dout[o], p.buffers[p.results.ids[o]].bytes);
  };
  b2_status st = B2_OK;
  cudaError_t e = cudaSuccess;
  for (size_t i = 0; i < n_inputs && st == B2_OK; ++i) {
    const size_t bytes = p.buffers[p.args.ids[i]].bytes;
    din[i] = rt->PoolAlloc(bytes, &m);
    if (!din[i]) { st = B2_RESOURCE_EXHAUSTED; break; }
    if (bytes && (e = cudaMemcpyAsync(din[i], inputs[i], bytes, cudaMemcpyHostToDevice, rt->stream)) != cudaSuccess) {
      m = CudaMsg("Execute: input write", e);
      st = B2_INTERNAL;
    }
  }
  for (size_t o = 0; o < n_outputs && st == B2_OK; ++o) {
    dout[o] = rt->PoolAlloc(p.buffers[p.results.ids[o]].bytes, &m);
    if (!dout[o]) st = B2_RESOURCE_EXHAUSTED;
  }
  if (st == B2_OK) st = BindAndRun(lp, din.data(), dout.data(), rt->stream, false, &m);
  if (st == B2_OK) st = FetchStatus(lp, rt->stream, &m);
  for (size_t o = 0; o < n_outputs && st == B2_OK; ++o) {
    const size_t bytes = p.buffers[p.results.ids[o]].bytes;
    if (bytes && (e = cudaMemcpyAsync(outputs[o], dout[o], bytes, cudaMemcpyDeviceToHost, rt->stream)) != cudaSuccess) {
      m = CudaMsg("Execute: output read", e);
      st = B2_INTERNAL;
    }
  }
  if (st == B2_OK) {
    if ((e = cudaStreamSynchronize(rt->stream)) != cudaSuccess) {
      m = CudaMsg("Execute", e);
      cudaGetLastError();
      st = B2_INTERNAL;
    } else {
      st = CheckDeviceStatus(lp, &m);
    }
  } else {
    cudaStreamSynchronize(rt->stream);
  }
  cleanup();
  if (st != B2_OK) SetErr(err, err_cap, m);
  return st;
}

}  // extern "C"
