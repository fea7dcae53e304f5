// b2_sum_f32_static: the full f32 sum (the RED_PART + RED_COMB pair of a
// program, pjrt_plugin/kernels/ops/reduce.cl:90-153,529-549) as one standalone
// launch that allocates nothing.
//
// Who needs it: a host whose device memory is owned by somebody else. A serving
// process that hands all of HBM to its own allocator at start-up leaves nothing
// for a later cudaMalloc to take, so loading a program (which allocates an arena
// and device tables) fails there with out-of-memory; and a caller on a latency
// path cannot afford cudaMalloc / cudaFree, which stall every stream of the
// device while they run. Such callers still own an input and an output buffer;
// what they cannot supply is the reduction's scratch (the per-chunk partial sums
// and the arrival counter). Here that scratch lives in a fixed array inside the
// library image itself, so the entry point needs no allocation at all.
//
// The price, stated once:
//  - the array is part of the library: every GPU that loads libb2vm.so holds its
//    kScratchBytes (about 16.3 KB) until the process exits, used or not;
//  - its size bounds the input: at most kMaxParts chunks of kChunk elements
//    (536 870 912 floats, 2 GiB); larger inputs are refused with a message;
//  - there is ONE array per GPU, shared by every call and keeping the previous
//    call's partial sums. The arrival counter is cleared on the stream before each
//    launch and every partial that is read was written by the same launch, so
//    calls one after another are independent; two calls running on the same GPU
//    at the same time (two streams, two threads) would overwrite each other's
//    partials and race. The entry point waits for its own launch to finish
//    before it returns, which keeps one thread's calls apart; callers on several
//    threads serialise among themselves.
//
// The array's name is only meaningful to device code. On the host it is a
// stand-in object: its address there is not a device address, so the host asks
// the CUDA runtime for the real one (cudaGetSymbolAddress) once per GPU, with
// that GPU current, and passes the returned pointer to the kernel. That lookup
// happens in the first call on each GPU; make that first call before any stream
// capture is begun.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "../../include/b2vm.h"

namespace {

constexpr uint32_t kChunk = 131072;    // elements per partial sum: the chunk of a full-sum program (python/pjrt_ocl/ops/reduce.py:81-91)
constexpr uint32_t kMaxParts = 4096;   // partial sums the scratch holds
constexpr uint64_t kMaxElems = static_cast<uint64_t>(kChunk) * kMaxParts;
constexpr int kThreads = 512;
constexpr int kMaxDevices = 64;

struct SumScratch {
  float partial[kMaxParts];
  unsigned int arrived;                // blocks that have stored their partials in this launch
  unsigned int pad[63];
};
constexpr size_t kScratchBytes = sizeof(SumScratch);

// The scratch itself. Host code must never pass `g_sum_scratch` to a kernel:
// see SumScratchAddress below.
static __device__ __align__(256) unsigned char g_sum_scratch[kScratchBytes];

__device__ __forceinline__ float WarpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum over the block; every thread returns the total. `red` = 32 floats of shared memory.
__device__ __forceinline__ float BlockSum(float v, float *red) {
  v = WarpSum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = l < (kThreads >> 5) ? red[l] : 0.0f;
  return WarpSum(r);
}

// Block b sums chunks b, b + gridDim.x, ... into scratch->partial[chunk]; the block
// that arrives last folds partial[0, n_parts) in index order and stores the total.
__global__ void __launch_bounds__(kThreads) b2_static_sum_f32(const float *__restrict__ in, unsigned long long n,
                                                              float *__restrict__ out, SumScratch *scratch,
                                                              unsigned int n_parts) {
  __shared__ float red[32];
  __shared__ unsigned int last;
  const bool vec = (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
  for (unsigned int part = blockIdx.x; part < n_parts; part += gridDim.x) {
    const unsigned long long lo = static_cast<unsigned long long>(part) * kChunk;
    const unsigned long long hi = lo + kChunk < n ? lo + kChunk : n;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    unsigned long long done = lo;
    if (vec) {   // lo is a multiple of 4 elements: 16-byte loads, four independent chains per thread
      const float4 *q = reinterpret_cast<const float4 *>(in + lo);
      const unsigned int groups = static_cast<unsigned int>((hi - lo) >> 2);
      unsigned int g = threadIdx.x;
      for (; g + 3u * kThreads < groups; g += 4u * kThreads) {
        const float4 a = q[g], b = q[g + kThreads], c = q[g + 2 * kThreads], d = q[g + 3 * kThreads];
        acc[0] += (a.x + a.y) + (a.z + a.w);
        acc[1] += (b.x + b.y) + (b.z + b.w);
        acc[2] += (c.x + c.y) + (c.z + c.w);
        acc[3] += (d.x + d.y) + (d.z + d.w);
      }
      for (; g < groups; g += kThreads) {
        const float4 a = q[g];
        acc[0] += (a.x + a.y) + (a.z + a.w);
      }
      done = lo + (static_cast<unsigned long long>(groups) << 2);
    }
    for (unsigned long long i = done + threadIdx.x; i < hi; i += kThreads) acc[0] += in[i];
    const float s = BlockSum((acc[0] + acc[1]) + (acc[2] + acc[3]), red);
    if (threadIdx.x == 0) scratch->partial[part] = s;
  }
  // publish this block's partials, then count it in
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&scratch->arrived, 1u) == gridDim.x - 1u ? 1u : 0u;
  __syncthreads();
  if (!last) return;
  __threadfence();   // the other blocks' partials are visible from here on
  float t = 0.0f;
  for (unsigned int p = threadIdx.x; p < n_parts; p += kThreads) t += __ldcg(&scratch->partial[p]);
  t = BlockSum(t, red);
  if (threadIdx.x == 0) {
    out[0] = t;
    scratch->arrived = 0u;   // rest state for the next call (the host clears it as well)
  }
}

// Device address of g_sum_scratch on `device`, looked up once per GPU with that
// GPU current. Returns nullptr and fills *why on failure.
SumScratch *SumScratchAddress(int device, std::string *why) {
  static std::mutex mu;
  static SumScratch *addr[kMaxDevices] = {};
  std::lock_guard<std::mutex> g(mu);
  if (addr[device]) return addr[device];
  void *p = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&p, g_sum_scratch);
  if (e != cudaSuccess || !p) {
    *why = std::string("scratch address lookup: ") + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    cudaGetLastError();
    return nullptr;
  }
  addr[device] = static_cast<SumScratch *>(p);
  return addr[device];
}

void SetMsg(char *err, size_t cap, const std::string &m) {
  if (err && cap) std::snprintf(err, cap, "%s", m.c_str());
}

}  // namespace

extern "C" {

uint64_t b2_sum_f32_static_max_elems(void) { return kMaxElems; }

b2_status b2_sum_f32_static(int device_ordinal, const void *dev_in, uint64_t n_elems, void *dev_out,
                            void *cuda_stream, char *err, size_t err_cap) {
  if (!dev_out || (!dev_in && n_elems)) {
    SetMsg(err, err_cap, "b2_sum_f32_static: null buffer");
    return B2_INVALID_ARGUMENT;
  }
  if (n_elems > kMaxElems) {
    SetMsg(err, err_cap, "b2_sum_f32_static: " + std::to_string(n_elems) + " elements exceed the " +
                             std::to_string(kMaxElems) + " the built-in scratch (" + std::to_string(kMaxParts) +
                             " partial sums of " + std::to_string(kChunk) + " elements) can hold");
    return B2_INVALID_ARGUMENT;
  }
  if (reinterpret_cast<uintptr_t>(dev_in) % 4 || reinterpret_cast<uintptr_t>(dev_out) % 4) {
    SetMsg(err, err_cap, "b2_sum_f32_static: buffers must be 4-byte aligned");
    return B2_INVALID_ARGUMENT;
  }
  if (device_ordinal < 0 || device_ordinal >= kMaxDevices) {
    SetMsg(err, err_cap, "b2_sum_f32_static: device ordinal out of range");
    return B2_INVALID_ARGUMENT;
  }
  int prev = -1;
  cudaError_t e = cudaGetDevice(&prev);
  if (e == cudaSuccess && prev != device_ordinal) e = cudaSetDevice(device_ordinal);
  if (e != cudaSuccess) {
    SetMsg(err, err_cap, std::string("b2_sum_f32_static: selecting the device: ") + cudaGetErrorString(e));
    cudaGetLastError();
    return B2_FAILED_PRECONDITION;
  }
  b2_status st = B2_OK;
  std::string why;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  SumScratch *scratch = SumScratchAddress(device_ordinal, &why);
  if (!scratch) {
    st = B2_INTERNAL;
  } else {
    const unsigned int n_parts = static_cast<unsigned int>((n_elems + kChunk - 1) / kChunk);
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_ordinal);
    // the arrival counter must start at zero whatever an earlier, failed launch left behind
    if (e == cudaSuccess) e = cudaMemsetAsync(&scratch->arrived, 0, sizeof(unsigned int), stream);
    if (e == cudaSuccess) {
      unsigned int blocks = n_parts < static_cast<unsigned int>(2 * sms) ? n_parts : static_cast<unsigned int>(2 * sms);
      if (blocks == 0) blocks = 1;   // n = 0: the fold of no partials stores 0
      b2_static_sum_f32<<<blocks, kThreads, 0, stream>>>(static_cast<const float *>(dev_in), n_elems,
                                                         static_cast<float *>(dev_out), scratch, n_parts);
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) {
      why = std::string("b2_sum_f32_static: ") + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
      cudaGetLastError();
      st = B2_INTERNAL;
    }
  }
  if (prev >= 0 && prev != device_ordinal) cudaSetDevice(prev);
  if (st != B2_OK) SetMsg(err, err_cap, why);
  return st;
}

}  // extern "C"
