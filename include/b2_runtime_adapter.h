// b2_runtime_adapter.h - the three classes pjrt_plugin/src/plugin.cc uses from
// pjrt_plugin/src/runtime.h (OclRuntime, VmProgram, LoadedProgram), with the same names,
// method names and bool + std::string* error convention, implemented over the C ABI of
// libb2vm (b2vm.h). Including this header where plugin.cc includes runtime.h, and storing
// `void*` device pointers where it stores `cl_mem`, is the whole binding; nothing above it
// (PJRT C API surface, lowering subprocess, Python passes, scheduler) changes.
//
// Header-only, C++14. A LoadedProgram takes ONE execute at a time (it owns one arena and
// one barrier block): callers serialise executes of the same loaded program, as the
// reference does with its runtime mutex (runtime.h:301).
#ifndef B2_RUNTIME_ADAPTER_H_
#define B2_RUNTIME_ADAPTER_H_

#include <cstdint>
#include <cstdlib>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "b2vm.h"

namespace pjrt_ocl {

// What plugin.cc reads from OclRuntime::info() (runtime.h:57-72; plugin.cc:328).
struct DeviceInfo {
  std::string name;
  std::string vendor = "NVIDIA";
  uint32_t compute_units = 0;
  uint64_t global_mem_bytes = 0;
};

class OclRuntime {
 public:
  // OclRuntime::Create (runtime.h:124, plugin.cc:325). PJRT_OCL_DEVICE="<n>" selects the CUDA ordinal.
  static std::unique_ptr<OclRuntime> Create(std::string* err) {
    char msg[512] = {0};
    b2_runtime* h = nullptr;
    const char* ord = std::getenv("PJRT_OCL_DEVICE");
    if (b2_runtime_create(ord ? std::atoi(ord) : 0, &h, msg, sizeof msg) != B2_OK) {
      if (err) *err = msg;
      return nullptr;
    }
    std::unique_ptr<OclRuntime> rt(new OclRuntime);
    rt->h_ = h;
    b2_runtime_info(h, &rt->raw_);
    rt->info_.name = rt->raw_.device_name;
    rt->info_.compute_units = static_cast<uint32_t>(rt->raw_.sm_count);
    rt->info_.global_mem_bytes = rt->raw_.total_mem_bytes;
    return rt;
  }
  ~OclRuntime() { if (h_) b2_runtime_destroy(h_); }
  OclRuntime(const OclRuntime&) = delete;
  OclRuntime& operator=(const OclRuntime&) = delete;

  const DeviceInfo& info() const { return info_; }
  uint32_t ngroups() const { return raw_.lanes; }   // -> PJRT_OCL_NLANES (plugin.cc:771)
  uint32_t ew_ts() const { return raw_.ew_ts; }     // -> PJRT_OCL_EW_TS  (plugin.cc:772)
  uint32_t mma_t() const { return raw_.mma_t; }     // -> PJRT_OCL_MMA_T  (plugin.cc:773)

  // AllocDevice / PoolFree / WriteToDevice / ReadFromDevice (runtime.cc:2244-2301).
  void* AllocDevice(size_t bytes, std::string* err) {
    void* p = nullptr;
    char m[512] = {0};
    if (b2_alloc(h_, bytes, &p, m, sizeof m) != B2_OK) { if (err) *err = m; return nullptr; }
    return p;
  }
  void PoolFree(void* dev, size_t bytes) { b2_free(h_, dev, bytes); }
  bool WriteToDevice(void* dev_dst, const void* host_src, size_t bytes, std::string* err) {
    char m[512] = {0};
    if (b2_h2d(h_, dev_dst, host_src, bytes, m, sizeof m) != B2_OK) { if (err) *err = m; return false; }
    return true;
  }
  bool ReadFromDevice(void* host_dst, const void* dev_src, size_t bytes, std::string* err) {
    char m[512] = {0};
    if (b2_d2h(h_, host_dst, dev_src, bytes, m, sizeof m) != B2_OK) { if (err) *err = m; return false; }
    return true;
  }
  b2_runtime* handle() const { return h_; }

 private:
  OclRuntime() = default;
  b2_runtime* h_ = nullptr;
  b2_device_info raw_{};
  DeviceInfo info_;
};

// VmProgram (runtime.h:77-104): a parsed blob. Move-only; Load consumes it.
class VmProgram {
 public:
  VmProgram() = default;
  VmProgram(VmProgram&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
  VmProgram& operator=(VmProgram&& o) noexcept {
    if (this != &o) { if (h_) b2_program_destroy(h_); h_ = o.h_; o.h_ = nullptr; }
    return *this;
  }
  ~VmProgram() { if (h_) b2_program_destroy(h_); }

  // VmProgram::Parse (runtime.h:100, plugin.cc:789): the same rejections as runtime.cc:90-251.
  static bool Parse(const uint8_t* data, size_t len, VmProgram* out, std::string* err) {
    char m[512] = {0};
    b2_program* h = nullptr;
    if (b2_program_parse(data, len, &h, m, sizeof m) != B2_OK) { if (err) *err = m; return false; }
    *out = VmProgram();
    out->h_ = h;
    return true;
  }
  size_t num_inputs() const { return b2_program_num_inputs(h_); }
  size_t num_outputs() const { return b2_program_num_outputs(h_); }
  uint64_t input_bytes(size_t i) const { return b2_program_io_bytes(h_, 0, static_cast<uint32_t>(i)); }
  uint64_t output_bytes(size_t i) const { return b2_program_io_bytes(h_, 1, static_cast<uint32_t>(i)); }
  uint32_t output_dtype(size_t i) const { return b2_program_io_dtype(h_, 1, static_cast<uint32_t>(i)); }
  std::vector<int64_t> output_dims(size_t i) const {
    std::vector<int64_t> d(b2_program_io_rank(h_, 1, static_cast<uint32_t>(i)));
    for (size_t k = 0; k < d.size(); ++k) d[k] = b2_program_io_dim(h_, 1, static_cast<uint32_t>(i), static_cast<uint32_t>(k));
    return d;
  }
  b2_program* release() { b2_program* h = h_; h_ = nullptr; return h; }
  const b2_program* handle() const { return h_; }

 private:
  friend class LoadedProgram;
  b2_program* h_ = nullptr;
};

// LoadedProgram (runtime.h:309-435).
class LoadedProgram {
 public:
  static std::unique_ptr<LoadedProgram> Load(OclRuntime* rt, VmProgram prog, std::string* err) {
    char m[512] = {0};
    b2_loaded* h = nullptr;
    if (b2_program_load(rt->handle(), prog.h_, &h, m, sizeof m) != B2_OK) { if (err) *err = m; return nullptr; }
    prog.h_ = nullptr;                       // moved into the loaded program
    std::unique_ptr<LoadedProgram> lp(new LoadedProgram);
    lp->h_ = h;
    lp->rt_ = rt;
    return lp;
  }
  ~LoadedProgram() { if (h_) b2_loaded_destroy(h_); }
  LoadedProgram(const LoadedProgram&) = delete;
  LoadedProgram& operator=(const LoadedProgram&) = delete;

  size_t num_inputs() const { return b2_program_num_inputs(b2_loaded_program(h_)); }
  size_t num_outputs() const { return b2_program_num_outputs(b2_loaded_program(h_)); }
  uint64_t output_bytes(size_t i) const { return b2_program_io_bytes(b2_loaded_program(h_), 1, static_cast<uint32_t>(i)); }

  // Host in / host out, synchronous (runtime.h:326; what runtime_test.cc drives).
  bool Execute(const std::vector<const void*>& inputs, std::vector<std::vector<uint8_t>>* outputs, std::string* err) {
    char m[512] = {0};
    outputs->resize(num_outputs());
    std::vector<void*> outs(outputs->size());
    for (size_t o = 0; o < outs.size(); ++o) {
      (*outputs)[o].resize(output_bytes(o));
      outs[o] = (*outputs)[o].data();
    }
    if (b2_execute_host(h_, inputs.data(), inputs.size(), outs.data(), outs.size(), m, sizeof m) != B2_OK) {
      if (err) *err = m;
      return false;
    }
    return true;
  }
  // Device in / device out: the plugin's hot path (runtime.h:333, plugin.cc:971). Outputs are pool
  // buffers the caller owns and returns through OclRuntime::PoolFree.
  bool ExecuteDevice(const std::vector<void*>& inputs, std::vector<void*>* outputs, std::string* err) {
    char m[512] = {0};
    outputs->assign(num_outputs(), nullptr);
    if (b2_execute_device(h_, inputs.data(), inputs.size(), outputs->data(), outputs->size(), m, sizeof m) != B2_OK) {
      if (err) *err = m;
      return false;
    }
    return true;
  }
  b2_loaded* handle() const { return h_; }

 private:
  LoadedProgram() = default;
  b2_loaded* h_ = nullptr;
  OclRuntime* rt_ = nullptr;
};

}  // namespace pjrt_ocl
#endif  // B2_RUNTIME_ADAPTER_H_
