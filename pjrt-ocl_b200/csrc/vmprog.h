// Parsed VMProgram v3 (host side). Mirrors the role of the reference's
// pjrt_ocl::VmProgram (pjrt_plugin/src/runtime.h:77-104).
#ifndef B2VM_VMPROG_H_
#define B2VM_VMPROG_H_

#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "format.h"

namespace b2 {

struct VmBuffer {
  uint64_t arena_byte_offset = 0;
  uint64_t size_bytes = 0;
  uint32_t dtype = 0;
};

struct VmProgram {
  uint64_t arena_bytes = 0;
  uint32_t main_len = 0;
  uint32_t n_instrs = 0;
  std::vector<VmBuffer> buffers;
  std::vector<uint32_t> inputs, outputs;               // buffer ids, argument / result order
  std::vector<std::vector<int64_t>> input_dims, output_dims;
  std::vector<std::pair<uint32_t, std::vector<uint8_t>>> consts;
  std::vector<int32_t> aux;
  uint32_t n_flags = 0, n_lanes = 0;
  std::vector<VmTask> tasks;
  std::vector<VmLane> lane_tab;
  std::vector<VmEntry> entries;
  uint32_t n_barriers = 0;

  // Parses and validates a serialized program. Returns false with *err set.
  static bool Parse(const uint8_t *data, size_t len, VmProgram *out, std::string *err);
};

inline size_t DtypeSize(uint32_t dt) {
  switch (dt) {
    case kBool: return 1;
    case kF16: case kBF16: return 2;
    case kI64: case kF64: return 8;
    default: return 4;
  }
}

}  // namespace b2
#endif
