// A decoded VMProgram v3 (host side): what the loader needs from the blob the
// reference's lowering + scheduler serialize (python/pjrt_ocl/lowering.py:286-331,
// python/pjrt_ocl/scheduler.py:226-248). Takes the place of pjrt_ocl::VmProgram
// (pjrt_plugin/src/runtime.h:77-104) behind the C ABI.
//
// Decoding is three passes over the blob (vmprog.cc): a layout pass that only
// locates the sections, a copy pass that lifts them into the vectors below, and
// a rule-table driven validation pass over buffers, tasks and lane streams.
#ifndef B2VM_VMPROG_H_
#define B2VM_VMPROG_H_

#include <cstdint>
#include <string>
#include <vector>

#include "format.h"

namespace b2 {

// One row of the buffer table.
struct BufferSlot {
  uint64_t offset = 0;   // byte offset in the arena
  uint64_t bytes = 0;
  uint32_t dtype = 0;
};

// The arguments or the results of a program: buffer ids in call order and the
// logical shape of each.
struct IoList {
  std::vector<uint32_t> ids;
  std::vector<std::vector<int64_t>> dims;
  size_t size() const { return ids.size(); }
};

// Bytes to place at the start of a buffer once, at load.
struct ConstInit {
  uint32_t buffer = 0;
  std::vector<uint8_t> data;
};

struct VmProgram {
  uint64_t arena_bytes = 0;
  std::vector<BufferSlot> buffers;
  IoList args, results;
  std::vector<int32_t> aux;            // descriptor pool, signed words
  std::vector<ConstInit> consts;
  // The tensor-level instruction list is the semantics the reference's numpy
  // validators execute; the device runs the schedule sections only, so the
  // instructions are counted and skipped.
  uint32_t n_instrs = 0, root_instrs = 0;
  // schedule
  uint32_t n_lanes = 0, n_flags = 0;
  std::vector<VmTask> tasks;
  std::vector<VmLane> lane_tab;
  std::vector<VmEntry> entries;
  uint32_t barriers_per_lane = 0;      // BARRIER entries in every lane's stream (equal by construction)

  // Decodes and validates a serialized program. Returns false with *err set
  // ("VMProgram parse error: ..."); the messages are the reference parser's
  // (pjrt_plugin/src/runtime.cc:90-251) so callers can match on them.
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
