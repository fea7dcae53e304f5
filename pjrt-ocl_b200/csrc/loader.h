// Host-side translation of a parsed VMProgram into the device tables the
// megakernel walks. Mirrors the role of LoadedProgram::Load in the reference
// (pjrt_plugin/src/runtime.cc:735-1074): buffer ids -> addresses / I/O ports,
// control cond ids -> addresses, dynamic-slice index locations; and adds what a
// B200 loader can decide once per program: collapsed access maps, vector-path
// eligibility, and the fused elementwise chains with their dead intermediates.
#ifndef B2VM_LOADER_H_
#define B2VM_LOADER_H_

#include <cstdint>
#include <string>
#include <vector>

#include "format.h"
#include "vmprog.h"

namespace b2 {

// What the runtime needs to encode the tensor map of one tensor-core matmul operand:
// a [batch, rows, k] tensor of 16-bit elements, unit stride along k ("K-major") or
// along rows ("MN-major").
struct TmapSpec {
  BufRef base;            // operand buffer (absolute address, or an I/O port)
  int64_t off;            // elements
  uint32_t dtype;         // kBF16 / kF16
  bool mn_major;
  int64_t rows, k, batch;
  int64_t ld, gs;         // elements
  uint32_t desc_word;     // where the owning DMma sits in the descriptor pool (to clear DMma::tmap on failure)
};

struct DeviceTables {
  std::vector<DTask> tasks;
  std::vector<DEntry> entries;
  std::vector<VmLane> lanes;            // per lane: its span of `entries` (the program's table, or the rebuilt one
                                        // when strided reductions were spread over the lanes)
  std::vector<uint64_t> desc;           // descriptor pool (word 0 reserved: offset 0 = none)
  std::vector<int> input_port;          // per program input: port index or -1 (goes through the arena)
  std::vector<int> output_port;         // per program output
  int n_ports = 0;
  std::vector<TmapSpec> tmaps;          // two per tensor-core matmul task (A, B), in DMma::tmap order
  // statistics for tests / logging
  uint32_t n_chains = 0;                // fused elementwise chains (length > 1)
  uint32_t n_forwarded = 0;             // operands taken from registers
  uint32_t n_dead_stores = 0;           // intermediate stores elided
  uint32_t n_mma = 0;                   // matmul tasks
  uint32_t n_mma_tc = 0;                // ... of which the tensor-core path takes
  uint64_t mma_flops = 0;               // sum over matmul tasks of 2 G M N K
  uint32_t n_flash = 0, n_flash_tc = 0; // flash-attention tasks / ... on the tensor-core path
  uint32_t n_spread = 0;                // strided-reduction phases spread over all lanes
};

// `arena_base` is the device address of the arena (only its value is used).
// Returns false with *err and *unimplemented set when the program uses a tile op
// or shape outside the backend's coverage.
bool BuildDeviceTables(const VmProgram &p, uint64_t arena_base, DeviceTables *out, std::string *err,
                       bool *unimplemented);

// Collapse {dims, strides, off} to at most kViewDims dims; exposed for unit tests.
bool CollapseView(const int32_t *dims, const int32_t *strides, int rank, int64_t off, DView *out);

}  // namespace b2
#endif
