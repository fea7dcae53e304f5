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

// What the runtime needs to encode one TMA tensor map over 16-bit elements: a tensor of
// rank 3 or 4 whose innermost dimension has unit stride, read in boxes with the 128-byte
// swizzle. Matmul operands: {inner = k or rows, outer, batch}; flash-attention operands:
// {inner, rows, h0, h1}.
struct TmapSpec {
  BufRef base;            // operand buffer (absolute address, or an I/O port)
  int64_t off;            // elements
  uint32_t dtype;         // kBF16 / kF16
  uint32_t rank;          // 3 or 4
  uint64_t dims[4];       // innermost first
  int64_t strides[3];     // elements, of dims[1..]; must be positive multiples of 8
  uint32_t box[4];
  uint32_t desc_word;     // where the owning DMma / DFlash sits in the descriptor pool (to clear its tmap on failure)
  uint32_t owner_is_flash;
  bool valid;             // false: known at load to be indescribable (e.g. a batch-broadcast operand)
};

struct DeviceTables {
  std::vector<DTask> tasks;
  std::vector<DEntry> entries;
  std::vector<VmLane> lanes;            // per lane: its span of `entries` (the program's table, or the rebuilt one
                                        // when strided reductions were spread over the lanes)
  std::vector<uint64_t> desc;           // descriptor pool (word 0 reserved: offset 0 = none)
  std::vector<int> input_port;          // per program input: port index or -1 (goes through the arena)
  std::vector<int> output_port;         // per program output
  std::vector<int> inout_result;        // per program input: the result that is the same buffer (an in/out port), or -1
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
  uint32_t n_flash_decode = 0;          // ... on the 16-byte-load decode path
  uint32_t n_rebalanced = 0;            // phases whose units were re-cut evenly over all lanes
  uint32_t n_carried_sums = 0;          // full sums whose input the row op that wrote it summed on the way (kRowCarrySum)
  uint32_t n_carried_barriers_removed = 0;   // barriers between such a row op and its sum that ordered nothing any more
  uint32_t n_rms_rows = 0;              // decomposed RMS norms over bf16 rows run as one row op
  uint32_t n_empty_phases_dropped = 0;  // barriers closing phases that hold nothing after such a rewrite
  uint32_t n_folded_converts = 0;       // 16-bit -> f32 converts folded into the full reduction that follows them
  uint32_t n_row_pipelines = 0;         // groups of neighbouring row-local phases run as one pipeline per lane, barriers removed
  uint32_t n_spread = 0;                // reduction phases re-cut over all lanes
  uint32_t n_fused_reduce = 0;          // ... of which full reductions (RED_PART + RED_COMB in one phase)
  bool needs_scratch = false;           // a re-cut full reduction leaves lane totals in the program's scratch
  uint32_t families = kFamEw;           // tile-op families the program's tasks use (picks the megakernel build)
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
