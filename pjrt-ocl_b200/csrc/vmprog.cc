// VMProgram v3 parser + validator: the same acceptance rules as the reference's
// VmProgram::Parse (pjrt_plugin/src/runtime.cc:90-251), plus the trailing-byte
// rejection of its Python reader (python/pjrt_ocl/vmreader.py:314-315,374-376).
#include "vmprog.h"

#include <cstring>

namespace b2 {
namespace {

class Cursor {
 public:
  Cursor(const uint8_t *d, size_t n) : d_(d), n_(n) {}
  template <typename T>
  bool Get(T *v) {
    if (n_ - pos_ < sizeof(T)) return false;
    std::memcpy(v, d_ + pos_, sizeof(T));
    pos_ += sizeof(T);
    return true;
  }
  bool Raw(void *dst, size_t bytes) {
    if (n_ - pos_ < bytes) return false;
    if (bytes) std::memcpy(dst, d_ + pos_, bytes);
    pos_ += bytes;
    return true;
  }
  bool Skip(size_t bytes) {
    if (n_ - pos_ < bytes) return false;
    pos_ += bytes;
    return true;
  }
  bool Pad8() {
    size_t p = (pos_ + 7) & ~size_t{7};
    if (p > n_) return false;
    pos_ = p;
    return true;
  }
  size_t pos() const { return pos_; }
  size_t left() const { return n_ - pos_; }

 private:
  const uint8_t *d_;
  size_t n_, pos_ = 0;
};

bool NeedsAuxBlock(uint32_t op) {
  return op == kTopGather || op == kTopIotaDim || op == kTopDynGather || op == kTopDynScatter ||
         op == kTopRedWindow || op == kTopGatherIndex || op == kTopScatterIndex;
}

}  // namespace

bool VmProgram::Parse(const uint8_t *data, size_t len, VmProgram *out, std::string *err) {
  Cursor c(data, len);
  auto fail = [&](const std::string &m) {
    *err = "VMProgram parse error: " + m;
    return false;
  };
  uint32_t magic, version, n_buffers, n_instrs, n_consts, main_len, n_inputs, n_outputs, n_aux, hpad;
  if (!c.Get(&magic) || !c.Get(&version)) return fail("truncated header");
  if (magic != kMagic) return fail("bad magic");
  if (version != kVersion)
    return fail("unsupported version " + std::to_string(version) + " (executor expects 3)");
  if (!c.Get(&n_buffers) || !c.Get(&n_instrs) || !c.Get(&n_consts) || !c.Get(&main_len) ||
      !c.Get(&n_inputs) || !c.Get(&n_outputs) || !c.Get(&n_aux) || !c.Get(&hpad) ||
      !c.Get(&out->arena_bytes))
    return fail("truncated header");
  out->main_len = main_len;
  out->n_instrs = n_instrs;

  if (uint64_t{n_buffers} * 24 > c.left()) return fail("truncated buffer table");
  out->buffers.resize(n_buffers);
  for (auto &b : out->buffers) {
    uint32_t pad;
    if (!c.Get(&b.arena_byte_offset) || !c.Get(&b.size_bytes) || !c.Get(&b.dtype) || !c.Get(&pad))
      return fail("truncated buffer table");
    if (b.dtype > kDtMax) return fail("unsupported dtype " + std::to_string(b.dtype));
    if (b.arena_byte_offset % 4 || b.arena_byte_offset + b.size_bytes > out->arena_bytes)
      return fail("buffer outside arena / misaligned");
  }

  auto read_ids = [&](uint32_t n, std::vector<uint32_t> *v) {
    if (uint64_t{n} * 4 > c.left()) return false;
    v->resize(n);
    for (auto &id : *v)
      if (!c.Get(&id) || id >= n_buffers) return false;
    return c.Pad8();
  };
  if (!read_ids(n_inputs, &out->inputs)) return fail("bad input map");
  if (!read_ids(n_outputs, &out->outputs)) return fail("bad output map");

  auto read_shapes = [&](size_t n, std::vector<std::vector<int64_t>> *v) {
    v->resize(n);
    for (auto &dims : *v) {
      uint32_t rank, pad;
      if (!c.Get(&rank) || !c.Get(&pad) || rank > 16) return false;
      dims.resize(rank);
      for (auto &d : dims) {
        uint64_t u;
        if (!c.Get(&u)) return false;
        d = static_cast<int64_t>(u);
      }
      if (!c.Pad8()) return false;
    }
    return true;
  };
  if (!read_shapes(n_inputs, &out->input_dims)) return fail("bad input shapes");
  if (!read_shapes(n_outputs, &out->output_dims)) return fail("bad output shapes");

  if (uint64_t{n_aux} * 4 > c.left()) return fail("truncated aux");
  out->aux.resize(n_aux);
  if (!c.Raw(out->aux.data(), size_t{n_aux} * 4)) return fail("truncated aux");
  if (!c.Pad8()) return fail("aux align");

  if (uint64_t{n_consts} * 8 > c.left()) return fail("bad const entry");
  out->consts.resize(n_consts);
  for (auto &entry : out->consts) {
    uint32_t byte_len;
    if (!c.Get(&entry.first) || !c.Get(&byte_len) || entry.first >= n_buffers)
      return fail("bad const entry");
    if (byte_len > out->buffers[entry.first].size_bytes) return fail("const too big");
    if (byte_len > c.left()) return fail("truncated const data");
    entry.second.resize(byte_len);
    if (!c.Raw(entry.second.data(), byte_len) || !c.Pad8()) return fail("truncated const data");
  }

  if (main_len > n_instrs) return fail("main_len > n_instrs");
  // The tensor instruction list is the reference semantics for the validators;
  // the device executes the schedule sections only.
  if (!c.Skip(size_t{n_instrs} * 32)) return fail("truncated instructions");
  if (!c.Pad8()) return fail("instr align");

  uint32_t n_tasks, n_entries;
  if (!c.Get(&n_tasks) || !c.Get(&n_entries) || !c.Get(&out->n_flags) || !c.Get(&out->n_lanes))
    return fail("truncated sched header");
  if (out->n_lanes == 0 || out->n_lanes > 4096) return fail("bad n_lanes");
  if (uint64_t{n_tasks} * sizeof(VmTask) > c.left()) return fail("truncated tasks");
  out->tasks.resize(n_tasks);
  if (!c.Raw(out->tasks.data(), size_t{n_tasks} * sizeof(VmTask))) return fail("truncated tasks");
  if (uint64_t{out->n_lanes} * sizeof(VmLane) > c.left()) return fail("truncated/bad lane tab");
  out->lane_tab.resize(out->n_lanes);
  for (auto &l : out->lane_tab)
    if (!c.Get(&l.off) || !c.Get(&l.count) || !c.Get(&l.root_len) || !c.Get(&l.pad) ||
        l.root_len > l.count)
      return fail("truncated/bad lane tab");
  if (!c.Pad8()) return fail("lane tab align");
  if (uint64_t{n_entries} * sizeof(VmEntry) > c.left()) return fail("truncated entries");
  out->entries.resize(n_entries);
  if (!c.Raw(out->entries.data(), size_t{n_entries} * sizeof(VmEntry)))
    return fail("truncated entries");
  if (c.left() != 0)
    return fail("trailing bytes: parsed " + std::to_string(c.pos()) + " of " + std::to_string(len));

  for (const VmTask &t : out->tasks) {
    const uint32_t op = t.tile_op & 0xFFu, dt = (t.tile_op >> 8) & 0xFFu, adt = (t.tile_op >> 16) & 0xFFu;
    if (op > kTopMax) return fail("unknown tile_op " + std::to_string(op));
    if (dt > kDtMax || adt > kDtMax) return fail("unknown dtype " + std::to_string(dt));
    for (uint32_t id : {t.dst, t.a, t.b})
      if (id >= n_buffers) return fail("task buffer id out of range");
    if (op == kTopMapRegion)
      for (uint32_t id : {t.p2, t.p3, t.p4, t.p5, t.p6, t.p7})
        if (id >= n_buffers) return fail("region input buffer id out of range");
    if (op == kTopEw && t.p0 == kSelect && t.p3 >= n_buffers) return fail("select pred id out of range");
    if (NeedsAuxBlock(op) && t.p0 >= n_aux) return fail("task aux offset out of range");
    if (op == kTopMma && (t.p4 > n_aux || t.p5 > n_aux)) return fail("mma view aux offset out of range");
    if (op == kTopMma && t.p6 && (t.p6 > n_aux || t.p7 >= n_buffers))
      return fail("mma epilogue aux offset / residual id out of range");
    if (op == kTopFlashAttn && (t.p0 >= n_buffers || uint64_t{t.p3} + 9 > n_aux))
      return fail("flash-attn V id / aux offset out of range");
  }
  uint32_t barrier_ref = 0;
  bool first = true;
  for (const VmLane &l : out->lane_tab) {
    if (uint64_t{l.off} + l.count > n_entries) return fail("lane range oob");
    uint32_t barriers = 0;
    for (uint32_t e = l.off; e < l.off + l.count; ++e) {
      const VmEntry &en = out->entries[e];
      if (en.task == kEntBarrier) {
        barriers++;
      } else if (en.task == kEntWhile || en.task == kEntIf) {
        if (en.signal_flag >= n_buffers) return fail("control cond buffer id out of range");
        if (uint64_t{en.tile_lo} + en.tile_hi > l.count || uint64_t{en.wait_flag} + en.wait_count > l.count)
          return fail("control sub-range out of lane stream");
      } else if (en.task == kEntFor) {
        if (uint64_t{en.tile_lo} + en.tile_hi > l.count) return fail("control sub-range out of lane stream");
      } else if (en.task != kEntNop && en.task >= n_tasks) {
        return fail("entry task index out of range");
      }
    }
    if (first) {
      barrier_ref = barriers;
      first = false;
    } else if (barriers != barrier_ref) {
      return fail("non-uniform top-level barrier counts across lanes");
    }
    if (barriers > out->n_barriers) out->n_barriers = barriers;
  }
  out->n_barriers = out->n_barriers ? out->n_barriers : 1;
  return true;
}

}  // namespace b2
