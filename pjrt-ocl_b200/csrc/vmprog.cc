// VMProgram v3 decoder. Accepts what the reference's VmProgram::Parse accepts
// (pjrt_plugin/src/runtime.cc:90-251) and, like its Python reader
// (python/pjrt_ocl/vmreader.py:314-315,374-376), refuses trailing bytes; buffers
// must also sit on a multiple of their element size, because the device reads
// 8-byte types with 8-byte accesses.
//
// Three passes:
//   1. Locate(): walks the blob once and records where every section starts and
//      how many records it holds; variable-length sections (shapes, constants)
//      are measured, nothing is copied. All "truncated ..." errors come from here.
//   2. Lift(): copies the located sections into the VmProgram vectors.
//   3. Check*(): validates buffers, I/O maps, constants, tasks (from a per-op
//      rule table) and lane streams against each other.
#include "vmprog.h"

#include <cstring>

namespace b2 {
namespace {

struct Span {
  size_t at = 0;      // byte offset of the first record
  size_t count = 0;   // records
};

// Where everything is. Record sizes are fixed by the format (format.h).
struct Sections {
  uint32_t n_buffers = 0, n_instrs = 0, n_consts = 0, root_instrs = 0, n_args = 0, n_results = 0, n_aux = 0;
  uint64_t arena_bytes = 0;
  Span buffers, arg_ids, result_ids, shapes, aux, consts, sched, tasks, lanes, entries;
  uint32_t n_tasks = 0, n_entries = 0, n_flags = 0, n_lanes = 0;
  size_t end = 0;
};

constexpr size_t kHeaderBytes = 48, kBufferRow = 24, kInstrRow = 32, kSchedHeader = 16;

class Walker {
 public:
  Walker(const uint8_t *d, size_t n) : d_(d), n_(n) {}
  size_t at() const { return at_; }
  size_t left() const { return n_ - at_; }
  // Claims `count` records of `rec` bytes; false when they do not fit.
  bool Take(size_t count, size_t rec, Span *s) {
    if (rec && count > left() / rec) return false;
    if (s) { s->at = at_; s->count = count; }
    at_ += count * rec;
    return true;
  }
  bool Align8() {
    const size_t a = (at_ + 7) & ~size_t{7};
    if (a > n_) return false;
    at_ = a;
    return true;
  }
  template <typename T>
  bool Peek(size_t off, T *v) const {      // value at at() + off, without moving
    if (left() < off + sizeof(T)) return false;
    std::memcpy(v, d_ + at_ + off, sizeof(T));
    return true;
  }

 private:
  const uint8_t *d_;
  size_t n_, at_ = 0;
};

template <typename T>
T Load(const uint8_t *d, size_t at) {
  T v;
  std::memcpy(&v, d + at, sizeof(T));
  return v;
}

// ---- pass 1 ------------------------------------------------------------------
const char *Locate(const uint8_t *d, size_t len, Sections *s, std::string *detail) {
  Walker w(d, len);
  uint32_t head[10];
  if (len < 8) return "truncated header";
  std::memcpy(head, d, 8);
  if (head[0] != kMagic) return "bad magic";
  if (head[1] != kVersion) {
    *detail = "unsupported version " + std::to_string(head[1]) + " (executor expects 3)";
    return "";
  }
  if (len < kHeaderBytes) return "truncated header";
  std::memcpy(head, d, sizeof(head));
  s->n_buffers = head[2]; s->n_instrs = head[3]; s->n_consts = head[4]; s->root_instrs = head[5];
  s->n_args = head[6]; s->n_results = head[7]; s->n_aux = head[8];
  s->arena_bytes = Load<uint64_t>(d, 40);
  w.Take(1, kHeaderBytes, nullptr);
  if (!w.Take(s->n_buffers, kBufferRow, &s->buffers)) return "truncated buffer table";
  if (!w.Take(s->n_args, 4, &s->arg_ids) || !w.Align8()) return "bad input map";
  if (!w.Take(s->n_results, 4, &s->result_ids) || !w.Align8()) return "bad output map";
  // shapes: {rank u32, pad u32, dims u64[rank]} per argument, then per result
  s->shapes.at = w.at();
  s->shapes.count = size_t{s->n_args} + s->n_results;
  for (size_t i = 0; i < s->shapes.count; ++i) {
    uint32_t rank;
    if (!w.Peek(0, &rank) || rank > 16 || !w.Take(1, 8 + size_t{rank} * 8, nullptr) || !w.Align8())
      return i < s->n_args ? "bad input shapes" : "bad output shapes";
  }
  if (!w.Take(s->n_aux, 4, &s->aux)) return "truncated aux";
  if (!w.Align8()) return "aux align";
  // constants: {buffer u32, byte_len u32, data, pad to 8}
  s->consts.at = w.at();
  s->consts.count = s->n_consts;
  for (uint32_t i = 0; i < s->n_consts; ++i) {
    uint32_t byte_len;
    if (!w.Peek(4, &byte_len)) return "bad const entry";
    if (!w.Take(1, 8, nullptr)) return "bad const entry";
    if (!w.Take(byte_len, 1, nullptr) || !w.Align8()) return "truncated const data";
  }
  if (s->root_instrs > s->n_instrs) return "main_len > n_instrs";
  if (!w.Take(s->n_instrs, kInstrRow, nullptr)) return "truncated instructions";
  if (!w.Align8()) return "instr align";
  uint32_t sh[4];
  if (!w.Peek(0, &sh)) return "truncated sched header";
  w.Take(1, kSchedHeader, &s->sched);
  s->n_tasks = sh[0]; s->n_entries = sh[1]; s->n_flags = sh[2]; s->n_lanes = sh[3];
  if (s->n_lanes == 0 || s->n_lanes > 4096) return "bad n_lanes";
  if (!w.Take(s->n_tasks, sizeof(VmTask), &s->tasks)) return "truncated tasks";
  if (!w.Take(s->n_lanes, sizeof(VmLane), &s->lanes)) return "truncated/bad lane tab";
  if (!w.Align8()) return "lane tab align";
  if (!w.Take(s->n_entries, sizeof(VmEntry), &s->entries)) return "truncated entries";
  s->end = w.at();
  if (w.left() != 0) {
    *detail = "trailing bytes: parsed " + std::to_string(w.at()) + " of " + std::to_string(len);
    return "";
  }
  return nullptr;
}

// ---- pass 2 ------------------------------------------------------------------
template <typename T>
void CopyRows(const uint8_t *d, const Span &s, std::vector<T> *v) {
  v->resize(s.count);
  if (s.count) std::memcpy(v->data(), d + s.at, s.count * sizeof(T));
}

void Lift(const uint8_t *d, const Sections &s, VmProgram *p) {
  p->arena_bytes = s.arena_bytes;
  p->n_instrs = s.n_instrs;
  p->root_instrs = s.root_instrs;
  p->buffers.resize(s.n_buffers);
  for (size_t i = 0; i < s.n_buffers; ++i) {
    const size_t at = s.buffers.at + i * kBufferRow;
    p->buffers[i] = BufferSlot{Load<uint64_t>(d, at), Load<uint64_t>(d, at + 8), Load<uint32_t>(d, at + 16)};
  }
  CopyRows(d, s.arg_ids, &p->args.ids);
  CopyRows(d, s.result_ids, &p->results.ids);
  size_t at = s.shapes.at;
  for (IoList *io : {&p->args, &p->results}) {
    io->dims.resize(io->ids.size());
    for (auto &dims : io->dims) {
      const uint32_t rank = Load<uint32_t>(d, at);
      dims.resize(rank);
      for (uint32_t k = 0; k < rank; ++k) dims[k] = static_cast<int64_t>(Load<uint64_t>(d, at + 8 + size_t{k} * 8));
      at = (at + 8 + size_t{rank} * 8 + 7) & ~size_t{7};
    }
  }
  CopyRows(d, s.aux, &p->aux);
  p->consts.resize(s.n_consts);
  at = s.consts.at;
  for (ConstInit &c : p->consts) {
    c.buffer = Load<uint32_t>(d, at);
    const uint32_t byte_len = Load<uint32_t>(d, at + 4);
    c.data.assign(d + at + 8, d + at + 8 + byte_len);
    at = (at + 8 + byte_len + 7) & ~size_t{7};
  }
  p->n_flags = s.n_flags;
  p->n_lanes = s.n_lanes;
  CopyRows(d, s.tasks, &p->tasks);
  CopyRows(d, s.lanes, &p->lane_tab);
  CopyRows(d, s.entries, &p->entries);
}

// ---- pass 3 ------------------------------------------------------------------
// Which task parameters refer to other tables. Bit k of a mask = parameter pk.
struct TaskRule {
  uint8_t ids;        // pk is a buffer id
  uint8_t aux_at;     // pk is the offset of a descriptor block: must be < n_aux
  uint8_t aux_opt;    // pk is 0 (absent) or 1 + an aux offset: must be <= n_aux
};

constexpr uint8_t P(int k) { return static_cast<uint8_t>(1u << k); }

TaskRule RuleFor(const VmTask &t) {
  switch (t.tile_op & 0xFFu) {
    case kTopEw: return {static_cast<uint8_t>(t.p0 == kSelect ? P(3) : 0), 0, 0};
    case kTopMma: return {static_cast<uint8_t>(t.p6 ? P(7) : 0), 0, static_cast<uint8_t>(P(4) | P(5) | P(6))};
    case kTopMapRegion: return {static_cast<uint8_t>(P(2) | P(3) | P(4) | P(5) | P(6) | P(7)), 0, 0};
    case kTopFlashAttn: return {P(0), P(3), 0};
    case kTopGather: case kTopIotaDim: case kTopScatter: case kTopDynGather: case kTopDynScatter:
    case kTopRedWindow: case kTopGatherIndex: case kTopScatterIndex: case kTopConv:
      return {0, P(0), 0};
    default: return {0, 0, 0};
  }
}

bool CheckBuffers(const VmProgram &p, std::string *m) {
  for (const BufferSlot &b : p.buffers) {
    if (b.dtype > kDtMax) { *m = "unsupported dtype " + std::to_string(b.dtype); return false; }
    const uint64_t unit = DtypeSize(b.dtype) > 4 ? DtypeSize(b.dtype) : 4;
    if (b.offset % unit || b.bytes > p.arena_bytes || b.offset > p.arena_bytes - b.bytes) {
      *m = "buffer outside arena / misaligned";
      return false;
    }
  }
  const uint32_t nb = static_cast<uint32_t>(p.buffers.size());
  for (uint32_t id : p.args.ids)
    if (id >= nb) { *m = "bad input map"; return false; }
  for (uint32_t id : p.results.ids)
    if (id >= nb) { *m = "bad output map"; return false; }
  for (const ConstInit &c : p.consts) {
    if (c.buffer >= nb) { *m = "bad const entry"; return false; }
    if (c.data.size() > p.buffers[c.buffer].bytes) { *m = "const too big"; return false; }
  }
  return true;
}

bool CheckTasks(const VmProgram &p, std::string *m) {
  const uint32_t nb = static_cast<uint32_t>(p.buffers.size()), na = static_cast<uint32_t>(p.aux.size());
  for (size_t i = 0; i < p.tasks.size(); ++i) {
    const VmTask &t = p.tasks[i];
    const uint32_t op = t.tile_op & 0xFFu, dt = (t.tile_op >> 8) & 0xFFu, adt = (t.tile_op >> 16) & 0xFFu;
    const std::string who = "task " + std::to_string(i) + ": ";
    if (op > kTopMax) { *m = who + "unknown tile_op " + std::to_string(op); return false; }
    if (dt > kDtMax || adt > kDtMax) { *m = who + "unknown dtype " + std::to_string(dt > kDtMax ? dt : adt); return false; }
    if (t.dst >= nb || t.a >= nb || t.b >= nb) { *m = who + "task buffer id out of range"; return false; }
    const TaskRule r = RuleFor(t);
    const uint32_t pk[8] = {t.p0, t.p1, t.p2, t.p3, t.p4, t.p5, t.p6, t.p7};
    for (int k = 0; k < 8; ++k) {
      if ((r.ids & P(k)) && pk[k] >= nb) { *m = who + "p" + std::to_string(k) + " buffer id out of range"; return false; }
      if ((r.aux_at & P(k)) && pk[k] >= na) { *m = who + "p" + std::to_string(k) + " aux offset out of range"; return false; }
      if ((r.aux_opt & P(k)) && pk[k] > na) { *m = who + "p" + std::to_string(k) + " aux offset out of range"; return false; }
    }
    if (op == kTopFlashAttn && uint64_t{t.p3} + 9 > na) { *m = who + "flash-attn descriptor out of range"; return false; }
  }
  return true;
}

// One lane's stream: entries name existing tasks, control entries name ranges
// inside the stream and an existing condition buffer. Returns the number of
// BARRIER entries through *barriers.
bool CheckLane(const VmProgram &p, const VmLane &l, uint32_t *barriers, std::string *m) {
  if (uint64_t{l.off} + l.count > p.entries.size()) { *m = "lane range oob"; return false; }
  if (l.root_len > l.count) { *m = "truncated/bad lane tab"; return false; }
  auto inside = [&](uint32_t start, uint32_t n) { return uint64_t{start} + n <= l.count; };
  *barriers = 0;
  for (uint32_t e = 0; e < l.count; ++e) {
    const VmEntry &en = p.entries[l.off + e];
    switch (en.task) {
      case kEntNop: break;
      case kEntBarrier: ++*barriers; break;
      case kEntFor:
        if (!inside(en.tile_lo, en.tile_hi)) { *m = "control sub-range out of lane stream"; return false; }
        break;
      case kEntWhile: case kEntIf:
        if (en.signal_flag >= p.buffers.size()) { *m = "control cond buffer id out of range"; return false; }
        if (!inside(en.tile_lo, en.tile_hi) || !inside(en.wait_flag, en.wait_count)) {
          *m = "control sub-range out of lane stream";
          return false;
        }
        break;
      default:
        if (en.task >= p.tasks.size()) { *m = "entry task index out of range"; return false; }
    }
  }
  return true;
}

}  // namespace

bool VmProgram::Parse(const uint8_t *data, size_t len, VmProgram *out, std::string *err) {
  auto fail = [&](const std::string &m) {
    *err = "VMProgram parse error: " + m;
    return false;
  };
  Sections s;
  std::string detail;
  if (const char *why = Locate(data, len, &s, &detail)) return fail(detail.empty() ? why : detail);
  Lift(data, s, out);
  std::string m;
  if (!CheckBuffers(*out, &m) || !CheckTasks(*out, &m)) return fail(m);
  // every lane must meet the same number of grid barriers, or the first one hangs the rest
  for (size_t l = 0; l < out->lane_tab.size(); ++l) {
    uint32_t barriers = 0;
    if (!CheckLane(*out, out->lane_tab[l], &barriers, &m)) return fail(m);
    if (l == 0) out->barriers_per_lane = barriers;
    else if (barriers != out->barriers_per_lane) return fail("non-uniform top-level barrier counts across lanes");
  }
  return true;
}

}  // namespace b2
