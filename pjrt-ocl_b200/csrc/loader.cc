// Builds the device tables for one program. See loader.h.
#include "loader.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <set>

namespace b2 {
namespace {

struct Ctx {
  const VmProgram &p;
  uint64_t arena_base;
  std::map<uint32_t, int> port_of;   // buffer id -> port
  DeviceTables *out;

  BufRef Ref(uint32_t id) const {
    auto it = port_of.find(id);
    if (it != port_of.end()) return kPortBit | static_cast<uint64_t>(it->second);
    return arena_base + p.buffers[id].offset;
  }
  // Arena buffers are 64-byte aligned by the format; port addresses are checked at execute.
  bool Aligned16(uint32_t id) const {
    if (port_of.count(id)) return true;
    return (arena_base + p.buffers[id].offset) % 16 == 0;
  }
  template <typename T>
  uint32_t PushDesc(const T &v) {
    const size_t words = (sizeof(T) + 7) / 8;
    const uint32_t off = static_cast<uint32_t>(out->desc.size());
    out->desc.resize(out->desc.size() + words, 0);
    std::memcpy(&out->desc[off], &v, sizeof(T));
    return off;
  }
};

bool IsBin(uint32_t s) { return s <= kPow || s == kAtan2 || s == kRemainder; }
bool IsUn(uint32_t s) { return (s >= kCopy && s <= kSign) || (s >= kLog1p && s <= kRound) || s == kGelu; }
bool EwReadsA(uint32_t s) { return !(s == kFill || s == kIotaFlat); }
bool EwReadsB(uint32_t s) {
  return IsBin(s) || s == kCmp || s == kSelect || s == kLts || (s >= kAnd && s <= kXor) ||
         (s >= kShl && s <= kShrA);
}
bool Wide(uint32_t dt) { return dt == kI64 || dt == kF64; }

// Buffer ids a task reads from memory (for the dead-store proof).
void TaskReads(const VmProgram &p, const VmTask &t, std::vector<uint32_t> *r) {
  const uint32_t op = t.tile_op & 0xFFu;
  switch (op) {
    case kTopEw:
      if (EwReadsA(t.p0)) r->push_back(t.a);
      if (EwReadsB(t.p0)) r->push_back(t.b);
      if (t.p0 == kSelect) r->push_back(t.p3);
      break;
    case kTopMma:
      r->push_back(t.a); r->push_back(t.b);
      if (t.p6) r->push_back(t.p7);
      break;
    case kTopRedSeg:
      r->push_back(t.a);
      if (t.p3) r->push_back(t.b);
      break;
    case kTopMapRegion:
      for (uint32_t id : {t.a, t.b, t.p2, t.p3, t.p4, t.p5, t.p6, t.p7}) r->push_back(id);
      break;
    case kTopFlashAttn:
      r->push_back(t.a); r->push_back(t.b); r->push_back(t.p0);
      break;
    case kTopDynGather: case kTopDynScatter: {
      r->push_back(t.a);
      const int32_t rank = p.aux[t.p0];
      for (int32_t d = 0; d < rank; ++d) r->push_back(static_cast<uint32_t>(p.aux[t.p0 + 1 + 4 * rank + d]));
      if (op == kTopDynScatter) r->push_back(t.dst);  // partial overwrite keeps the rest
      break;
    }
    case kTopScatter:
      r->push_back(t.a); r->push_back(t.dst);
      break;
    case kTopIotaDim:
      break;
    default:
      r->push_back(t.a); r->push_back(t.b);
      break;
  }
}

bool ViewFromAux(const VmProgram &p, uint32_t aux_off, DView *v, std::string *err) {
  if (aux_off >= p.aux.size()) { *err = "view descriptor out of the aux pool"; return false; }
  const int32_t rank = p.aux[aux_off];
  if (rank < 0 || static_cast<size_t>(aux_off) + 2 + 2 * static_cast<size_t>(rank) > p.aux.size()) {
    *err = "view descriptor out of the aux pool";
    return false;
  }
  const int32_t *dims = &p.aux[aux_off + 1], *strides = &p.aux[aux_off + 1 + rank];
  if (!CollapseView(dims, strides, rank, p.aux[aux_off + 1 + 2 * rank], v)) {
    *err = "access map does not collapse to " + std::to_string(kViewDims) + " dims";
    return false;
  }
  return true;
}

// Is the view, read over the row-major flat index of a [n0, n1, n2] tensor, affine
// in the three coordinates? The view's (collapsed) dims and [n0, n1, n2] are two
// factorisations of the same index space; walk their common refinement from the
// innermost digit and require every piece of one coordinate to agree on that
// coordinate's stride.
bool AffineOverAxes(const DView &v, const int64_t n[3], int64_t stride[3], int64_t *off) {
  *off = v.off;
  stride[0] = stride[1] = stride[2] = 0;
  bool have[3] = {false, false, false};
  int a = 2, j = v.rank - 1;
  int64_t ra = n[2], wa = 1, rv = j >= 0 ? v.dim[j] : 1, wv = 1;
  auto next_axis = [&]() { while (a >= 0 && ra == 1) { --a; if (a >= 0) { ra = n[a]; wa = 1; } } };
  auto next_dim = [&]() { while (j >= 0 && rv == 1) { --j; if (j >= 0) { rv = v.dim[j]; wv = 1; } } };
  next_axis();
  next_dim();
  while (a >= 0 && j >= 0) {
    const int64_t p = std::min(ra, rv);
    if (ra % p != 0 || rv % p != 0) return false;
    const int64_t contrib = wv * static_cast<int64_t>(v.stride[j]);   // address step of one digit of this piece
    if (!have[a]) {
      if (wa != 1) return false;
      stride[a] = contrib;
      have[a] = true;
    } else if (contrib != wa * stride[a]) {
      return false;
    }
    ra /= p; wa *= p; rv /= p; wv *= p;
    next_axis();
    next_dim();
  }
  return a < 0 && j < 0;   // both factorisations consumed: same number of elements
}

// Classify one matmul operand for the tensor-core path. rows x K operand (A: rows = M;
// B: rows = N), given the element strides of (batch, row, k). Returns false when the
// layout cannot be fed to the tensor cores directly.
bool TcOperand(int64_t rows, int64_t K, int64_t sg, int64_t sr, int64_t sk, int64_t off, bool *mn_major, int64_t *ld,
               int64_t *gs) {
  if (off < 0 || off % 8 != 0 || sg < 0 || sg % 8 != 0) return false;
  *gs = sg;
  if (sk == 1 || K == 1) {                       // K-major: rows at pitch sr
    if (rows > 1 && (sr <= 0 || sr % 8 != 0)) return false;
    *mn_major = false;
    *ld = rows > 1 ? sr : 8;
    return true;
  }
  if (sr == 1 || rows == 1) {                    // MN-major: k rows at pitch sk
    if (sk <= 0 || sk % 8 != 0) return false;
    *mn_major = true;
    *ld = sk;
    return true;
  }
  return false;
}

// ---- spreading strided reductions over the lanes ----
//
// The scheduler tiles RED_STRIDED by outputs, EW_TS per tile (scheduler.py:178-197),
// so a reduction over a long interior axis with few outputs (config 4: 12288
// outputs of 4096 terms each) lands on 3 lanes while the others wait at the
// barrier. Where such a task is alone in its owners' runs the loader re-cuts it by rows:
// every lane gets an entry naming a row range (DEntry::a, b) instead of output
// tiles, and the original entries become NOPs. The new entries are inserted into
// the lanes' streams, so control ranges and the lane table are re-indexed.
//
// A lane's stream is a set of contiguous ranges: the root walk [0, root_len) and
// the cond / body / branch ranges of its control entries, in stream order.
// Barrier entries split a range into runs; run k is the same phase on every lane
// (the parser checked that barrier counts agree; range and run counts are
// compared again here and the pass backs off when they differ).
struct StreamRun {
  uint32_t range, start, end;   // entries [start, end) of the lane's stream, no barrier inside
  bool at_range_start, in_empty_range;
};

void LaneRuns(const VmProgram &p, const VmLane &l, std::vector<StreamRun> *runs) {
  std::vector<std::pair<uint32_t, uint32_t>> ranges;
  ranges.push_back({0u, l.root_len});
  for (uint32_t e = 0; e < l.count; ++e) {
    const VmEntry &en = p.entries[l.off + e];
    if (en.task == kEntFor || en.task == kEntWhile || en.task == kEntIf) ranges.push_back({en.tile_lo, en.tile_hi});
    if (en.task == kEntWhile || en.task == kEntIf) ranges.push_back({en.wait_flag, en.wait_count});
  }
  for (uint32_t r = 0; r < ranges.size(); ++r) {
    const uint32_t s = ranges[r].first, e = s + ranges[r].second;
    uint32_t run_start = s;
    for (uint32_t i = s; i <= e; ++i) {
      if (i == e || p.entries[l.off + i].task == kEntBarrier) {
        runs->push_back({r, run_start, i, run_start == s, s == e});
        run_start = i + 1;
      }
    }
  }
}

void SpreadStridedReductions(const VmProgram &p, DeviceTables *out) {
  const uint32_t n_lanes = static_cast<uint32_t>(p.lane_tab.size());
  if (n_lanes < 4) return;
  std::vector<std::vector<StreamRun>> runs(n_lanes);
  for (uint32_t l = 0; l < n_lanes; ++l) LaneRuns(p, p.lane_tab[l], &runs[l]);
  for (uint32_t l = 1; l < n_lanes; ++l) {
    if (runs[l].size() != runs[0].size()) return;
    for (size_t k = 0; k < runs[0].size(); ++k)
      if (runs[l][k].range != runs[0][k].range) return;
  }
  struct Insert { uint32_t pos; bool at_start; DEntry e; };
  std::vector<std::vector<Insert>> ins(n_lanes);
  for (size_t k = 0; k < runs[0].size(); ++k) {
    // One eligible RED_STRIDED task in this phase, alone in the runs of the lanes that
    // own it (entries of one lane run in order and may depend on each other; entries
    // of different lanes in one phase never do, so its rows can be appended to any
    // lane's run).
    int64_t task = -1;
    uint64_t tiles = 0;
    bool ok = true;
    for (uint32_t l = 0; l < n_lanes && ok; ++l) {
      const StreamRun &r = runs[l][k];
      if (r.in_empty_range) ok = false;
      uint32_t mine = 0, others = 0;
      for (uint32_t i = r.start; i < r.end && ok; ++i) {
        const VmEntry &en = p.entries[p.lane_tab[l].off + i];
        if (en.task == kEntNop) continue;
        if (en.task >= p.tasks.size()) { ok = false; break; }          // a control entry inside the run
        if ((p.tasks[en.task].tile_op & 0xFFu) != kTopRedStrided) { ++others; continue; }
        if (task >= 0 && task != static_cast<int64_t>(en.task)) { ok = false; break; }
        task = en.task;
        ++mine;
        tiles += en.tile_hi > en.tile_lo ? en.tile_hi - en.tile_lo : 0u;
      }
      if (mine && others) ok = false;
    }
    if (!ok || task < 0) continue;
    const VmTask &t = p.tasks[task];
    const uint32_t dt = (t.tile_op >> 8) & 0xFFu;
    const int64_t n_out = t.p0, red = t.p1, inner = t.p2;
    if (!red_strided_rows_ok(dt, red, inner, t.p3) || n_out % inner != 0) continue;
    const uint64_t nt = (static_cast<uint64_t>(n_out) + kEwTs - 1) / kEwTs;
    if (tiles != nt || nt * 2 > n_lanes) continue;
    const int64_t rows = n_out / inner;
    for (uint32_t l = 0; l < n_lanes; ++l) {
      const StreamRun &r = runs[l][k];
      for (uint32_t i = r.start; i < r.end; ++i)
        if (p.entries[p.lane_tab[l].off + i].task == static_cast<uint32_t>(task)) out->entries[p.lane_tab[l].off + i].task = kEntNop;
      const int64_t lo = rows * l / n_lanes, hi = rows * (l + 1) / n_lanes;
      if (hi <= lo) continue;
      DEntry e;
      std::memset(&e, 0, sizeof(e));
      e.task = static_cast<uint32_t>(task);
      e.a = static_cast<uint32_t>(lo);
      e.b = static_cast<uint32_t>(hi);
      const bool empty_at_start = r.start == r.end && r.at_range_start;
      ins[l].push_back({r.end, empty_at_start, e});
    }
    out->n_spread++;
  }
  if (!out->n_spread) return;
  std::vector<DEntry> rebuilt;
  rebuilt.reserve(out->entries.size() + static_cast<size_t>(out->n_spread) * n_lanes);
  for (uint32_t l = 0; l < n_lanes; ++l) {
    const VmLane &ln = p.lane_tab[l];
    const uint32_t new_off = static_cast<uint32_t>(rebuilt.size());
    // boundary[i]: new index where old position i starts, after the entries that
    // close the run ending at i and before those that open a range at i
    std::vector<uint32_t> boundary(ln.count + 1);
    for (uint32_t i = 0; i <= ln.count; ++i) {
      for (const Insert &x : ins[l])
        if (x.pos == i && !x.at_start) rebuilt.push_back(x.e);
      boundary[i] = static_cast<uint32_t>(rebuilt.size()) - new_off;
      for (const Insert &x : ins[l])
        if (x.pos == i && x.at_start) rebuilt.push_back(x.e);
      if (i < ln.count) rebuilt.push_back(out->entries[ln.off + i]);
    }
    const uint32_t new_count = static_cast<uint32_t>(rebuilt.size()) - new_off;
    for (uint32_t i = new_off; i < new_off + new_count; ++i) {
      DEntry &d = rebuilt[i];
      if (d.task == kEntFor || d.task == kEntWhile || d.task == kEntIf) {
        const uint32_t s = d.tile_lo, n = d.tile_hi;
        d.tile_lo = boundary[s];
        d.tile_hi = boundary[s + n] - boundary[s];
      }
      if (d.task == kEntWhile || d.task == kEntIf) {
        const uint32_t s = d.a, n = d.b;
        d.a = boundary[s];
        d.b = boundary[s + n] - boundary[s];
      }
    }
    out->lanes[l] = VmLane{new_off, new_count, boundary[ln.root_len], 0u};
  }
  out->entries.swap(rebuilt);
}

}  // namespace

bool CollapseView(const int32_t *dims, const int32_t *strides, int rank, int64_t off, DView *out) {
  std::vector<int64_t> d, s;
  for (int k = 0; k < rank; ++k) {
    if (dims[k] <= 0) return false;
    if (dims[k] == 1) continue;              // a size-1 axis contributes coordinate 0
    if (!d.empty() && s.back() == static_cast<int64_t>(strides[k]) * dims[k]) {
      d.back() *= dims[k];                   // row-major mergeable with the previous axis
      s.back() = strides[k];
    } else {
      d.push_back(dims[k]);
      s.push_back(strides[k]);
    }
  }
  if (d.size() > static_cast<size_t>(kViewDims)) return false;
  std::memset(out, 0, sizeof(*out));
  out->rank = static_cast<int32_t>(d.size());
  out->off = off;
  for (size_t k = 0; k < d.size(); ++k) {
    if (d[k] > 0xFFFFFFFFll) return false;
    out->dim[k] = static_cast<uint32_t>(d[k]);
    out->stride[k] = static_cast<int32_t>(s[k]);
    // branch-free magic-number division by dim[k] (>= 2 here: size-1 axes were dropped)
    const uint32_t dv = out->dim[k];
    uint32_t sh = 31;
    while (!(dv >> sh)) --sh;                       // floor(log2(dv))
    if ((dv & (dv - 1)) == 0) {
      out->magic[k] = 0;
      out->shift[k] = sh - 1;
    } else {
      const unsigned __int128 two = static_cast<unsigned __int128>(1) << (32 + sh);
      uint64_t m = static_cast<uint64_t>(two / dv);
      const uint64_t rem = static_cast<uint64_t>(two - static_cast<unsigned __int128>(m) * dv);
      m *= 2;
      if (rem * 2 >= dv) m += 1;
      out->magic[k] = static_cast<uint32_t>(m + 1);
      out->shift[k] = sh;
    }
  }
  if (out->rank == 0) {
    out->vec_ok = 1;
    out->inner_stride = 0;
    out->aligned4 = 1;
    return true;
  }
  const int last = out->rank - 1;
  out->inner_stride = out->stride[last];
  out->vec_ok = (out->dim[last] % 4 == 0 && (out->stride[last] == 0 || out->stride[last] == 1)) ? 1 : 0;
  bool a4 = off % 4 == 0;
  for (int k = 0; k < last; ++k) a4 = a4 && (out->stride[k] % 4 == 0);
  out->aligned4 = a4 ? 1 : 0;
  return true;
}

bool BuildDeviceTables(const VmProgram &p, uint64_t arena_base, DeviceTables *out, std::string *err,
                       bool *unimplemented) {
  *unimplemented = false;
  Ctx c{p, arena_base, {}, out};
  out->desc.assign(1, 0);

  // ---- zero-copy I/O ports (runtime.cc:798-821): a buffer that is only an input
  // or only an output, is not a constant, and is among the first kMaxIoPorts such.
  std::set<uint32_t> in_ids(p.args.ids.begin(), p.args.ids.end()), out_ids(p.results.ids.begin(), p.results.ids.end());
  std::set<uint32_t> const_ids;
  for (const auto &k : p.consts) const_ids.insert(k.buffer);
  auto assign_port = [&](uint32_t id) -> int {
    if (in_ids.count(id) && out_ids.count(id)) return -1;
    if (const_ids.count(id)) return -1;
    auto it = c.port_of.find(id);
    if (it != c.port_of.end()) return it->second;
    if (out->n_ports >= static_cast<int>(kMaxIoPorts)) return -1;
    return c.port_of[id] = out->n_ports++;
  };
  // A result buffer that no task ever writes (a pass-through of arena-resident
  // data) has to come out of the arena.
  std::set<uint32_t> written;
  for (const VmTask &t : p.tasks) written.insert(t.dst);
  out->input_port.assign(p.args.ids.size(), -1);
  out->output_port.assign(p.results.ids.size(), -1);
  for (size_t i = 0; i < p.args.ids.size(); ++i) out->input_port[i] = assign_port(p.args.ids[i]);
  for (size_t o = 0; o < p.results.ids.size(); ++o)
    out->output_port[o] = written.count(p.results.ids[o]) ? assign_port(p.results.ids[o]) : -1;

  // ---- tasks ----
  out->tasks.resize(p.tasks.size());
  for (size_t ti = 0; ti < p.tasks.size(); ++ti) {
    const VmTask &t = p.tasks[ti];
    DTask &d = out->tasks[ti];
    std::memset(&d, 0, sizeof(d));
    d.op = t.tile_op & 0xFFu;
    d.dt = (t.tile_op >> 8) & 0xFFu;
    d.adt = (t.tile_op >> 16) & 0xFFu;
    const uint32_t raw[8] = {t.p0, t.p1, t.p2, t.p3, t.p4, t.p5, t.p6, t.p7};
    std::memcpy(d.p, raw, sizeof(raw));
    d.ptr[0] = c.Ref(t.dst);
    d.ptr[1] = c.Ref(t.a);
    d.ptr[2] = c.Ref(t.b);
    auto fail_unimpl = [&](const std::string &m) {
      *err = "task " + std::to_string(ti) + ": " + m;
      *unimplemented = true;
      return false;
    };
    switch (d.op) {
      case kTopEw: {
        const uint32_t sub = t.p0;
        if (sub > kSubMax) return fail_unimpl("unknown elementwise subop " + std::to_string(sub));
        if (sub == kSelect) d.ptr[3] = c.Ref(t.p3);
        const bool viewable = IsBin(sub) || IsUn(sub);
        DView views[2];
        std::memset(views, 0, sizeof(views));
        if (viewable && t.p2) {
          if (!ViewFromAux(p, t.p2 - 1, &views[0], err)) return fail_unimpl(*err);
          d.flags |= kViewA;
        }
        if (viewable && IsBin(sub) && t.p3) {
          if (!ViewFromAux(p, t.p3 - 1, &views[1], err)) return fail_unimpl(*err);
          d.flags |= kViewB;
        }
        if (d.flags & (kViewA | kViewB)) d.desc = c.PushDesc(views);
        bool vec = !Wide(d.dt) && !Wide(d.adt) && c.Aligned16(t.dst);
        if (EwReadsA(sub)) vec = vec && c.Aligned16(t.a);
        if (EwReadsB(sub)) vec = vec && c.Aligned16(t.b);
        if (sub == kSelect) vec = vec && c.Aligned16(t.p3);
        if (vec) d.flags |= kVecPath;
        break;
      }
      case kTopGather: case kTopScatter: case kTopDynGather: case kTopDynScatter: {
        DMove m;
        std::memset(&m, 0, sizeof(m));
        const bool dyn = d.op == kTopDynGather || d.op == kTopDynScatter;
        const uint32_t x = t.p0;
        const int32_t rank = p.aux[x];
        const size_t need = dyn ? 2 + 5 * static_cast<size_t>(rank) : 2 + 2 * static_cast<size_t>(rank);
        if (rank < 0 || x + need > p.aux.size()) { *err = "move descriptor out of the aux pool"; return false; }
        if (!CollapseView(&p.aux[x + 1], &p.aux[x + 1 + rank], rank, dyn ? 0 : p.aux[x + 1 + 2 * rank], &m.view))
          return fail_unimpl("access map does not collapse");
        m.esz = static_cast<uint32_t>(DtypeSize(d.dt));
        if (dyn) {
          if (rank > 8) return fail_unimpl("dynamic slice of rank > 8");
          m.n_idx = static_cast<uint32_t>(rank);
          m.is64 = static_cast<uint32_t>(p.aux[x + 1 + 5 * rank]);
          for (int32_t k = 0; k < rank; ++k) {
            m.idx_stride[k] = p.aux[x + 1 + rank + k];
            m.clamp_max[k] = p.aux[x + 1 + 2 * rank + k];
            const uint32_t id = static_cast<uint32_t>(p.aux[x + 1 + 4 * rank + k]);
            if (id >= p.buffers.size()) { *err = "dynamic slice index buffer id out of range"; return false; }
            m.idx_ptr[k] = c.Ref(id);
          }
        }
        // 16-byte chunks: the strided side's innermost run is contiguous, a whole
        // number of chunks, and every chunk start is chunk-aligned on both sides.
        const uint32_t chunk = 16u / m.esz;
        const DView &v = m.view;
        bool ok = c.Aligned16(t.dst) && c.Aligned16(t.a) && v.rank >= 1 && v.stride[v.rank - 1] == 1 &&
                  v.dim[v.rank - 1] % chunk == 0 && v.off % chunk == 0;
        for (int k = 0; ok && k < v.rank - 1; ++k) ok = v.stride[k] % static_cast<int32_t>(chunk) == 0;
        m.chunk = ok ? chunk : 0u;
        // a transpose: dst[..., r, c] = src[... + r + c * ld], 2- or 4-byte elements
        m.transposed = (d.op == kTopGather && !m.chunk && (m.esz == 2 || m.esz == 4) && v.rank >= 2 &&
                        v.stride[v.rank - 2] == 1 && v.stride[v.rank - 1] > 1 && v.dim[v.rank - 1] >= 32 &&
                        v.dim[v.rank - 2] >= 8) ? 1u : 0u;
        d.desc = c.PushDesc(m);
        break;
      }
      case kTopIotaDim: {
        const uint32_t x = t.p0;
        const int32_t rank = p.aux[x];
        if (rank < 0 || x + 2 + static_cast<size_t>(rank) > p.aux.size()) { *err = "iota descriptor out of the aux pool"; return false; }
        uint32_t words[2] = {0u, 1u};
        if (rank > 0) {
          const int32_t dim = p.aux[x + 1 + rank];
          if (dim < 0 || dim >= rank) { *err = "iota dimension out of range"; return false; }
          uint64_t inner = 1;
          for (int32_t k = dim + 1; k < rank; ++k) inner *= static_cast<uint32_t>(p.aux[x + 1 + k]);
          words[0] = static_cast<uint32_t>(p.aux[x + 1 + dim]);
          words[1] = static_cast<uint32_t>(inner);
        }
        d.desc = c.PushDesc(words);
        break;
      }
      case kTopMapRegion: {
        const uint32_t x = t.p0;
        if (x + 3 > p.aux.size()) { *err = "region descriptor out of the aux pool"; return false; }
        const uint32_t n_in = static_cast<uint32_t>(p.aux[x]), n_micro = static_cast<uint32_t>(p.aux[x + 2]);
        if (n_in > 8 || n_micro > 96 || x + 3 + n_in + 6ull * n_micro > p.aux.size())
          return fail_unimpl("map-region descriptor exceeds 8 inputs / 96 micro-ops");
        DRegion r;
        const uint32_t ids[8] = {t.a, t.b, t.p2, t.p3, t.p4, t.p5, t.p6, t.p7};
        bool vec = !Wide(d.dt) && !Wide(d.adt) && c.Aligned16(t.dst);
        for (int k = 0; k < 8; ++k) {
          r.in[k] = c.Ref(ids[k]);
          if (static_cast<uint32_t>(k) < n_in) vec = vec && c.Aligned16(ids[k]);
        }
        if (vec) d.flags |= kVecPath;
        d.desc = c.PushDesc(r);
        break;
      }
      case kTopMma: {
        DMma m;
        std::memset(&m, 0, sizeof(m));
        if (t.p4) {
          if (!ViewFromAux(p, t.p4 - 1, &m.va, err)) return fail_unimpl(*err);
          d.flags |= kViewA;
        }
        if (t.p5) {
          if (!ViewFromAux(p, t.p5 - 1, &m.vb, err)) return fail_unimpl(*err);
          d.flags |= kViewB;
        }
        if (t.p6) {
          d.ptr[3] = c.Ref(t.p7);
          d.cdt = p.buffers[t.p7].dtype;
          const uint32_t e = t.p6 - 1;
          if (e >= p.aux.size() || e + 1 + 4ull * static_cast<uint32_t>(p.aux[e]) > p.aux.size()) {
            *err = "matmul epilogue descriptor out of the aux pool";
            return false;
          }
        }
        // tensor-core eligibility: 16-bit float operands in a directly loadable layout
        if (d.adt == kBF16 || d.adt == kF16) {
          const int64_t M = t.p0, N = t.p1, K = t.p2, G = t.p3 ? t.p3 : 1;
          int64_t sa[3] = {M * K, K, 1}, sb[3] = {K * N, N, 1}, oa = 0, ob = 0;
          bool ok = M > 0 && N > 0 && K > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31);
          const int64_t na[3] = {G, M, K}, nb[3] = {G, K, N};
          if (ok && t.p4) ok = AffineOverAxes(m.va, na, sa, &oa);
          if (ok && t.p5) ok = AffineOverAxes(m.vb, nb, sb, &ob);
          if (G == 1) sa[0] = sb[0] = 0;
          bool amn = false, bmn = false;
          ok = ok && TcOperand(M, K, sa[0], sa[1], sa[2], oa, &amn, &m.a_ld, &m.a_gs);
          ok = ok && TcOperand(N, K, sb[0], sb[2], sb[1], ob, &bmn, &m.b_ld, &m.b_gs);
          if (ok) {
            m.a_off = oa;
            m.b_off = ob;
            m.tc_mode = kTcOk | (amn ? kTcAmn : 0u) | (bmn ? kTcBmn : 0u);
            ++out->n_mma_tc;
            m.tmap = static_cast<int32_t>(out->tmaps.size());
            out->tmaps.push_back(TmapSpec{d.ptr[1], oa, d.adt, amn, M, K, G, m.a_ld, m.a_gs, 0u});
            out->tmaps.push_back(TmapSpec{d.ptr[2], ob, d.adt, bmn, N, K, G, m.b_ld, m.b_gs, 0u});
          }
        }
        if (!(m.tc_mode & kTcOk)) m.tmap = -1;
        ++out->n_mma;
        out->mma_flops += 2ull * (t.p3 ? t.p3 : 1u) * t.p0 * static_cast<uint64_t>(t.p1) * t.p2;
        d.desc = c.PushDesc(m);
        if (m.tc_mode & kTcOk) {
          out->tmaps[m.tmap].desc_word = d.desc;
          out->tmaps[m.tmap + 1].desc_word = d.desc;
        }
        break;
      }
      case kTopFlashAttn: {
        DFlash f;
        std::memset(&f, 0, sizeof(f));
        d.ptr[3] = c.Ref(t.p0);
        const int32_t *x = &p.aux[t.p3];
        if (x[3] > 256) return fail_unimpl("flash-attention head_dim > 256");
        const uint32_t qv = static_cast<uint32_t>(x[6]), kv = static_cast<uint32_t>(x[7]), vv = static_cast<uint32_t>(x[8]);
        if (qv) { if (!ViewFromAux(p, qv - 1, &f.vq, err)) return fail_unimpl(*err); f.has_q = 1; }
        if (kv) { if (!ViewFromAux(p, kv - 1, &f.vk, err)) return fail_unimpl(*err); f.has_k = 1; }
        if (vv) { if (!ViewFromAux(p, vv - 1, &f.vv, err)) return fail_unimpl(*err); f.has_v = 1; }
        // tensor-core eligibility: 16-bit floats, plain operands, head_dim 64, 16-byte friendly rows
        if ((d.adt == kBF16 || d.adt == kF16) && (d.dt == kBF16 || d.dt == kF16 || d.dt == kF32) && !qv && !kv && !vv &&
            x[3] == 64 && x[2] % 8 == 0 && x[1] >= 16 && x[2] > 0) {
          f.tc_mode = 1;
          ++out->n_flash_tc;
        }
        ++out->n_flash;
        d.desc = c.PushDesc(f);
        break;
      }
      case kTopRedPart: case kTopRedComb: case kTopRedSeg: case kTopRedStrided:
      case kTopSoftmaxSeg: case kTopLayernormSeg:
        break;
      default:
        return fail_unimpl("tile op " + std::to_string(d.op) + " is not implemented by this backend");
    }
  }

  // ---- entries: resolve control cond buffers ----
  out->entries.resize(p.entries.size());
  for (size_t i = 0; i < p.entries.size(); ++i) {
    const VmEntry &e = p.entries[i];
    DEntry &d = out->entries[i];
    std::memset(&d, 0, sizeof(d));
    d.task = e.task; d.tile_lo = e.tile_lo; d.tile_hi = e.tile_hi;
    const bool control = e.task == kEntWhile || e.task == kEntIf || e.task == kEntFor;
    if (control) { d.a = e.wait_flag; d.b = e.wait_count; }   // tile entries: the reserved words stay 0
    if (e.task == kEntWhile || e.task == kEntIf) d.cond = c.Ref(e.signal_flag);
  }

  // ---- fused elementwise chains ----
  // A chain = consecutive entries of one lane, all TILE_EW, same tile range, same
  // element count (what scheduler.py:552-578 emits for a lane-local unit).
  auto is_ew = [&](const VmEntry &e) { return e.task < p.tasks.size() && (p.tasks[e.task].tile_op & 0xFFu) == kTopEw; };
  constexpr int kNone = -1, kConflict = -2, kUnset = -3;
  std::vector<int> pred(p.tasks.size(), kUnset), succ(p.tasks.size(), kUnset);
  auto note = [&](std::vector<int> &m, uint32_t task, int v) {
    if (m[task] == kUnset) m[task] = v;
    else if (m[task] != v) m[task] = kConflict;
  };
  for (const VmLane &l : p.lane_tab) {
    uint32_t i = l.off;
    const uint32_t end = l.off + l.count;
    // A chain must stay inside one control range: the root walk and every
    // cond / body / branch range are contiguous in the stream, so consecutive
    // entries can belong to different frames.
    std::set<uint32_t> cuts;
    cuts.insert(l.off + l.root_len);
    for (uint32_t e = l.off; e < end; ++e) {
      const VmEntry &en = p.entries[e];
      if (en.task == kEntWhile || en.task == kEntIf || en.task == kEntFor) {
        cuts.insert(l.off + en.tile_lo);
        cuts.insert(l.off + en.tile_lo + en.tile_hi);
        if (en.task != kEntFor) {
          cuts.insert(l.off + en.wait_flag);
          cuts.insert(l.off + en.wait_flag + en.wait_count);
        }
      }
    }
    while (i < end) {
      if (!is_ew(p.entries[i])) { ++i; continue; }
      uint32_t j = i + 1;
      while (j < end && !cuts.count(j) && j - i < static_cast<uint32_t>(8) && is_ew(p.entries[j]) &&
             p.entries[j].tile_lo == p.entries[i].tile_lo && p.entries[j].tile_hi == p.entries[i].tile_hi &&
             p.tasks[p.entries[j].task].p1 == p.tasks[p.entries[i].task].p1)
        ++j;
      out->entries[i].chain = j - i;
      if (j - i > 1) out->n_chains++;
      for (uint32_t k = i; k < j; ++k) {
        note(pred, p.entries[k].task, k > i ? static_cast<int>(p.entries[k - 1].task) : kNone);
        note(succ, p.entries[k].task, k + 1 < j ? static_cast<int>(p.entries[k + 1].task) : kNone);
      }
      i = j;
    }
  }
  // readers of every buffer, by task; plus buffers something other than a task reads
  std::vector<std::set<uint32_t>> readers(p.buffers.size());
  for (size_t ti = 0; ti < p.tasks.size(); ++ti) {
    std::vector<uint32_t> r;
    TaskReads(p, p.tasks[ti], &r);
    for (uint32_t id : r)
      if (id < p.buffers.size()) readers[id].insert(static_cast<uint32_t>(ti));
  }
  std::set<uint32_t> pinned(p.results.ids.begin(), p.results.ids.end());
  for (const VmEntry &e : p.entries)
    if (e.task == kEntWhile || e.task == kEntIf) pinned.insert(e.signal_flag);
  // Two buffer ids may share arena bytes (liveness reuse, lowering.py:2813-2973).
  // A reader of another id never observes this id's value: every id is written
  // before it is read, so elision is decided per id.
  for (size_t ti = 0; ti < p.tasks.size(); ++ti) {
    const int pr = pred[ti];
    if (pr < 0) continue;
    const VmTask &cur = p.tasks[ti], &prev = p.tasks[pr];
    DTask &dc = out->tasks[ti], &dp = out->tasks[pr];
    if (!(dc.flags & kVecPath) || !(dp.flags & kVecPath)) continue;
    if (succ[pr] != static_cast<int>(ti)) continue;
    // every member of every chain these tasks sit in must be on the vector path;
    // the device checks that per chain and otherwise ignores nothing - so only
    // forward when the whole neighbourhood is vector-capable.
    const uint32_t sub = cur.p0;
    const bool viewable = IsBin(sub) || IsUn(sub);
    bool fa = EwReadsA(sub) && cur.a == prev.dst && !(viewable && cur.p2);
    bool fb = EwReadsB(sub) && cur.b == prev.dst && !(viewable && IsBin(sub) && cur.p3);
    if (prev.p0 == kLts) fa = fb = false;   // LTS writes one element only
    if (!fa && !fb) continue;
    if (fa) { dc.flags |= kFwdA; out->n_forwarded++; }
    if (fb) { dc.flags |= kFwdB; out->n_forwarded++; }
    // dead store: cur is the only reader, reads it only through forwarded operands
    bool other_use = (EwReadsA(sub) && cur.a == prev.dst && !fa) || (EwReadsB(sub) && cur.b == prev.dst && !fb) ||
                     (sub == kSelect && cur.p3 == prev.dst);
    const auto &rs = readers[prev.dst];
    if (!other_use && !pinned.count(prev.dst) && rs.size() == 1 && *rs.begin() == ti &&
        !in_ids.count(prev.dst) && !const_ids.count(prev.dst)) {
      dp.flags |= kDeadStore;
      out->n_dead_stores++;
    }
  }
  // The device runs a chain on the vector path only if ALL members are vector-
  // capable; forwarding flags are meaningless otherwise, so clear them on chains
  // that contain a non-vector member.
  for (const VmLane &l : p.lane_tab) {
    for (uint32_t i = l.off; i < l.off + l.count; ++i) {
      const uint32_t n = out->entries[i].chain;
      if (n <= 1) continue;
      bool vec = true;
      for (uint32_t k = i; k < i + n; ++k) vec = vec && (out->tasks[p.entries[k].task].flags & kVecPath);
      if (!vec)
        for (uint32_t k = i; k < i + n; ++k)
          out->tasks[p.entries[k].task].flags &= ~(kFwdA | kFwdB | kDeadStore);
      i += n - 1;
    }
  }
  out->lanes = p.lane_tab;
  SpreadStridedReductions(p, out);
  return true;
}

}  // namespace b2
