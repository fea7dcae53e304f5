// Builds the device tables for one program. See loader.h.
#include "loader.h"

#include <algorithm>
#include <cstdlib>
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
    case kTopGatherIndex: case kTopScatterIndex:
      r->push_back(t.a);
      if (static_cast<size_t>(t.p0) + 5 < p.aux.size()) r->push_back(static_cast<uint32_t>(p.aux[t.p0 + 5]));
      if (op == kTopScatterIndex) r->push_back(t.dst);  // combines into / partially overwrites what is there
      break;
    case kTopRedWindow:
      r->push_back(t.a);
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

// Does every index an access map can produce fall inside a buffer of `n_elems` elements?
// `slack` is the largest dynamic start offset (dynamic slices: sum of clamp_max x index stride).
// A malformed blob must fail on the host, not fault on the device.
bool AccessInside(const int32_t *dims, const int32_t *strides, int rank, int64_t off, int64_t slack, uint64_t n_elems) {
  int64_t lo = off, hi = off + slack;
  for (int k = 0; k < rank; ++k) {
    if (dims[k] <= 0) return true;                       // an empty index space touches nothing
    const int64_t span = static_cast<int64_t>(dims[k] - 1) * strides[k];
    if (span < 0) lo += span; else hi += span;
  }
  return lo >= 0 && static_cast<uint64_t>(hi) < n_elems;
}

// The view at aux[aux_off] (rank, dims, strides, offset), read from buffer `buf` as elements of `dtype`.
bool ViewInsideBuffer(const VmProgram &p, uint32_t aux_off, uint32_t buf, uint32_t dtype, std::string *err) {
  const int32_t rank = p.aux[aux_off];
  const uint64_t n = buf < p.buffers.size() ? p.buffers[buf].bytes / std::max<uint64_t>(1, DtypeSize(dtype)) : 0;
  if (AccessInside(&p.aux[aux_off + 1], &p.aux[aux_off + 1 + rank], rank, p.aux[aux_off + 1 + 2 * rank], 0, n)) return true;
  *err = "operand view reaches outside buffer " + std::to_string(buf) + " (" + std::to_string(n) + " elements)";
  return false;
}

// Is the view, read over the row-major flat index of a [n0, n1, n2] tensor, affine
// in the three coordinates? The view's (collapsed) dims and [n0, n1, n2] are two
// factorisations of the same index space; walk their common refinement from the
// innermost digit and require every piece of one coordinate to agree on that
// coordinate's stride.
bool AffineOverAxesN(const DView &v, const int64_t *n, int naxes, int64_t *stride, int64_t *off) {
  *off = v.off;
  bool have[8] = {false, false, false, false, false, false, false, false};
  for (int k = 0; k < naxes; ++k) stride[k] = 0;
  int a = naxes - 1, j = v.rank - 1;
  int64_t ra = n[a], wa = 1, rv = j >= 0 ? v.dim[j] : 1, wv = 1;
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
bool AffineOverAxes(const DView &v, const int64_t n[3], int64_t stride[3], int64_t *off) {
  return AffineOverAxesN(v, n, 3, stride, off);
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

// The same pass re-cuts a full reduction (RED_PART whose partials only its RED_COMB
// reads; `fused_comb[task]` = that RED_COMB) over all lanes: the scheduler's
// ceil(n / chunk) partial tiles rarely divide evenly by the lane count (config 2:
// 256 tiles on 148 lanes, so 108 lanes reduce twice what the other 40 do), and the
// combine is a serial phase of its own. Re-cut, every lane reduces an equal share
// of 16-byte words (DEntry::a, b), leaves its total in the program's scratch, and
// the lane that arrives last folds the lanes' totals in lane order into the
// RED_COMB's result; the RED_COMB entry becomes a NOP.
// After entries of a chain were turned into no-ops: the chain closes up over the gaps, live members first, the
// count on the new head.
void CompactChains(DeviceTables *out) {
  for (const VmLane &l : out->lanes)
    for (uint32_t i = l.off; i < l.off + l.count; ++i) {
      const uint32_t n = out->entries[i].chain;
      if (n <= 1u) continue;
      uint32_t live = 0;
      for (uint32_t k = i; k < i + n; ++k)
        if (out->entries[k].task != kEntNop) {
          DEntry m = out->entries[k];
          out->entries[k].task = kEntNop;
          out->entries[i + live++] = m;
        }
      for (uint32_t k = i; k < i + n; ++k) out->entries[k].chain = 0u;
      if (live) out->entries[i].chain = live;
      i += n - 1u;
    }
}

void SpreadReductions(const VmProgram &p, const std::vector<int> &fused_comb, const std::vector<int> &half_src, Ctx *cx,
                      DeviceTables *out) {
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
        const uint32_t eop = p.tasks[en.task].tile_op & 0xFFu;
        if (!(eop == kTopRedStrided || (eop == kTopRedPart && fused_comb[en.task] >= 0))) { ++others; continue; }
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
    const bool full = (t.tile_op & 0xFFu) == kTopRedPart;
    int64_t rows;   // units split over the lanes: rows of a strided reduction, 16-byte words of a full one
    if (full) {
      const uint64_t nt = (static_cast<uint64_t>(t.p0) + t.p1 - 1) / t.p1;
      if (tiles != nt) continue;
      rows = half_src[task] >= 0 ? t.p0 / 8 : t.p0 / 4;     // 16-byte words of the stream
    } else {
      const int64_t n_out = t.p0, red = t.p1, inner = t.p2;
      if (!red_strided_rows_ok(dt, red, inner, t.p3) || n_out % inner != 0) continue;
      const uint64_t nt = (static_cast<uint64_t>(n_out) + kEwTs - 1) / kEwTs;
      if (tiles != nt || nt * 2 > n_lanes) continue;
      rows = n_out / inner;
    }
    for (uint32_t l = 0; l < n_lanes; ++l) {
      const StreamRun &r = runs[l][k];
      for (uint32_t i = r.start; i < r.end; ++i)
        if (p.entries[p.lane_tab[l].off + i].task == static_cast<uint32_t>(task)) out->entries[p.lane_tab[l].off + i].task = kEntNop;
      const int64_t lo = rows * l / n_lanes, hi = rows * (l + 1) / n_lanes;
      if (hi <= lo && !full) continue;   // a full reduction counts every lane in, also one with nothing to add
      DEntry e;
      std::memset(&e, 0, sizeof(e));
      e.task = static_cast<uint32_t>(task);
      e.a = static_cast<uint32_t>(lo);
      e.b = static_cast<uint32_t>(hi);
      const bool empty_at_start = r.start == r.end && r.at_range_start;
      ins[l].push_back({r.end, empty_at_start, e});
    }
    if (full) {
      DTask &dp = out->tasks[task];
      const int comb = fused_comb[task];
      dp.flags |= kRedFused;
      dp.ptr[3] = out->tasks[comb].ptr[0];        // where the RED_COMB would have put the result
      if (half_src[task] >= 0) {
        // the convert that fed this reduction is folded in: stream its 16-bit source, never write the f32 copy
        const VmTask &cv = p.tasks[half_src[task]];
        dp.ptr[1] = cx->Ref(cv.a);
        dp.flags |= ((cv.tile_op >> 16) & 0xFFu) == kBF16 ? kRedSrcBf16 : kRedSrcF16;
        for (DEntry &e : out->entries)
          if (e.task == static_cast<uint32_t>(half_src[task])) e.task = kEntNop;
        CompactChains(out);
        out->n_folded_converts++;
      }
      for (DEntry &e : out->entries)
        if (e.task == static_cast<uint32_t>(comb)) e.task = kEntNop;
      out->n_fused_reduce++;
      out->needs_scratch = true;
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

// Branch-free division by d >= 2 for every 32-bit n: q = umulhi(n, magic);
// (((n - q) >> 1) + q) >> shift.
void MagicDivider(uint32_t d, uint32_t *magic, uint32_t *shift) {
  uint32_t sh = 31;
  while (!(d >> sh)) --sh;                        // floor(log2(d))
  if ((d & (d - 1)) == 0) {
    *magic = 0;
    *shift = sh - 1;
    return;
  }
  const unsigned __int128 two = static_cast<unsigned __int128>(1) << (32 + sh);
  uint64_t m = static_cast<uint64_t>(two / d);
  const uint64_t rem = static_cast<uint64_t>(two - static_cast<unsigned __int128>(m) * d);
  m *= 2;
  if (rem * 2 >= d) m += 1;
  *magic = static_cast<uint32_t>(m + 1);
  *shift = sh;
}

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
    MagicDivider(out->dim[k], &out->magic[k], &out->shift[k]);   // dim >= 2 here: size-1 axes were dropped
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

// ---- re-cutting phases whose units differ in cost per tile ----
//
// The scheduler packs a phase's units onto lanes by a cost per tile that is one constant per
// tile-op class (scheduler.py:115-156, 396-432): a matmul tile with K = 8192 counts like one
// with K = 1024, a GELU-gradient region like a cast. In a phase that mixes such units the
// lanes holding the dear ones finish last by factors (config 3: a weight-gradient matmul
// with K = 8192 on 14 lanes beside a forward matmul with K = 1024 on 109 lanes: 708 us of
// wall time against a median lane at 129 us). Units of one phase are independent of each
// other (entries of different lanes in a phase never depend on one another; entries of one
// lane may, but only as a chain over the SAME tile range), so the loader may hand every lane
// an equal share of every unit instead: no cost model, every lane does a little of each.
// Applied to straight-line programs (no control entries), to phases of elementwise /
// region / matmul units whose cost classes differ; everything else keeps the scheduler's cut.
namespace {
struct RebUnit {
  std::vector<uint32_t> tasks;                        // the chain, in lane order
  std::vector<std::pair<uint32_t, uint32_t>> ranges;  // tile ranges held by the lanes
  VmEntry proto[8];                                   // one original entry per chain task
  uint64_t tiles = 0;
};
}  // namespace

bool RebalancePhases(const VmProgram &p, VmProgram *q, uint32_t *n_done, uint32_t *n_piped_out) {
  const uint32_t L = static_cast<uint32_t>(p.lane_tab.size());
  *n_done = 0;
  *n_piped_out = 0;
  if (L < 4) return false;
  for (const VmEntry &e : p.entries)
    if (e.task == kEntWhile || e.task == kEntIf || e.task == kEntFor) return false;
  std::vector<std::vector<std::vector<VmEntry>>> ph(L);   // lane -> phase -> tile entries
  for (uint32_t l = 0; l < L; ++l) {
    const VmLane &ln = p.lane_tab[l];
    if (ln.root_len != ln.count) return false;
    ph[l].emplace_back();
    for (uint32_t i = 0; i < ln.count; ++i) {
      const VmEntry &e = p.entries[ln.off + i];
      if (e.task == kEntBarrier) { ph[l].emplace_back(); continue; }
      if (e.task == kEntNop) continue;
      if (e.task >= p.tasks.size()) return false;
      ph[l].back().push_back(e);
    }
    if (ph[l].size() != ph[0].size()) return false;
  }
  // ---- row pipelines ----
  // Neighbouring phases that each hold ONE unit working row by row on rows of exactly one elementwise tile
  // (LAYERNORM_SEG / SOFTMAX_SEG with a segment of kEwTs elements, elementwise chains over rows x kEwTs
  // elements), cut the same way over the lanes, each reading its predecessor's result at the same index: row r
  // of a later unit needs row r of the earlier one and nothing else that the group writes. The grid barriers
  // between them order nothing the lane's own program order does not, so they go; optionally (B2VM_ROW_BLOCK)
  // the lane walks its rows in blocks - unit 1, unit 2, unit 3 on block 0, then block 1, ... - so that a block's
  // intermediates are read back from L2 instead of HBM. Refused whenever a result's memory overlaps anything a unit of the group
  // reads through a view or under another buffer id (arena slots are reused).
  uint32_t n_piped = 0;
  {
    struct One { std::vector<uint32_t> tasks; bool ok; };
    auto unit_of_phase = [&](size_t k) {
      One u{{}, true};
      bool any = false;
      for (uint32_t l = 0; l < L && u.ok; ++l) {
        const auto &es = ph[l][k];
        if (es.empty()) continue;
        std::vector<uint32_t> key;
        for (const VmEntry &e : es) {
          const VmTask &t = p.tasks[e.task];
          const uint32_t op = t.tile_op & 0xFFu;
          if (e.tile_lo != es[0].tile_lo || e.tile_hi != es[0].tile_hi) u.ok = false;
          if (op == kTopEw) {
            if (t.p0 == kSelect || t.p1 % kEwTs != 0u) u.ok = false;
          } else if (op == kTopSoftmaxSeg || op == kTopLayernormSeg) {
            if (t.p1 != kEwTs || es.size() != 1u) u.ok = false;
          } else {
            u.ok = false;
          }
          key.push_back(e.task);
        }
        if (!any) { u.tasks = key; any = true; }
        else if (u.tasks != key) u.ok = false;
      }
      if (!any) u.ok = false;
      return u;
    };
    auto n_tiles = [&](uint32_t ti) {
      const VmTask &t = p.tasks[ti];
      return (t.tile_op & 0xFFu) == kTopEw ? t.p1 / kEwTs : t.p0;
    };
    auto overlap = [&](uint32_t x, uint32_t y) {
      const BufferSlot &bx = p.buffers[x], &by = p.buffers[y];
      return bx.bytes && by.bytes && bx.offset < by.offset + by.bytes && by.offset < bx.offset + bx.bytes;
    };
    struct Read { uint32_t buf; bool viewed; };
    auto reads_of = [&](uint32_t ti, std::vector<Read> *r) {
      const VmTask &t = p.tasks[ti];
      if ((t.tile_op & 0xFFu) != kTopEw) { r->push_back({t.a, false}); return; }
      if (EwReadsA(t.p0)) r->push_back({t.a, t.p2 != 0u});
      if (EwReadsB(t.p0)) r->push_back({t.b, t.p3 != 0u});
    };
    const char *rb_env = std::getenv("B2VM_ROW_BLOCK");
    // Rows per block. Measured on config 2 (55 rows of 16 KB per lane): every extra block costs ~9 us per unit in
    // fill, drain and entry set-up, more than the L2 hits return (one block 224 us, two 252 us, four 279 us against
    // 235 us with the barriers in place), so by default a lane's whole range is one block and only the barriers go.
    const uint32_t row_block = rb_env ? static_cast<uint32_t>(std::max(1, std::atoi(rb_env))) : 0x7fffffffu;
    size_t k = 0;
    while (k + 1 < ph[0].size()) {
      // the longest run of phases k, k + 1, ... that form one pipeline
      std::vector<One> grp;
      grp.push_back(unit_of_phase(k));
      size_t n = 1;
      while (grp[0].ok && k + n < ph[0].size()) {
        One nx = unit_of_phase(k + n);
        bool ok = nx.ok && n_tiles(nx.tasks[0]) == n_tiles(grp[0].tasks[0]);
        for (uint32_t l = 0; l < L && ok; ++l) {          // the same cut on every lane
          const auto &ea = ph[l][k], &eb = ph[l][k + n];
          if (ea.empty() != eb.empty()) ok = false;
          else if (!ea.empty() && (ea[0].tile_lo != eb[0].tile_lo || ea[0].tile_hi != eb[0].tile_hi)) ok = false;
        }
        if (ok) {
          std::vector<uint32_t> all;
          for (const One &g : grp) all.insert(all.end(), g.tasks.begin(), g.tasks.end());
          all.insert(all.end(), nx.tasks.begin(), nx.tasks.end());
          std::vector<Read> rd;
          for (uint32_t ti : all) reads_of(ti, &rd);
          // two ids on exactly the same bytes (a reused arena slot) and the same element size behave like one
          // buffer here: every access in the group is row-local
          auto same_bytes = [&](uint32_t x, uint32_t y) {
            return x == y || (p.buffers[x].offset == p.buffers[y].offset && p.buffers[x].bytes == p.buffers[y].bytes &&
                              DtypeSize(p.buffers[x].dtype) == DtypeSize(p.buffers[y].dtype));
          };
          for (size_t i = 0; i < all.size() && ok; ++i) {
            const uint32_t d = p.tasks[all[i]].dst;
            for (const Read &r : rd)
              if (overlap(d, r.buf) && (!same_bytes(r.buf, d) || r.viewed)) ok = false;
            for (size_t j = 0; j < all.size(); ++j)
              if (j != i && overlap(d, p.tasks[all[j]].dst) && !same_bytes(d, p.tasks[all[j]].dst)) ok = false;
          }
        }
        if (!ok) break;
        grp.push_back(nx);
        ++n;
      }
      if (n < 2) { ++k; continue; }
      for (uint32_t l = 0; l < L; ++l) {
        if (ph[l][k].empty()) { for (size_t i = 1; i < n; ++i) ph[l].erase(ph[l].begin() + static_cast<long>(k) + 1); continue; }
        const uint32_t lo = ph[l][k][0].tile_lo, hi = ph[l][k][0].tile_hi;
        std::vector<VmEntry> merged;
        for (uint64_t b0 = lo; b0 < hi; b0 += row_block) {
          const uint32_t b1 = static_cast<uint32_t>(std::min<uint64_t>(hi, b0 + row_block));
          for (size_t i = 0; i < n; ++i)
            for (VmEntry e : ph[l][k + i]) { e.tile_lo = static_cast<uint32_t>(b0); e.tile_hi = b1; merged.push_back(e); }
        }
        ph[l][k] = merged;
        for (size_t i = 1; i < n; ++i) ph[l].erase(ph[l].begin() + static_cast<long>(k) + 1);
      }
      ++n_piped;
      ++k;
    }
  }
  const size_t n_ph = ph[0].size();
  auto cost_class = [&](const RebUnit &u) {
    const VmTask &t = p.tasks[u.tasks[0]];
    const uint32_t op = t.tile_op & 0xFFu;
    // matmuls: by K (p2) and batch; regions: by program length (p0 is the aux offset: use the task id, regions differ);
    // elementwise: by chain length
    if (op == kTopMma) return (static_cast<uint64_t>(1) << 60) | (static_cast<uint64_t>(t.p2) << 8) | (t.p3 & 0xFFu);
    if (op == kTopMapRegion) return (static_cast<uint64_t>(2) << 60) | u.tasks[0];
    return (static_cast<uint64_t>(3) << 60) | u.tasks.size();
  };
  for (size_t k = 0; k < n_ph; ++k) {
    std::vector<RebUnit> units;
    std::map<uint32_t, size_t> unit_of;     // task -> unit
    bool ok = true;
    for (uint32_t l = 0; l < L && ok; ++l) {
      const auto &es = ph[l][k];
      for (size_t i = 0; i < es.size() && ok;) {
        size_t j = i + 1;
        while (j < es.size() && es[j].tile_lo == es[i].tile_lo && es[j].tile_hi == es[i].tile_hi && es[j].task != es[i].task) ++j;
        if (j - i > 8) { ok = false; break; }
        std::vector<uint32_t> key;
        for (size_t x = i; x < j; ++x) key.push_back(es[x].task);
        auto it = unit_of.find(key[0]);
        size_t ui;
        if (it == unit_of.end()) {
          for (uint32_t t : key) if (unit_of.count(t)) ok = false;
          if (!ok) break;
          ui = units.size();
          units.emplace_back();
          units[ui].tasks = key;
          for (size_t x = i; x < j; ++x) { units[ui].proto[x - i] = es[x]; unit_of[es[x].task] = ui; }
        } else {
          ui = it->second;
          if (units[ui].tasks != key) { ok = false; break; }
        }
        if (es[i].tile_hi > es[i].tile_lo) units[ui].ranges.push_back({es[i].tile_lo, es[i].tile_hi});
        i = j;
      }
    }
    if (!ok || units.size() < 2) continue;
    bool differ = false;
    for (RebUnit &u : units) {
      for (uint32_t t : u.tasks) {
        const uint32_t op = p.tasks[t].tile_op & 0xFFu;
        if (!(op == kTopEw || op == kTopMapRegion || op == kTopMma)) ok = false;
      }
      std::sort(u.ranges.begin(), u.ranges.end());
      uint32_t at = 0;
      for (const auto &r : u.ranges) { if (r.first != at) ok = false; at = r.second; }   // an exact partition of [0, tiles)
      u.tiles = at;
      if (!u.tiles) ok = false;
      if (cost_class(u) != cost_class(units[0])) differ = true;
    }
    if (!ok || !differ) continue;
    for (uint32_t l = 0; l < L; ++l) {
      auto &es = ph[l][k];
      es.clear();
      for (const RebUnit &u : units) {
        const uint32_t lo = static_cast<uint32_t>(u.tiles * l / L), hi = static_cast<uint32_t>(u.tiles * (l + 1) / L);
        if (hi <= lo) continue;
        for (size_t x = 0; x < u.tasks.size(); ++x) {
          VmEntry e = u.proto[x];
          e.tile_lo = lo; e.tile_hi = hi;
          es.push_back(e);
        }
      }
    }
    ++*n_done;
  }
  if (!*n_done && !n_piped) return false;
  *n_piped_out = n_piped;
  *q = p;
  q->entries.clear();
  VmEntry bar;
  std::memset(&bar, 0, sizeof(bar));
  bar.task = kEntBarrier; bar.wait_flag = 0xFFFFFFFFu; bar.signal_flag = 0xFFFFFFFFu;
  for (uint32_t l = 0; l < L; ++l) {
    const uint32_t off = static_cast<uint32_t>(q->entries.size());
    for (size_t k = 0; k < n_ph; ++k) {
      if (k) q->entries.push_back(bar);
      for (const VmEntry &e : ph[l][k]) q->entries.push_back(e);
    }
    const uint32_t cnt = static_cast<uint32_t>(q->entries.size()) - off;
    q->lane_tab[l] = VmLane{off, cnt, cnt, 0u};
  }
  return true;
}

static bool BuildDeviceTablesFor(const VmProgram &p, uint64_t arena_base, DeviceTables *out, std::string *err,
                                 bool *unimplemented);

bool BuildDeviceTables(const VmProgram &p, uint64_t arena_base, DeviceTables *out, std::string *err,
                       bool *unimplemented) {
  VmProgram q;
  uint32_t n_reb = 0, n_piped = 0;
  const bool recut = std::getenv("B2VM_NO_REBALANCE") == nullptr && RebalancePhases(p, &q, &n_reb, &n_piped);
  const bool ok = BuildDeviceTablesFor(recut ? q : p, arena_base, out, err, unimplemented);
  out->n_rebalanced = n_reb;
  out->n_row_pipelines = n_piped;
  return ok;
}

static bool BuildDeviceTablesFor(const VmProgram &p, uint64_t arena_base, DeviceTables *out, std::string *err,
                                 bool *unimplemented) {
  *unimplemented = false;
  Ctx c{p, arena_base, {}, out};
  out->desc.assign(1, 0);

  // ---- zero-copy I/O ports (runtime.cc:798-821): a buffer that is only an input
  // or only an output, is not a constant, and is among the first kMaxIoPorts such.
  // Beyond the reference (whose donated buffers fall back to the arena): a buffer that
  // is one argument AND one result and that some task writes - a cache updated in
  // place - is an in/out port: the kernel works on the result's memory, which the
  // argument is copied into first unless the caller passed the same address for both.
  std::set<uint32_t> in_ids(p.args.ids.begin(), p.args.ids.end()), out_ids(p.results.ids.begin(), p.results.ids.end());
  std::set<uint32_t> const_ids;
  for (const auto &k : p.consts) const_ids.insert(k.buffer);
  // A result buffer that no task ever writes (a pass-through of arena-resident
  // data) has to come out of the arena.
  std::set<uint32_t> written;
  for (const VmTask &t : p.tasks) written.insert(t.dst);
  auto times_in = [](const std::vector<uint32_t> &v, uint32_t id) { return std::count(v.begin(), v.end(), id); };
  auto assign_port = [&](uint32_t id) -> int {
    if (in_ids.count(id) && out_ids.count(id) &&
        !(written.count(id) && times_in(p.args.ids, id) == 1 && times_in(p.results.ids, id) == 1))
      return -1;
    if (const_ids.count(id)) return -1;
    auto it = c.port_of.find(id);
    if (it != c.port_of.end()) return it->second;
    if (out->n_ports >= static_cast<int>(kMaxIoPorts)) return -1;
    return c.port_of[id] = out->n_ports++;
  };
  out->input_port.assign(p.args.ids.size(), -1);
  out->output_port.assign(p.results.ids.size(), -1);
  out->inout_result.assign(p.args.ids.size(), -1);
  for (size_t i = 0; i < p.args.ids.size(); ++i) out->input_port[i] = assign_port(p.args.ids[i]);
  for (size_t o = 0; o < p.results.ids.size(); ++o)
    out->output_port[o] = written.count(p.results.ids[o]) ? assign_port(p.results.ids[o]) : -1;
  for (size_t i = 0; i < p.args.ids.size(); ++i) {
    if (out->input_port[i] < 0 || !out_ids.count(p.args.ids[i])) continue;
    for (size_t o = 0; o < p.results.ids.size(); ++o)
      if (p.results.ids[o] == p.args.ids[i]) out->inout_result[i] = static_cast<int>(o);
  }

  // ---- tasks ----
  out->tasks.resize(p.tasks.size());
  for (size_t ti = 0; ti < p.tasks.size(); ++ti) {
    const VmTask &t = p.tasks[ti];
    DTask &d = out->tasks[ti];
    std::memset(&d, 0, sizeof(d));
    d.op = t.tile_op & 0xFFu;
    d.dt = (t.tile_op >> 8) & 0xFFu;
    d.adt = (t.tile_op >> 16) & 0xFFu;
    out->families |= family_of(d.op);
    // the short-run paths (a build of their own, so that programs without such work do not carry them)
    if (d.op == kTopRedSeg && !t.p3 && d.dt == kF32 && d.adt == kF32 && t.p1 >= 2 && t.p1 <= 8) out->families |= kFamShort;
    if (d.op == kTopEw && t.p0 == kPow && d.dt == kF32) out->families |= kFamShort;
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
          if (!ViewInsideBuffer(p, t.p2 - 1, t.a, d.adt, err)) return false;
          if (!views[0].vec_ok && views[0].rank >= 1 && views[0].rank <= 3) out->families |= kFamShort;
          d.flags |= kViewA;
        }
        if (viewable && IsBin(sub) && t.p3) {
          if (!ViewFromAux(p, t.p3 - 1, &views[1], err)) return fail_unimpl(*err);
          if (!ViewInsideBuffer(p, t.p3 - 1, t.b, d.adt, err)) return false;
          if (!views[1].vec_ok && views[1].rank >= 1 && views[1].rank <= 3) out->families |= kFamShort;
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
        {
          // the strided side: the source of a gather, the destination of a scatter
          const uint32_t side = (d.op == kTopGather || d.op == kTopDynGather) ? t.a : t.dst;
          int64_t slack = 0;
          if (dyn) for (int32_t k = 0; k < rank; ++k) slack += static_cast<int64_t>(p.aux[x + 1 + 2 * rank + k]) * p.aux[x + 1 + rank + k];
          const uint64_t n_side = p.buffers[side].bytes / std::max<uint64_t>(1, m.esz);
          const int32_t *mv_strides = &p.aux[x + 1 + rank];
          if (!AccessInside(&p.aux[x + 1], mv_strides, rank, dyn ? 0 : p.aux[x + 1 + 2 * rank], slack, n_side)) {
            *err = "task " + std::to_string(ti) + ": access map reaches outside buffer " + std::to_string(side);
            return false;
          }
        }
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
        if (d.op == kTopGather && !m.chunk && m.esz == 4 && m.view.rank >= 1 && m.view.rank <= 3) out->families |= kFamShort;
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
          if (!ViewInsideBuffer(p, t.p4 - 1, t.a, d.adt, err)) return false;
          d.flags |= kViewA;
        }
        if (t.p5) {
          if (!ViewFromAux(p, t.p5 - 1, &m.vb, err)) return fail_unimpl(*err);
          if (!ViewInsideBuffer(p, t.p5 - 1, t.b, d.adt, err)) return false;
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
            // rank-3 maps {inner, outer, batch}: the inner dimension is the unit-stride one (k for a
            // K-major operand, the row / column index for an MN-major one), boxes of 64 inner elements
            // (one 128-byte swizzle line) x 128 or 64 outer rows
            auto mm_spec = [&](BufRef base, int64_t off, bool mn, int64_t rows, int64_t ld, int64_t gs) {
              TmapSpec sp;
              std::memset(&sp, 0, sizeof(sp));
              sp.base = base; sp.off = off; sp.dtype = d.adt; sp.rank = 3;
              sp.dims[0] = static_cast<uint64_t>(mn ? rows : K);
              sp.dims[1] = static_cast<uint64_t>(mn ? K : rows);
              sp.dims[2] = static_cast<uint64_t>(G);
              sp.strides[0] = ld;
              sp.strides[1] = G > 1 ? gs : ld * static_cast<int64_t>(sp.dims[1]);
              sp.box[0] = 64u; sp.box[1] = mn ? 64u : 128u; sp.box[2] = 1u;
              sp.valid = !(G > 1 && gs <= 0);           // a batch-broadcast operand has no stride to give
              return sp;
            };
            out->tmaps.push_back(mm_spec(d.ptr[1], oa, amn, M, m.a_ld, m.a_gs));
            out->tmaps.push_back(mm_spec(d.ptr[2], ob, bmn, N, m.b_ld, m.b_gs));
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
        if (qv) { if (!ViewFromAux(p, qv - 1, &f.vq, err)) return fail_unimpl(*err); if (!ViewInsideBuffer(p, qv - 1, t.a, d.adt, err)) return false; f.has_q = 1; }
        if (kv) { if (!ViewFromAux(p, kv - 1, &f.vk, err)) return fail_unimpl(*err); if (!ViewInsideBuffer(p, kv - 1, t.b, d.adt, err)) return false; f.has_k = 1; }
        if (vv) { if (!ViewFromAux(p, vv - 1, &f.vv, err)) return fail_unimpl(*err); if (!ViewInsideBuffer(p, vv - 1, t.p0, d.adt, err)) return false; f.has_v = 1; }
        float scale_f;
        std::memcpy(&scale_f, &x[4], 4);
        const bool scale_positive = scale_f > 0.0f && scale_f < 1e30f;   // the row maximum is taken before scaling
        // Tensor-core eligibility: 16-bit floats, head_dim 64, and every operand affine over
        // (h1, h0, row, column) with a unit stride along d (Q, V; K along d or along the keys) and
        // 16-byte friendly outer strides, so that three rank-4 tensor maps describe them.
        f.tmap = -1;
        f.work_slot = kNoWorkSlot;
        if ((d.adt == kBF16 || d.adt == kF16) && (d.dt == kBF16 || d.dt == kF16 || d.dt == kF32) &&
            x[3] == 64 && x[0] > 0 && x[1] >= 16 && x[2] > 0 && c.Aligned16(t.dst) && scale_positive) {
          const int64_t H = x[0], T = x[1], C = x[2];
          for (int64_t h0 = H; h0 >= 1 && !f.tc_mode; --h0) {
            if (H % h0) continue;
            const int64_t nq[4] = {H / h0, h0, T, 64}, nk[4] = {H / h0, h0, 64, C}, nv[4] = {H / h0, h0, C, 64};
            int64_t sq[4] = {h0 * T * 64, T * 64, 64, 1}, sk[4] = {h0 * 64 * C, 64 * C, C, 1}, sv[4] = {h0 * C * 64, C * 64, 64, 1};
            int64_t oq = 0, ok_ = 0, ov = 0;
            bool ok = true;
            if (qv) ok = ok && AffineOverAxesN(f.vq, nq, 4, sq, &oq);
            if (kv) ok = ok && AffineOverAxesN(f.vk, nk, 4, sk, &ok_);
            if (vv) ok = ok && AffineOverAxesN(f.vv, nv, 4, sv, &ov);
            if (H / h0 == 1) sq[0] = sk[0] = sv[0] = 8;   // a size-1 axis: any legal stride
            if (h0 == 1) sq[1] = sk[1] = sv[1] = 8;
            const bool k_dmajor = sk[2] == 1 && sk[3] != 1;          // d contiguous, keys strided
            auto good = [](int64_t st) { return st > 0 && st % 8 == 0; };
            ok = ok && sq[3] == 1 && sv[3] == 1 && (k_dmajor || sk[3] == 1) && oq >= 0 && ok_ >= 0 && ov >= 0 &&
                 oq % 8 == 0 && ok_ % 8 == 0 && ov % 8 == 0 && good(sq[0]) && good(sq[1]) && good(sq[2]) &&
                 good(sk[0]) && good(sk[1]) && good(k_dmajor ? sk[3] : sk[2]) && good(sv[0]) && good(sv[1]) && good(sv[2]);
            if (!ok) continue;
            auto fa_spec = [&](BufRef base, int64_t off, uint64_t inner, uint64_t rows, int64_t s_row, int64_t s_h0, int64_t s_h1,
                               uint32_t box_rows) {
              TmapSpec sp;
              std::memset(&sp, 0, sizeof(sp));
              sp.base = base; sp.off = off; sp.dtype = d.adt; sp.rank = 4;
              sp.dims[0] = inner; sp.dims[1] = rows; sp.dims[2] = static_cast<uint64_t>(h0); sp.dims[3] = static_cast<uint64_t>(H / h0);
              sp.strides[0] = s_row; sp.strides[1] = s_h0; sp.strides[2] = s_h1;
              sp.box[0] = 64u; sp.box[1] = box_rows; sp.box[2] = 1u; sp.box[3] = 1u;
              sp.owner_is_flash = 1u;
              sp.valid = true;
              return sp;
            };
            f.tc_mode = 1;
            f.h0_size = static_cast<uint32_t>(h0);
            f.k_mn = k_dmajor ? 0u : 1u;
            f.tmap = static_cast<int32_t>(out->tmaps.size());
            out->tmaps.push_back(fa_spec(d.ptr[1], oq, 64, static_cast<uint64_t>(T), sq[2], sq[1], sq[0], 128u));
            if (k_dmajor) out->tmaps.push_back(fa_spec(d.ptr[2], ok_, 64, static_cast<uint64_t>(C), sk[3], sk[1], sk[0], 128u));
            else out->tmaps.push_back(fa_spec(d.ptr[2], ok_, static_cast<uint64_t>(C), 64, sk[2], sk[1], sk[0], 64u));
            out->tmaps.push_back(fa_spec(d.ptr[3], ov, 64, static_cast<uint64_t>(C), sv[2], sv[1], sv[0], 128u));
            ++out->n_flash_tc;
          }
        }
        // Decode-shaped tasks (few query rows, CUDA-core path): K and V rows by 16-byte loads when
        // head_dim is their unit-stride axis. K arrives as [H, hd, C] (a view of a [H, C, hd] cache).
        if (!f.tc_mode && (d.adt == kBF16 || d.adt == kF16) && !qv && (x[3] == 64 || x[3] == 128) && x[1] <= 8 &&
            x[0] > 0 && x[2] > 0 && c.Aligned16(t.a) && c.Aligned16(t.b) && c.Aligned16(t.p0)) {
          const int64_t H = x[0], C = x[2], hd = x[3];
          const int64_t nk[3] = {H, hd, C}, nv[3] = {H, C, hd};
          int64_t sk[3] = {hd * C, C, 1}, sv[3] = {C * hd, hd, 1}, ko = 0, vo = 0;
          bool ok = true;
          if (kv) ok = ok && AffineOverAxesN(f.vk, nk, 3, sk, &ko);
          if (vv) ok = ok && AffineOverAxesN(f.vv, nv, 3, sv, &vo);
          if (H == 1) sk[0] = sv[0] = 8;
          auto good = [](int64_t st) { return st >= 0 && st % 8 == 0; };
          if (ok && sk[1] == 1 && sv[2] == 1 && good(sk[0]) && good(sk[2]) && sk[2] > 0 && good(sv[0]) && good(sv[1]) && sv[1] > 0 &&
              good(ko) && good(vo)) {
            f.dec_mode = 1;
            f.dk_g = sk[0]; f.dk_c = sk[2]; f.dk_off = ko;
            f.dv_g = sv[0]; f.dv_c = sv[1]; f.dv_off = vo;
            ++out->n_flash_decode;
          }
        }
        ++out->n_flash;
        d.desc = c.PushDesc(f);
        if (f.tmap >= 0)
          for (int k = 0; k < 3; ++k) out->tmaps[f.tmap + k].desc_word = d.desc;
        break;
      }
      case kTopRedPart: case kTopRedComb: case kTopRedSeg: case kTopRedStrided:
      case kTopSoftmaxSeg: case kTopLayernormSeg:
        break;
      case kTopRedWindow: {
        const size_t x = t.p0;
        if (x + 2 > p.aux.size()) { *err = "reduce-window descriptor out of the aux pool"; return false; }
        const int32_t kind = p.aux[x], rank = p.aux[x + 1];
        if (rank < 0 || x + 2 + 6 * static_cast<size_t>(rank) > p.aux.size()) { *err = "reduce-window descriptor out of the aux pool"; return false; }
        if (rank > kWinDims) return fail_unimpl("reduce_window of rank > " + std::to_string(kWinDims));
        if (kind < 0 || kind > 2) return fail_unimpl("reduce_window kind " + std::to_string(kind));
        if (!(d.dt == kF32 || d.dt == kI32 || d.dt == kU32)) return fail_unimpl("reduce_window on dtype " + std::to_string(d.dt));
        DWindow w;
        std::memset(&w, 0, sizeof(w));
        w.kind = static_cast<uint32_t>(kind);
        w.rank = static_cast<uint32_t>(rank);
        uint64_t wcount = 1, n_in = 1;
        const int32_t *od = &p.aux[x + 2], *wd = od + rank, *ws = wd + rank, *pl = ws + rank, *id = pl + rank, *is = id + rank;
        for (int32_t k = 0; k < rank; ++k) {
          if (od[k] <= 0 || wd[k] <= 0 || ws[k] <= 0 || id[k] <= 0 || pl[k] < 0 || is[k] < 0) { *err = "reduce-window descriptor has a non-positive extent"; return false; }
          w.odim[k] = od[k]; w.wdim[k] = wd[k]; w.wstr[k] = ws[k]; w.idim[k] = id[k]; w.plow[k] = pl[k]; w.istr[k] = is[k];
          if (od[k] >= 2) MagicDivider(w.odim[k], &w.omagic[k], &w.oshift[k]);
          wcount *= static_cast<uint32_t>(wd[k]);
          n_in = std::max<uint64_t>(n_in, static_cast<uint64_t>(id[k]) * static_cast<uint64_t>(is[k]));
        }
        if (wcount > 0xFFFFFFFFull) return fail_unimpl("reduce_window with more than 2^32 taps");
        if (n_in * 4 > p.buffers[t.a].bytes) { *err = "reduce-window input dims exceed the operand buffer"; return false; }
        w.wcount = static_cast<uint32_t>(wcount);
        if (rank >= 1) {
          const int32_t l = rank - 1;
          bool v = wd[l] == 1 && ws[l] == 1 && pl[l] == 0 && od[l] == id[l] && is[l] == 1 && od[l] % 4 == 0 &&
                   c.Aligned16(t.dst) && c.Aligned16(t.a);
          for (int32_t k = 0; v && k < l; ++k) v = is[k] % 4 == 0;
          w.vec4 = v ? 1u : 0u;
        }
        d.desc = c.PushDesc(w);
        break;
      }
      case kTopGatherIndex: case kTopScatterIndex: {
        const bool scat = d.op == kTopScatterIndex;
        const size_t x = t.p0, head = scat ? 7 : 6;
        if (x + head > p.aux.size()) { *err = "indexed-move descriptor out of the aux pool"; return false; }
        const int32_t rank = p.aux[x], nidx = p.aux[x + 1];
        if (rank < 0 || nidx < 0 || x + head + 3 * static_cast<size_t>(rank) + 2 * static_cast<size_t>(nidx) > p.aux.size()) {
          *err = "indexed-move descriptor out of the aux pool";
          return false;
        }
        if (rank > kIdxDims || nidx > kIdxDims) return fail_unimpl("indexed gather / scatter of rank > " + std::to_string(kIdxDims));
        const uint32_t idx_id = static_cast<uint32_t>(p.aux[x + 5]);
        if (idx_id >= p.buffers.size()) { *err = "start-indices buffer id out of range"; return false; }
        DIndexed g;
        std::memset(&g, 0, sizeof(g));
        g.rank = static_cast<uint32_t>(rank);
        g.nidx = static_cast<uint32_t>(nidx);
        g.vec_stride = p.aux[x + 2];
        g.is64 = p.aux[x + 3] ? 1u : 0u;
        g.kind = scat ? static_cast<uint32_t>(p.aux[x + 6]) : 0u;
        g.esz = static_cast<uint32_t>(DtypeSize(d.dt));
        g.idx = c.Ref(idx_id);
        if (g.kind > 3u) return fail_unimpl("scatter combiner " + std::to_string(g.kind));
        if (g.kind != 0u && !(d.dt == kF32 || d.dt == kI32 || d.dt == kU32))
          return fail_unimpl("scatter add / max / min on dtype " + std::to_string(d.dt));
        if (DtypeSize(p.buffers[idx_id].dtype) != (g.is64 ? 8u : 4u)) { *err = "start-indices buffer width disagrees with the descriptor"; return false; }
        const int32_t *dims = &p.aux[x + head], *ops = dims + rank, *sis = ops + rank, *ios = sis + rank, *cmax = ios + nidx;
        for (int32_t k = 0; k < rank; ++k) {
          if (dims[k] <= 0) { *err = "indexed-move descriptor has a non-positive extent"; return false; }
          g.dim[k] = dims[k]; g.op_stride[k] = ops[k]; g.si_stride[k] = sis[k];
          if (dims[k] >= 2) MagicDivider(g.dim[k], &g.magic[k], &g.shift[k]);
        }
        for (int32_t k = 0; k < nidx; ++k) { g.idx_op_stride[k] = ios[k]; g.clamp_max[k] = cmax[k]; }
        // 16-byte words along the innermost dim: it walks the operand with stride 1, selects no
        // new index, and every run starts on a word boundary of the linear side
        if (rank >= 1 && g.esz <= 8) {
          const uint32_t chunk = 16u / g.esz;
          if (ops[rank - 1] == 1 && sis[rank - 1] == 0 && static_cast<uint32_t>(dims[rank - 1]) % chunk == 0) g.chunk = chunk;
        }
        d.desc = c.PushDesc(g);
        break;
      }
      case kTopConv: {
        const size_t x = t.p0;
        if (x + 3 > p.aux.size()) { *err = "convolution descriptor out of the aux pool"; return false; }
        const int32_t sdim = p.aux[x];
        if (sdim < 1 || sdim > 4) return fail_unimpl("convolution with " + std::to_string(sdim) + " spatial dims");
        if (x + 3 + 6 * static_cast<size_t>(sdim) > p.aux.size()) { *err = "convolution descriptor out of the aux pool"; return false; }
        if (d.dt != kF32) return fail_unimpl("convolution on dtype " + std::to_string(d.dt));
        DConv k;
        std::memset(&k, 0, sizeof(k));
        k.sdim = static_cast<uint32_t>(sdim);
        k.cin = static_cast<uint32_t>(p.aux[x + 1]);
        k.cout = static_cast<uint32_t>(p.aux[x + 2]);
        const int32_t *osp = &p.aux[x + 3], *win = osp + sdim, *st = win + sdim, *pl = st + sdim, *dil = pl + sdim, *isp = dil + sdim;
        if (p.aux[x + 1] <= 0 || p.aux[x + 2] <= 0) { *err = "convolution descriptor has a non-positive extent"; return false; }
        uint64_t wcount = 1;
        int64_t acc = k.cin;
        for (int32_t q = sdim - 1; q >= 0; --q) {
          if (osp[q] <= 0 || win[q] <= 0 || st[q] <= 0 || dil[q] <= 0 || isp[q] <= 0 || pl[q] < 0) { *err = "convolution descriptor has a non-positive extent"; return false; }
          k.osp[q] = osp[q]; k.win[q] = win[q]; k.str[q] = st[q]; k.dil[q] = dil[q]; k.isp[q] = isp[q]; k.plow[q] = pl[q];
          k.istr[q] = acc;
          acc *= isp[q];
          wcount *= static_cast<uint32_t>(win[q]);
        }
        k.ibatch = acc;
        if (wcount > 0xFFFFFFFFull) return fail_unimpl("convolution with more than 2^32 taps");
        k.wcount = static_cast<uint32_t>(wcount);
        if (wcount * k.cin * k.cout * 4 > p.buffers[t.b].bytes) { *err = "convolution weights exceed their buffer"; return false; }
        d.desc = c.PushDesc(k);
        break;
      }
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
    if (control) { d.a = e.wait_flag; d.b = e.wait_count; }   // tile entries: the device words stay 0
    // Point-to-point dependencies (scheduler.py:201-209 reserves wait_flag / wait_count / signal_flag of tile and
    // barrier entries for them; the reference emits "no flag" and a zero count): this backend orders phases by grid
    // barriers only, so an entry that names a flag is refused rather than run without its ordering.
    constexpr uint32_t kFlagNone = 0xFFFFFFFFu;
    if (!control && ((e.wait_flag != kFlagNone && e.wait_flag != 0u) || e.wait_count ||
                     (e.signal_flag != kFlagNone && e.signal_flag != 0u))) {
      *unimplemented = true;
      *err = "entry " + std::to_string(i) + " carries point-to-point wait / signal fields: not implemented by this backend";
      return false;
    }
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
  // Full reductions the lanes can share evenly: 4-byte elements, enough of them, and
  // partials that nothing but the combine reads.
  std::vector<int> fused_comb(p.tasks.size(), -1);
  for (size_t ti = 0; ti < p.tasks.size(); ++ti) {
    const VmTask &tp = p.tasks[ti];
    if ((tp.tile_op & 0xFFu) != kTopRedPart || tp.p1 == 0 || tp.p0 < 65536) continue;
    const uint32_t dt = (tp.tile_op >> 8) & 0xFFu;
    if (!(dt == kF32 || dt == kI32 || dt == kU32) || tp.p2 > kRXor) continue;
    const auto &rs = readers[tp.dst];
    if (rs.size() != 1 || pinned.count(tp.dst) || in_ids.count(tp.dst) || const_ids.count(tp.dst)) continue;
    const uint32_t ci = *rs.begin();
    const VmTask &tc = p.tasks[ci];
    const uint64_t nt = (static_cast<uint64_t>(tp.p0) + tp.p1 - 1) / tp.p1;
    if ((tc.tile_op & 0xFFu) != kTopRedComb || tc.a != tp.dst || tc.p1 != tp.p2 || tc.p0 != nt ||
        ((tc.tile_op >> 8) & 0xFFu) != dt || tc.dst == tp.dst || tc.dst == tp.a)
      continue;
    uint32_t writers = 0;
    for (const VmTask &o : p.tasks) writers += o.dst == tp.dst ? 1u : 0u;
    if (writers != 1) continue;
    // The result is now written one phase earlier than the schedule says. Arena slots are
    // shared between buffers whose live ranges are phase-disjoint (lowering.py:2824-2853), so
    // the result buffer may share bytes with something still being read in the RED_PART's
    // phase: only a result with bytes of its own (an I/O port, or an unshared slot) qualifies.
    if (!c.port_of.count(tc.dst)) {
      const BufferSlot &rb = p.buffers[tc.dst];
      bool shared = false;
      for (size_t j = 0; j < p.buffers.size() && !shared; ++j) {
        const BufferSlot &ob = p.buffers[j];
        if (j == tc.dst || !ob.bytes || c.port_of.count(static_cast<uint32_t>(j))) continue;
        shared = ob.offset < rb.offset + rb.bytes && rb.offset < ob.offset + ob.bytes;
      }
      if (shared) continue;
    }
    fused_comb[ti] = static_cast<int>(ci);
  }
  // A full f32 sum whose input is the f32 copy of a 16-bit buffer, made by a plain convert in the phase just
  // before and read by nothing else: the reduction streams the 16-bit source instead (half the bytes) and the
  // convert's phase does nothing. Straight-line programs only (phases counted by barriers in the root walk).
  std::vector<int> half_src(p.tasks.size(), -1);
  bool straight_line = true;
  for (const VmEntry &e : p.entries)
    if (e.task == kEntWhile || e.task == kEntIf || e.task == kEntFor) straight_line = false;
  std::vector<int> phase_lo(p.tasks.size(), 1 << 30), phase_hi(p.tasks.size(), -1);
  {
    const bool straight = straight_line && std::getenv("B2VM_NO_CONVERT_FOLD") == nullptr;
    if (straight_line)
      for (const VmLane &l : p.lane_tab) {
        int ph = 0;
        for (uint32_t i = 0; i < l.count; ++i) {
          const VmEntry &e = p.entries[l.off + i];
          if (e.task == kEntBarrier) { ++ph; continue; }
          if (e.task >= p.tasks.size()) continue;
          phase_lo[e.task] = std::min(phase_lo[e.task], ph);
          phase_hi[e.task] = std::max(phase_hi[e.task], ph);
        }
      }
    for (size_t ti = 0; straight && ti < p.tasks.size(); ++ti) {
      if (fused_comb[ti] < 0) continue;
      const VmTask &tp = p.tasks[ti];
      if (((tp.tile_op >> 8) & 0xFFu) != kF32 || tp.p2 != kSum) continue;
      const uint32_t src = tp.a;
      if (readers[src].size() != 1 || pinned.count(src) || in_ids.count(src) || out_ids.count(src) || const_ids.count(src)) continue;
      int conv = -1;
      uint32_t writers = 0;
      for (size_t k = 0; k < p.tasks.size(); ++k)
        if (p.tasks[k].dst == src) { ++writers; conv = static_cast<int>(k); }
      if (writers != 1) continue;
      const VmTask &cv = p.tasks[conv];
      const uint32_t cadt = (cv.tile_op >> 16) & 0xFFu;
      if ((cv.tile_op & 0xFFu) != kTopEw || cv.p0 != kConvert || ((cv.tile_op >> 8) & 0xFFu) != kF32 || !(cadt == kBF16 || cadt == kF16) ||
          cv.p2 != 0u || cv.p1 != tp.p0 || !c.Aligned16(cv.a) || tp.p0 % 8u != 0u)
        continue;
      if (phase_lo[conv] != phase_hi[conv] || phase_lo[ti] != phase_hi[ti] || phase_hi[conv] + 1 != phase_lo[ti]) continue;
      // nothing may write the 16-bit source (or bytes it shares) in the convert's or the reduction's phase
      bool clobbered = false;
      for (size_t k = 0; k < p.tasks.size() && !clobbered; ++k) {
        if (static_cast<int>(k) == conv || phase_hi[k] < phase_lo[conv] || phase_lo[k] > phase_lo[ti]) continue;
        const BufferSlot &wb = p.buffers[p.tasks[k].dst], &sb = p.buffers[cv.a];
        if (wb.bytes && sb.bytes && wb.offset < sb.offset + sb.bytes && sb.offset < wb.offset + wb.bytes && !c.port_of.count(cv.a)) clobbered = true;
        if (p.tasks[k].dst == cv.a) clobbered = true;
      }
      if (clobbered) continue;
      // the convert leaves its chain, so it may neither take nor hand over a value in registers
      bool forwards = (out->tasks[conv].flags & (kFwdA | kFwdB | kDeadStore)) != 0u;
      for (size_t k = 0; k < p.tasks.size(); ++k)
        if (pred[k] == conv && (out->tasks[k].flags & (kFwdA | kFwdB))) forwards = true;
      if (forwards) continue;
      half_src[ti] = conv;
    }
  }
  SpreadReductions(p, fused_comb, half_src, &c, out);
  // A full f32 sum (already shared by all lanes) over a buffer that one SOFTMAX_SEG / LAYERNORM_SEG task wrote in an
  // earlier phase: the row op adds what it stores to its lane's carry word, the sum's lanes read those words and
  // never stream the buffer. One such pair per program (the lanes have one carry word each). Straight-line only.
  if (straight_line && std::getenv("B2VM_NO_CARRIED_SUM") == nullptr) {
    for (size_t ti = 0; ti < p.tasks.size(); ++ti) {
      const VmTask &tp = p.tasks[ti];
      DTask &dt_ = out->tasks[ti];
      if ((tp.tile_op & 0xFFu) != kTopRedPart || !(dt_.flags & kRedFused) || ((tp.tile_op >> 8) & 0xFFu) != kF32 || tp.p2 != kSum) continue;
      const uint32_t src = half_src[ti] >= 0 ? p.tasks[half_src[ti]].a : tp.a;
      const uint32_t sdt = half_src[ti] >= 0 ? (p.tasks[half_src[ti]].tile_op >> 16) & 0xFFu : static_cast<uint32_t>(kF32);
      if (half_src[ti] < 0 && tp.p0 % 4u != 0u) continue;
      int wr = -1;
      uint32_t writers = 0;
      for (size_t k = 0; k < p.tasks.size(); ++k)
        if (p.tasks[k].dst == src) { ++writers; wr = static_cast<int>(k); }
      if (writers != 1 || in_ids.count(src) || const_ids.count(src)) continue;
      const VmTask &wt = p.tasks[wr];
      const uint32_t wop = wt.tile_op & 0xFFu;
      if (wop != kTopSoftmaxSeg && wop != kTopLayernormSeg) continue;
      if (((wt.tile_op >> 8) & 0xFFu) != sdt || static_cast<uint64_t>(wt.p0) * wt.p1 != tp.p0) continue;
      if (phase_lo[wr] != phase_hi[wr] || phase_lo[ti] != phase_hi[ti] || phase_hi[wr] >= phase_lo[ti]) continue;
      // every row exactly once, and nothing else may write the buffer's bytes from the row op's phase to the sum's
      uint64_t rows = 0;
      for (const DEntry &e : out->entries)
        if (e.task == static_cast<uint32_t>(wr)) rows += std::min(e.tile_hi, wt.p0) > e.tile_lo ? std::min(e.tile_hi, wt.p0) - e.tile_lo : 0u;
      if (rows != wt.p0) continue;
      bool clobbered = false;
      const BufferSlot &sb = p.buffers[src];
      for (size_t k = 0; k < p.tasks.size() && !clobbered; ++k) {
        if (static_cast<int>(k) == wr || phase_hi[k] < phase_lo[wr] || phase_lo[k] > phase_lo[ti]) continue;
        const BufferSlot &wb = p.buffers[p.tasks[k].dst];
        if (!c.port_of.count(src) && !c.port_of.count(p.tasks[k].dst) && wb.bytes && sb.bytes &&
            wb.offset < sb.offset + sb.bytes && sb.offset < wb.offset + wb.bytes)
          clobbered = true;
      }
      if (clobbered) continue;
      out->tasks[wr].flags |= kRowCarrySum;
      dt_.flags |= kRedCarried;
      out->n_carried_sums++;
      // A lane's share of the sum is now its own carry word, and the lanes' totals meet through the arrival counter:
      // when the phases after the row op's up to the sum's hold nothing but the sum, and no other shared reduction
      // runs beside the row op (one arrival counter), the barriers in between order nothing and go.
      const int pw = phase_lo[wr], pt = phase_lo[ti];
      bool alone = true;
      for (const VmLane &l : out->lanes) {
        int ph = 0;
        for (uint32_t i = l.off; i < l.off + l.count && alone; ++i) {
          const DEntry &e = out->entries[i];
          if (e.task == kEntBarrier) { ++ph; continue; }
          if (e.task == kEntNop || e.task >= out->tasks.size() || ph < pw || ph > pt) continue;
          if (e.task == static_cast<uint32_t>(ti)) continue;
          if (ph > pw || (out->tasks[e.task].flags & kRedFused && (p.tasks[e.task].tile_op & 0xFFu) == kTopRedPart)) alone = false;
        }
      }
      if (alone) {
        for (const VmLane &l : out->lanes) {
          int ph = 0;
          for (uint32_t i = l.off; i < l.off + l.count; ++i) {
            DEntry &e = out->entries[i];
            if (e.task != kEntBarrier) continue;
            if (ph >= pw && ph < pt) e.task = kEntNop;
            ++ph;
          }
        }
        out->n_carried_barriers_removed += static_cast<uint32_t>(pt - pw);
      }
      break;
    }
  }
  // The decomposed RMS norm over bf16 rows - convert to f32, square, RED_SEG row sums, a MAP_REGION {affine, rsqrt} on them,
  // multiply by the broadcast row scalar, multiply by the broadcast f32 gain, convert to bf16 - becomes one row op
  // on the last convert's entries (rms_rows_tiles); the six other tasks' entries leave the stream. Every
  // intermediate must be read by the idiom alone. Straight-line programs only.
  if (straight_line && std::getenv("B2VM_NO_RMS_FUSION") == nullptr) {
    auto sole_writer = [&](uint32_t id) {
      int w = -1;
      for (size_t k = 0; k < p.tasks.size(); ++k)
        if (p.tasks[k].dst == id) { if (w >= 0) return -1; w = static_cast<int>(k); }
      return w;
    };
    auto scratch_only = [&](uint32_t id, std::initializer_list<uint32_t> want) {
      if (pinned.count(id) || in_ids.count(id) || out_ids.count(id) || const_ids.count(id)) return false;
      return readers[id] == std::set<uint32_t>(want);
    };
    auto is_ew = [&](const VmTask &t, uint32_t subop, uint32_t dt, uint32_t adt) {
      return (t.tile_op & 0xFFu) == kTopEw && t.p0 == subop && ((t.tile_op >> 8) & 0xFFu) == dt && ((t.tile_op >> 16) & 0xFFu) == adt;
    };
    // view descriptor (rank, dims, strides, offset) of a [rows, d] broadcast with the given strides
    auto is_broadcast = [&](uint32_t field, int64_t rows, int64_t d, int64_t s0, int64_t s1) {
      if (!field) return false;
      const size_t x = field - 1;
      if (x + 6 > p.aux.size()) return false;
      return p.aux[x] == 2 && p.aux[x + 1] == rows && p.aux[x + 2] == d && p.aux[x + 3] == s0 && p.aux[x + 4] == s1 && p.aux[x + 5] == 0;
    };
    bool any = false;
    for (size_t cvi = 0; cvi < p.tasks.size(); ++cvi) {
      const VmTask &cv = p.tasks[cvi];
      if (!is_ew(cv, kConvert, kBF16, kF32) || cv.p2 != 0u) continue;
      const int m2i = sole_writer(cv.a);
      if (m2i < 0) continue;
      const VmTask &m2 = p.tasks[m2i];
      if (!is_ew(m2, kMul, kF32, kF32) || m2.p2 != 0u || m2.p1 != cv.p1) continue;
      const int m1i = sole_writer(m2.a);
      if (m1i < 0) continue;
      const VmTask &m1 = p.tasks[m1i];
      if (!is_ew(m1, kMul, kF32, kF32) || m1.p2 != 0u || m1.p1 != cv.p1) continue;
      const int ci = sole_writer(m1.a), gi = sole_writer(m1.b);
      if (ci < 0 || gi < 0) continue;
      const VmTask &cx = p.tasks[ci], &gr = p.tasks[gi];
      if (!is_ew(cx, kConvert, kF32, kBF16) || cx.p2 != 0u || cx.p1 != cv.p1) continue;
      if ((gr.tile_op & 0xFFu) != kTopMapRegion || ((gr.tile_op >> 8) & 0xFFu) != kF32 || ((gr.tile_op >> 16) & 0xFFu) != kF32) continue;
      const int64_t rows = gr.p1, d = rows ? static_cast<int64_t>(cv.p1) / rows : 0;
      if (rows <= 0 || rows * d != static_cast<int64_t>(cv.p1) || !(d == 256 || d == 512 || d == 1024 || d == 2048)) continue;
      if (!is_broadcast(m1.p3, rows, d, 1, 0) || !is_broadcast(m2.p3, rows, d, 0, 1)) continue;
      const int ri = sole_writer(gr.a);
      if (ri < 0) continue;
      const VmTask &rd = p.tasks[ri];
      if ((rd.tile_op & 0xFFu) != kTopRedSeg || ((rd.tile_op >> 8) & 0xFFu) != kF32 || rd.p0 != rows || rd.p1 != d || rd.p2 != kSum) continue;
      // the region (region.py:19-23: n_in, out_slot, n_micro, in_slot[n_in], n_micro x {kind, dst, a, b, s, t}) is
      // exactly r = rsqrt(affine(row sum)): one input, two micro-ops
      const size_t gx = gr.p0;
      if (gx + 4 + 12 > p.aux.size() || p.aux[gx] != 1 || p.aux[gx + 2] != 2 || gr.a != rd.dst) continue;
      const int32_t *mo = &p.aux[gx + 4];
      if (mo[0] != static_cast<int32_t>(kAffine) || mo[2] != p.aux[gx + 3] || mo[6] != static_cast<int32_t>(kRsqrt) || mo[8] != mo[1] ||
          p.aux[gx + 1] != mo[7])
        continue;
      const int si = sole_writer(rd.a);
      if (si < 0) continue;
      const VmTask &sq = p.tasks[si];
      if (!is_ew(sq, kMul, kF32, kF32) || sq.p2 != 0u || sq.p3 != 0u || sq.a != cx.dst || sq.b != cx.dst || sq.p1 != cv.p1) continue;
      const uint32_t U = static_cast<uint32_t>(cvi), M2 = static_cast<uint32_t>(m2i), M1 = static_cast<uint32_t>(m1i), C = static_cast<uint32_t>(ci),
                     G = static_cast<uint32_t>(gi), R = static_cast<uint32_t>(ri), S = static_cast<uint32_t>(si);
      if (!scratch_only(cv.a, {U}) || !scratch_only(m2.a, {M2}) || !scratch_only(cx.dst, {S, M1}) || !scratch_only(gr.dst, {M1}) ||
          !scratch_only(rd.dst, {G}) || !scratch_only(sq.dst, {R}))
        continue;
      // x and the gain are read in the last convert's phase now: both written before it, x in memory (not a value a
      // chain only hands on in registers), neither's bytes written from their old readers' phases to that one
      const uint32_t xid = cx.a, gid = m2.b;
      const int pu = phase_lo[cvi];
      if (phase_lo[cvi] != phase_hi[cvi] || !c.Aligned16(xid) || !c.Aligned16(gid) || !c.Aligned16(cv.dst)) continue;
      bool safe = true;
      for (uint32_t id : {xid, gid}) {
        const int first_read = id == xid ? phase_lo[ci] : phase_lo[m2i];
        for (size_t k = 0; k < p.tasks.size() && safe; ++k) {
          if (phase_hi[k] < 0) continue;
          if (p.tasks[k].dst == id) {      // its writer: a whole phase earlier than the row op, and storing
            if (phase_hi[k] >= pu || (out->tasks[k].flags & kDeadStore)) safe = false;
            continue;
          }
          if (phase_hi[k] < first_read || phase_lo[k] > pu || c.port_of.count(id) || c.port_of.count(p.tasks[k].dst)) continue;
          const BufferSlot &wb = p.buffers[p.tasks[k].dst], &sb = p.buffers[id];
          if (wb.bytes && sb.bytes && wb.offset < sb.offset + sb.bytes && sb.offset < wb.offset + wb.bytes) safe = false;
        }
      }
      // the result's bytes may not be anything the idiom still had to read when the convert ran: it is written in
      // the same phase as before, so that holds as it did.
      if (!safe) continue;
      uint64_t covered = 0;
      for (const DEntry &e : out->entries)
        if (e.task == U) covered += e.tile_hi > e.tile_lo ? e.tile_hi - e.tile_lo : 0u;
      if (covered != (static_cast<uint64_t>(cv.p1) + kEwTs - 1) / kEwTs) continue;
      DTask &du = out->tasks[cvi];
      du.op = kTopRmsRows;
      du.flags = 0u;
      du.desc = 0u;
      du.ptr[1] = c.Ref(xid);
      du.ptr[2] = c.Ref(gid);
      std::memset(du.p, 0, sizeof(du.p));
      du.p[0] = static_cast<uint32_t>(rows);
      du.p[1] = static_cast<uint32_t>(d);
      du.p[2] = static_cast<uint32_t>(mo[4]);      // the affine's s and t
      du.p[4] = static_cast<uint32_t>(mo[5]);
      du.adt = kBF16;
      for (DEntry &e : out->entries)
        if (e.task == M2 || e.task == M1 || e.task == C || e.task == G || e.task == R || e.task == S) e.task = kEntNop;
      // the gain's own convert from bf16 goes too when the idiom alone reads its result and the bf16 source is a
      // program argument nothing writes
      const int gw = sole_writer(gid);
      if (gw >= 0) {
        const VmTask &gc = p.tasks[gw];
        bool written = false;
        for (const VmTask &o : p.tasks) written = written || o.dst == gc.a;
        if (is_ew(gc, kConvert, kF32, kBF16) && gc.p2 == 0u && gc.p1 == static_cast<uint32_t>(d) && scratch_only(gid, {M2}) &&
            in_ids.count(gc.a) && !written && c.Aligned16(gc.a)) {
          du.ptr[2] = c.Ref(gc.a);
          du.p[3] = 1u;
          for (DEntry &e : out->entries)
            if (e.task == static_cast<uint32_t>(gw)) e.task = kEntNop;
        }
      }
      // a task that forwarded into one of these in a chain stores its result again
      for (size_t k = 0; k < p.tasks.size(); ++k)
        if (succ[k] == ci || succ[k] == m1i || succ[k] == m2i || succ[k] == si) out->tasks[k].flags &= ~kDeadStore;
      out->families |= kFamRows;
      out->n_rms_rows++;
      any = true;
    }
    if (any) {
      CompactChains(out);
      // phases that hold nothing any more lose the barrier that closed them
      const uint32_t n_bar = [&] { uint32_t n = 0; const VmLane &l = out->lanes[0];
                                   for (uint32_t i = l.off; i < l.off + l.count; ++i) n += out->entries[i].task == kEntBarrier; return n; }();
      std::vector<char> busy(n_bar + 1, 0);
      for (const VmLane &l : out->lanes) {
        uint32_t ph = 0;
        for (uint32_t i = l.off; i < l.off + l.count; ++i) {
          const uint32_t tk = out->entries[i].task;
          if (tk == kEntBarrier) { ++ph; continue; }
          if (tk != kEntNop && ph <= n_bar) busy[ph] = 1;
        }
      }
      for (const VmLane &l : out->lanes) {
        uint32_t ph = 0;
        for (uint32_t i = l.off; i < l.off + l.count; ++i) {
          if (out->entries[i].task != kEntBarrier) continue;
          if (ph <= n_bar && !busy[ph]) out->entries[i].task = kEntNop;
          ++ph;
        }
      }
      for (uint32_t ph = 0; ph < n_bar; ++ph) out->n_empty_phases_dropped += busy[ph] ? 0u : 1u;
    }
  }
  // Dynamic work distribution for tensor-core attention tasks: allowed when the task's
  // entries cover all its query rows, no lane holds more than one of them, and they
  // sit outside the sub-ranges of WHILE / IF entries (where lanes may not all arrive).
  {
    uint32_t slots = 0;
    for (size_t ti = 0; ti < p.tasks.size() && slots < kMaxWorkSlots; ++ti) {
      DTask &d = out->tasks[ti];
      if (d.op != kTopFlashAttn || !d.desc) continue;
      DFlash *f = reinterpret_cast<DFlash *>(&out->desc[d.desc]);
      if (!f->tc_mode) continue;
      const int32_t *x = &p.aux[p.tasks[ti].p3];
      const uint64_t rows = static_cast<uint64_t>(x[0]) * static_cast<uint64_t>(x[1]);
      uint64_t covered = 0;
      uint32_t owners = 0;
      bool ok = true;
      for (const VmLane &l : out->lanes) {
        uint32_t mine = 0;
        for (uint32_t e = 0; e < l.count; ++e) {
          const DEntry &en = out->entries[l.off + e];
          if (en.task != ti) continue;
          ++mine;
          if (e >= l.root_len) ok = false;          // inside a control range: keep the static split
          covered += std::min<uint64_t>(en.tile_hi, rows) - std::min<uint64_t>(en.tile_lo, rows);
        }
        if (mine > 1) ok = false;
        owners += mine ? 1u : 0u;
      }
      if (!ok || covered != rows || owners == 0) continue;
      f->work_slot = slots++;
      f->n_owner_lanes = owners;
      out->needs_scratch = true;
    }
  }
  return true;
}

}  // namespace b2
