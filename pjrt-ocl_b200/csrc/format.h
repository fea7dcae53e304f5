// VMProgram v3 wire format and the device-side tables the loader derives from it.
// Shared by the host runtime (.cc) and the megakernel (.cu).
//
// Wire layout (little-endian, every section 8-byte aligned), as written by the
// reference's VMProgram.serialize (python/pjrt_ocl/lowering.py:286-331) and
// Schedule.serialize_sections (python/pjrt_ocl/scheduler.py:226-248):
//   header 48 B | buffer table n x 24 B | input ids | output ids | io shapes |
//   aux pool u32[n_aux] | const pool | instrs n x 32 B |
//   sched header 16 B | tasks n x 48 B | lane table n_lanes x 16 B | entries n x 32 B
#ifndef B2VM_FORMAT_H_
#define B2VM_FORMAT_H_

#include <stdint.h>

namespace b2 {

constexpr uint32_t kMagic = 0x314D5056u;  // "VPM1"
constexpr uint32_t kVersion = 3;

#if defined(__CUDACC__)
#define B2_HOST_DEVICE __host__ __device__
#else
#define B2_HOST_DEVICE
#endif

// dtype enum (lowering.py:59-68)
enum Dtype : uint32_t { kF32 = 0, kI32, kU32, kBool, kI64, kF64, kF16, kBF16, kDtMax = kBF16 };

// tile ops (scheduler.py:47-71)
enum TileOp : uint32_t {
  kTopEw = 0, kTopMma, kTopGather, kTopRedPart, kTopRedComb, kTopIotaDim, kTopScatter,
  kTopDynGather, kTopDynScatter, kTopRedWindow, kTopRedSeg, kTopSoftmaxSeg, kTopLayernormSeg,
  kTopMapRegion, kTopFlashAttn, kTopRedStrided, kTopGatherIndex, kTopConv, kTopScatterIndex,
  kTopMax = kTopScatterIndex,
  // Not on the wire: the loader's own row op for a recognised RMS-norm idiom over bf16 rows (convert, square, row sum,
  // per-row scalar region, two broadcast multiplies, convert back), see rms_rows_tiles.
  kTopRmsRows = 32
};

// Tile-op families: the unit in which code is compiled into a build of the
// megakernel (variants.h). Every tile op belongs to exactly one.
enum Family : uint32_t {
  kFamEw = 1u << 0,      // TILE_EW
  kFamMove = 1u << 1,    // GATHER, SCATTER, DYN_GATHER, DYN_SCATTER, IOTA_DIM
  kFamRed = 1u << 2,     // RED_PART, RED_COMB, RED_SEG, RED_STRIDED
  kFamRows = 1u << 3,    // SOFTMAX_SEG, LAYERNORM_SEG
  kFamRegion = 1u << 4,  // MAP_REGION
  kFamMma = 1u << 5,     // TILE_MMA
  kFamFlash = 1u << 6,   // FLASH_ATTN
  kFamIndex = 1u << 7,   // RED_WINDOW, GATHER_INDEX, SCATTER_INDEX, CONV
  kFamShort = 1u << 8,   // short-run paths of the families above: RED_SEG over segments of 2..8 elements, elementwise
                         // views and gathers whose source runs are shorter than 16 bytes, pow with constant exponents
  kFamAll = 0xFFFFFFFFu
};
B2_HOST_DEVICE inline uint32_t family_of(uint32_t tile_op) {
  switch (tile_op) {
    case kTopEw: return kFamEw;
    case kTopGather: case kTopScatter: case kTopDynGather: case kTopDynScatter: case kTopIotaDim: return kFamMove;
    case kTopRedPart: case kTopRedComb: case kTopRedSeg: case kTopRedStrided: return kFamRed;
    case kTopSoftmaxSeg: case kTopLayernormSeg: case kTopRmsRows: return kFamRows;
    case kTopMapRegion: return kFamRegion;
    case kTopMma: return kFamMma;
    case kTopFlashAttn: return kFamFlash;
    default: return kFamIndex;
  }
}

// elementwise subops (pjrt_plugin/kernels/vm_common.cl:118-146)
enum Sub : uint32_t {
  kAdd = 0, kMul, kSubt, kDiv, kMax, kMin, kPow, kCopy, kNeg, kExp, kLog, kSqrt, kRsqrt, kTanh,
  kAbs, kFloor, kCeil, kSign, kFill, kIotaFlat, kCmp, kSelect, kLts, kConvert, kBitcast, kAtan2,
  kRemainder, kLog1p, kExpm1, kCbrt, kSin, kCos, kTan, kRint, kRound, kAnd, kOr, kXor, kNot,
  kIsFinite, kAffine, kGelu, kShl, kShrL, kShrA, kSubMax = kShrA
};

// reduction kinds (python/pjrt_ocl/ops/reduce.py:56)
enum RedKind : uint32_t { kSum = 0, kRMax, kRMin, kProd, kRAnd, kROr, kRXor };

// RED_STRIDED tasks the device reduces row by row (a warp streams the red*inner
// contiguous elements of one row): f32, inner axis of 2..4, rows of whole 16-byte
// words and at least 1 KB, sums. The loader spreads such a task over
// all lanes when its output tiles are few; both sides use this one rule.
B2_HOST_DEVICE inline bool red_strided_rows_ok(uint32_t dt, int64_t red, int64_t inner, uint32_t kind) {
  return dt == kF32 && inner >= 2 && inner <= 4 && (red * inner) % 4 == 0 && red * inner >= 256 &&
         kind == kSum;
}

// entry sentinels (scheduler.py:80-85)
constexpr uint32_t kEntNop = 0xFFFFFFFFu;
constexpr uint32_t kEntBarrier = 0xFFFFFFFEu;
constexpr uint32_t kEntWhile = 0xFFFFFFFDu;
constexpr uint32_t kEntIf = 0xFFFFFFFCu;
constexpr uint32_t kEntFor = 0xFFFFFFFBu;

struct VmTask { uint32_t tile_op, dst, a, b, p0, p1, p2, p3, p4, p5, p6, p7; };
struct VmEntry { uint32_t task, tile_lo, tile_hi, wait_flag, wait_count, signal_flag, slots, pad; };
struct VmLane { uint32_t off, count, root_len, pad; };
static_assert(sizeof(VmTask) == 48 && sizeof(VmEntry) == 32 && sizeof(VmLane) == 16, "wire structs");

// Tile geometry this backend executes with and advertises to the scheduler
// (PJRT_OCL_EW_TS / PJRT_OCL_MMA_T; scheduler.py:36-45).
constexpr uint32_t kEwTs = 4096;
constexpr uint32_t kMmaT = 128;
constexpr int kMaxDepth = 8;          // control frame stack (vm_main.cl:103)
constexpr uint32_t kMaxIoPorts = 64;  // zero-copy I/O buffers passed by kernel parameter

// ---------------------------------------------------------------------------
// Device tables
// ---------------------------------------------------------------------------

// A buffer reference in a device task: either an absolute device address
// (arena-resident buffers, resolved once at load) or, with bit 63 set, the index
// of an I/O port whose address arrives with each launch.
typedef uint64_t BufRef;
constexpr uint64_t kPortBit = 1ull << 63;

// A strided view, collapsed at load time to at most kViewDims dims (outermost first).
// index(i) = off + sum_k coord_k(i) * stride[k], coord by row-major unravel of i
// over dim[]. rank 0 = every element reads `off`.
struct DView {
  int32_t rank;
  int32_t vec_ok;       // 1: dim[rank-1] % 4 == 0, innermost stride is 0 or 1, and a
                        // group of 4 consecutive consumer elements never straddles it
  int32_t inner_stride; // stride[rank-1] (0 or 1 when vec_ok)
  int32_t aligned4;     // 1: off and every outer stride are multiples of 4 elements
  int64_t off;
  uint32_t dim[6];
  int32_t stride[6];
  // n / dim[k] without a divide instruction, for every 32-bit n (dim >= 2):
  // q = umulhi(n, magic); ((n - q) >> 1) + q >> shift.
  uint32_t magic[6];
  uint32_t shift[6];
};
constexpr int kViewDims = 6;

enum TaskFlags : uint32_t {
  kFwdA = 1u << 0,      // EW chain: operand a is the previous chain op's result (in registers)
  kFwdB = 1u << 1,
  kDeadStore = 1u << 2, // EW chain: nothing but the next chain op reads dst; skip the store
  kViewA = 1u << 3,
  kViewB = 1u << 4,
  kVecPath = 1u << 5,   // every pointer 16-byte aligned and dtypes on the 4-wide path
  kFwdC = 1u << 6,      // select predicate forwarded
  kRedFused = 1u << 7,  // RED_PART re-cut over all lanes with the combine folded in: entries carry word
                        // ranges, ptr[3] is the final result, lane totals meet in KParams::scratch
  kRedSrcBf16 = 1u << 8, // ... and its input is the bf16 (kRedSrcF16: f16) source of the convert that fed it: the
  kRedSrcF16 = 1u << 9,  // f32 copy is never written, each 32-bit word of the stream holds two elements
  kRowCarrySum = 1u << 10, // SOFTMAX_SEG / LAYERNORM_SEG: also add every value stored to this lane's carry word in the
                           // scratch (as f32, after rounding to the output type): the full sum that follows reads
  kRedCarried = 1u << 11,  // ... that word instead of the array (on the kRedFused RED_PART)
};

// Scratch of a loaded program (KParams::scratch): where the lanes of a re-cut full
// reduction leave their totals. `arrived` returns to 0 after every use.
constexpr uint32_t kMaxWorkSlots = 6;
struct RedScratch {
  uint32_t arrived;
  uint32_t pad[3];
  uint32_t work[2 * kMaxWorkSlots];   // {next unit, lanes done} per dynamically distributed task; at rest 0
  unsigned long long total[1];        // [n_lanes] lane totals, then [n_lanes] carry words (kRowCarrySum; at rest 0)
};

struct DTask {
  uint32_t op, dt, adt, flags;
  BufRef ptr[4];        // dst, a, b, c (select predicate / flash V / epilogue residual)
  uint32_t p[8];        // p0..p7 as in the wire task (buffer ids already resolved elsewhere)
  uint32_t desc;        // word offset into the descriptor pool (op specific), 0 = none
  uint32_t cdt;         // dtype of ptr[3] where it matters (epilogue residual)
  uint32_t pad[2];
};
static_assert(sizeof(DTask) == 96, "DTask layout");

// A device entry: the wire entry with control cond buffers resolved and chain
// annotations added by the loader.
struct DEntry {
  uint32_t task, tile_lo, tile_hi, a, b;  // a/b: wait_flag / wait_count of the wire entry (control ranges, trip counts);
                                          // on a RED_STRIDED entry the loader spread over the lanes: rows [a, b)
  uint32_t chain;        // number of consecutive EW entries (this one included) to run as one fused chain; 0/1 = alone
  BufRef cond;           // WHILE / IF: address of the 4-byte condition word
};
static_assert(sizeof(DEntry) == 32, "DEntry layout");

enum StatusCode : uint32_t { kStOk = 0, kStBarrierTimeout = 1, kStStackOverflow = 2, kStBadOp = 3, kStTensorTimeout = 4 };

// Barrier + status block in device memory (one per loaded program).
struct DSync {
  uint32_t arrive;       // arrival counter
  uint32_t pad;
  uint32_t gen;          // barrier generation   } one aligned 8-byte word: a waiting lane polls
  uint32_t abort;        // set by the first lane } both with a single load
                         // whose wait ran out
  uint32_t status[4];    // code, lane, where, detail (first writer wins)
  unsigned long long barriers;   // lane 0
  unsigned long long device_ns;  // lane 0
  // lane 0's arrival time (ns since kernel entry) at each of its first
  // kPhaseSlots grid barriers: per-phase wall time, as the reference's
  // per-barrier timestamps (vm_common.cl:258-282) give it.
  unsigned long long phase_ns[64];
};
constexpr uint32_t kPhaseSlots = 64;
static_assert(offsetof(DSync, gen) % 8 == 0 && offsetof(DSync, abort) == offsetof(DSync, gen) + 4, "gen and abort are polled as one 8-byte word");

// ---- per-op descriptors the loader writes into the descriptor pool -------------
// Descriptor the loader writes for GATHER / SCATTER / DYN_* tasks.
struct DMove {
  DView view;          // linear side index -> strided side index (in elements)
  uint32_t esz;        // element size in bytes
  uint32_t chunk;      // elements per 16-byte chunk when vector-movable, else 0
  uint32_t transposed; // gather whose innermost linear dim is strided on the other side while the next
                       // one is contiguous there (a transpose): moved through shared-memory tiles
  uint32_t pad;
  uint32_t n_idx;      // DYN_*: number of runtime start indices (rank), else 0
  uint32_t is64;       // DYN_*: start scalars are i64
  int32_t clamp_max[8];
  int32_t idx_stride[8];
  BufRef idx_ptr[8];   // DYN_*: where each start scalar lives
};

struct DRegion {            // loader-built: the 8 input references (a, b, p2..p7)
  BufRef in[8];
};

// tc_mode bits: the operands are affine in (batch, row, k) with a unit stride along
// k ("K-major") or along the row / column index ("MN-major"), 16-byte friendly.
constexpr uint32_t kTcOk = 1u, kTcAmn = 2u, kTcBmn = 4u;
// A TMA tensor map (CUtensorMap, opaque to this code), 64-byte aligned as the
// hardware requires. Built on the host for every tensor-core matmul operand.
struct alignas(64) DTmap { uint64_t w[16]; };

struct DMma {          // loader-built
  DView va, vb;
  uint32_t tc_mode;    // 0: CUDA-core path only
  int32_t tmap;        // index of the operands' tensor maps (A at tmap, B at tmap + 1) in KParams::tmaps, or -1
  // tensor-core path, in elements: A(g,m,k) = a_off + g*a_gs + (K-major: m*a_ld + k | MN-major: k*a_ld + m),
  // B(g,k,n) = b_off + g*b_gs + (K-major: n*b_ld + k | MN-major: k*b_ld + n)
  int64_t a_ld, b_ld;
  int64_t a_gs, b_gs;
  int64_t a_off, b_off;
};

struct DFlash {        // loader-built
  DView vq, vk, vv;
  uint32_t has_q, has_k, has_v;   // operand is read through its view
  uint32_t tc_mode;               // 0: CUDA-core path only
  // Tensor-core path. The operands are reached through three TMA tensor maps (Q, K, V at
  // KParams::tmaps[tmap .. tmap + 2]) of rank 4 {inner, rows, h0, h1}: head h is
  // (h1, h0) = (h / h0_size, h % h0_size), which lets a [batch, seq, heads, hd] tensor
  // be read in place as [batch * heads, seq, hd].
  int32_t tmap;
  uint32_t h0_size;
  uint32_t k_mn;                  // K: keys are the unit-stride dimension (the plain [H, hd, C] operand), else d is
  // Dynamic work distribution: when every lane that owns a share of the task enters it
  // exactly once per phase, the lanes draw 256-row units from one counter pair in the
  // program's scratch (heaviest first) instead of keeping their static ranges.
  uint32_t work_slot;             // index of the {next, done} pair in the scratch, or kNoWorkSlot
  uint32_t n_owner_lanes;
  // Few query rows per head (a decode step) with 16-bit K and V whose head_dim axis is the
  // unit-stride one: element (g, key, d) of K at dk_off + g * dk_g + key * dk_c + d (V alike),
  // every term a multiple of 8 elements, so a key's row is read with 16-byte loads.
  uint32_t dec_mode;
  int64_t dk_g, dk_c, dk_off, dv_g, dv_c, dv_off;
};
constexpr uint32_t kNoWorkSlot = 0xFFFFFFFFu;

// RED_WINDOW (aux layout: pjrt_plugin/kernels/ops/reduce_window.cl:10-13), with the
// divisions by the output dims prepared.
constexpr int kWinDims = 8;
struct DWindow {       // loader-built
  uint32_t kind, rank, wcount;
  uint32_t vec4;       // the innermost axis is not windowed, strided or padded and is a multiple of 4
                       // (4-byte elements, aligned): 4 outputs per thread from one 16-byte load per tap
  uint32_t odim[kWinDims], wdim[kWinDims], wstr[kWinDims], idim[kWinDims];
  int32_t plow[kWinDims], istr[kWinDims];
  uint32_t omagic[kWinDims], oshift[kWinDims];
};

// GATHER_INDEX / SCATTER_INDEX (aux layouts: ops/gather.cl:90-107, ops/scatter.cl:95-104):
// the output's (gather) or the updates' (scatter) dims with the operand / index strides each
// adds, and per index component its operand stride and clamp.
constexpr int kIdxDims = 8;
struct DIndexed {      // loader-built
  uint32_t rank, nidx, is64, kind;      // kind: scatter combiner 0 set 1 add 2 max 3 min
  int32_t vec_stride;
  uint32_t esz;
  uint32_t chunk;      // elements per 16-byte word when the innermost dim is a contiguous run on both
                       // sides made of whole words, else 0
  uint32_t pad;
  BufRef idx;          // the start-indices buffer
  uint32_t dim[kIdxDims];
  int32_t op_stride[kIdxDims], si_stride[kIdxDims];
  uint32_t magic[kIdxDims], shift[kIdxDims];
  int32_t idx_op_stride[kIdxDims], clamp_max[kIdxDims];
};

// CONV (aux layout: ops/conv.cl:15-20), input strides precomputed.
struct DConv {         // loader-built
  uint32_t sdim, cin, cout, wcount;
  uint32_t osp[4], win[4], str[4], dil[4], isp[4];
  int32_t plow[4];
  int64_t istr[4], ibatch;
};

struct IoTable { void *p[kMaxIoPorts]; };

struct KParams {
  const DTask *tasks;
  const DEntry *entries;
  const VmLane *lanes;
  const int32_t *aux;       // the program's aux pool, unmodified
  const uint64_t *desc;     // loader-built descriptor pool (views, pointers, ...)
  DSync *sync;
  uint8_t *scratch;         // per-program scratch (split reductions, tensor-core staging)
  const DTmap *tmaps;       // tensor maps of the tensor-core matmul operands
  uint32_t n_lanes;
  uint32_t pad;
  unsigned long long wait_budget_ns;
  // Optional per-lane timing (null = off): kLaneTsSlots words per lane - [0] the lane's
  // start, [1] its exit, [2 + i] its ARRIVAL at grid barrier i (first kPhaseSlots
  // barriers), all in globaltimer nanoseconds. What the reference records under
  // VMO_TS_REC (pjrt_plugin/kernels/vm_common.cl:258-282).
  unsigned long long *lane_ts;
  IoTable io;
};
constexpr uint32_t kLaneTsSlots = kPhaseSlots + 2;

}  // namespace b2
#endif
