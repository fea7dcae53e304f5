/* vmoracle - CPU restatement of the reference's VMProgram v3 device path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests and the
 * benchmark's cpu_baseline leg use; the CUDA backend never links, loads or
 * calls it.  It is plain C (optionally OpenMP across host cores) and restates,
 * function by function, what the reference executes for one `Execute`:
 *
 *   parse        pjrt_plugin/src/runtime.cc:90-251 (VmProgram::Parse) and
 *                python/pjrt_ocl/vmreader.py:182-380
 *   load         pjrt_plugin/src/runtime.cc:735-1074 (ids -> addresses; here
 *                ids are resolved to host pointers into one arena)
 *   control walk pjrt_plugin/kernels/vm_main.cl:107-258 (vm2 frame stack) in
 *                the per-phase host order of runtime.cc:1546-1602
 *                (LaunchHostDispatch) / vmreader.py:655-773 (_run_control)
 *   tile ops     pjrt_plugin/kernels/ops/{ew,gather,reduce,mma,iota,scatter,
 *                dynslice,region,attention,reduce_window,conv}.cl with the numeric
 *                conventions of the numpy validators in python/pjrt_ocl/ops/
 *                {elementwise,reduce,dot,attention,region,shape,making,bitcast,
 *                dynslice,concat,reduce_window,gather_index,scatter_index,conv}.py
 *                where the two differ (the validators are what the reference's
 *                own tests pin).
 *
 * Pinning: tests/test_oracle.py replays every fixture of tests/golden/ (blobs
 * assembled by the reference's lowering + scheduler, outputs produced by BOTH
 * reference validators) through this file; integer/bool/index results must be
 * bit-exact and float results within the fixture's stated tolerance.  The
 * reference's device kernels (OpenCL C) cannot be compiled here, so the
 * transcendental builtins are pinned against numpy, not against an OpenCL
 * runtime.
 *
 * Deliberate choices where the reference's device code and its validators
 * disagree (validators win, because they are what its tests assert):
 *   - float max/min propagate NaN (numpy maximum/minimum), unlike fmax/fmin;
 *   - u32 elementwise max/min/div/compare/convert are unsigned;
 *   - compare on bool operands reads 1-byte values;
 *   - f32 -> bf16 rounds to nearest even and keeps NaN a NaN;
 *   - affine is a*s+t with two roundings (no fused multiply-add);
 * and where only the device defines behaviour: integer division by zero
 * yields 0 (ew.cl:410), i64 shift counts are masked to 63 (ew.cl:455-457).
 * Float reductions accumulate in double and round once.
 */
#define _GNU_SOURCE
#include <math.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { DT_F32 = 0, DT_I32, DT_U32, DT_BOOL, DT_I64, DT_F64, DT_F16, DT_BF16, DT_MAX = DT_BF16 };
enum { TOP_EW = 0, TOP_MMA, TOP_GATHER, TOP_RED_PART, TOP_RED_COMB, TOP_IOTA_DIM, TOP_SCATTER,
       TOP_DYN_GATHER, TOP_DYN_SCATTER, TOP_RED_WINDOW, TOP_RED_SEG, TOP_SOFTMAX_SEG,
       TOP_LAYERNORM_SEG, TOP_MAP_REGION, TOP_FLASH_ATTN, TOP_RED_STRIDED, TOP_GATHER_INDEX,
       TOP_CONV, TOP_SCATTER_INDEX, TOP_MAX = TOP_SCATTER_INDEX };
enum { SUB_ADD = 0, SUB_MUL, SUB_SUB, SUB_DIV, SUB_MAX, SUB_MIN, SUB_POW, SUB_COPY, SUB_NEG, SUB_EXP,
       SUB_LOG, SUB_SQRT, SUB_RSQRT, SUB_TANH, SUB_ABS, SUB_FLOOR, SUB_CEIL, SUB_SIGN, SUB_FILL,
       SUB_IOTA_FLAT, SUB_CMP, SUB_SELECT, SUB_LTS, SUB_CONVERT, SUB_BITCAST, SUB_ATAN2,
       SUB_REMAINDER, SUB_LOG1P, SUB_EXPM1, SUB_CBRT, SUB_SIN, SUB_COS, SUB_TAN, SUB_RINT, SUB_ROUND,
       SUB_AND, SUB_OR, SUB_XOR, SUB_NOT, SUB_ISFINITE, SUB_AFFINE, SUB_GELU, SUB_SHL, SUB_SHR_L,
       SUB_SHR_A };
enum { K_SUM = 0, K_MAX, K_MIN, K_PROD, K_AND, K_OR, K_XOR };
#define ENT_NOP 0xFFFFFFFFu
#define ENT_BARRIER 0xFFFFFFFEu
#define ENT_WHILE 0xFFFFFFFDu
#define ENT_IF 0xFFFFFFFCu
#define ENT_FOR 0xFFFFFFFBu
#define MAX_DEPTH 8

typedef struct { uint64_t off, size; uint32_t dtype; } vmo_buf;
typedef struct { uint32_t tile_op, dst, a, b, p0, p1, p2, p3, p4, p5, p6, p7; } vmo_task;
typedef struct { uint32_t task, tile_lo, tile_hi, wait_flag, wait_count, signal_flag, slots, pad; } vmo_entry;
typedef struct { uint32_t off, count, root_len, pad; } vmo_lane;

typedef struct vmo_prog {
  uint64_t arena_bytes;
  uint32_t n_buffers, n_inputs, n_outputs, n_aux, n_consts, n_tasks, n_entries, n_lanes;
  vmo_buf *buffers;
  uint32_t *inputs, *outputs;
  int32_t *aux;
  uint32_t *const_id, *const_len;
  const uint8_t **const_data;
  uint8_t *blob; /* private copy (const data points into it) */
  vmo_task *tasks;
  vmo_lane *lanes;
  vmo_entry *entries;
  uint32_t ew_ts, mma_t;
  uint8_t *arena;
} vmo_prog;

static int failf(char *err, size_t cap, const char *fmt, ...) {
  if (err && cap) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, cap, fmt, ap);
    va_end(ap);
  }
  return 1;
}

static size_t dt_size(uint32_t dt) {
  switch (dt) {
    case DT_BOOL: return 1;
    case DT_F16: case DT_BF16: return 2;
    case DT_I64: case DT_F64: return 8;
    default: return 4;
  }
}

/* ---- bit-level float helpers ------------------------------------------- */
static float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
static uint16_t f32_to_bf16(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN stays NaN */
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
static float f16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0) {
    if (!m) return bits_f32(s);
    float v = (float)m * (1.0f / 16777216.0f); /* m * 2^-24 */
    return (h & 0x8000u) ? -v : v;
  }
  if (e == 31) return bits_f32(s | 0x7f800000u | (m << 13));
  return bits_f32(s | ((e + 112u) << 23) | (m << 13));
}
static uint16_t f32_to_f16(float f) {
  uint32_t u = f32_bits(f), s = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(s | 0x7e00u);
  if (a >= 0x47800000u) return (uint16_t)(s | 0x7c00u); /* >= 65536 -> inf (after rounding check below) */
  if (a < 0x33000000u) return (uint16_t)s;            /* < 2^-25 -> 0 */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) { shift = 13 + (-14 - e); base = 0; } else { shift = 13; base = (uint32_t)(e + 15) << 10; }
  uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (e >= -14) q &= 0x3ffu;
  uint32_t r = base + q;
  if (rem > half || (rem == half && (r & 1u))) r++;
  return (uint16_t)(s | r);
}

static float ldf(const void *p, uint32_t dt, size_t i) {
  switch (dt) {
    case DT_F32: return ((const float *)p)[i];
    case DT_F16: return f16_to_f32(((const uint16_t *)p)[i]);
    case DT_BF16: return bf16_to_f32(((const uint16_t *)p)[i]);
    case DT_F64: return (float)((const double *)p)[i];
    case DT_I32: return (float)((const int32_t *)p)[i];
    case DT_U32: return (float)((const uint32_t *)p)[i];
    case DT_I64: return (float)((const int64_t *)p)[i];
    default: return (float)((const uint8_t *)p)[i];
  }
}
static void stf(void *p, uint32_t dt, size_t i, float v) {
  switch (dt) {
    case DT_F32: ((float *)p)[i] = v; break;
    case DT_F16: ((uint16_t *)p)[i] = f32_to_f16(v); break;
    case DT_BF16: ((uint16_t *)p)[i] = f32_to_bf16(v); break;
    case DT_F64: ((double *)p)[i] = v; break;
    default: break;
  }
}
static int is_float_dt(uint32_t dt) { return dt == DT_F32 || dt == DT_F16 || dt == DT_BF16; }

/* ---- parser (runtime.cc:90-251) ---------------------------------------- */
typedef struct { const uint8_t *d; size_t n, pos; } rd_t;
static int rd_u32(rd_t *r, uint32_t *v) { if (r->pos + 4 > r->n) return 0; memcpy(v, r->d + r->pos, 4); r->pos += 4; return 1; }
static int rd_u64(rd_t *r, uint64_t *v) { if (r->pos + 8 > r->n) return 0; memcpy(v, r->d + r->pos, 8); r->pos += 8; return 1; }
static int rd_align8(rd_t *r) { size_t p = (r->pos + 7) & ~(size_t)7; if (p > r->n) return 0; r->pos = p; return 1; }

void vmo_free(vmo_prog *p) {
  if (!p) return;
  free(p->buffers); free(p->inputs); free(p->outputs); free(p->aux);
  free(p->const_id); free(p->const_len); free((void *)p->const_data);
  free(p->tasks); free(p->lanes); free(p->entries); free(p->blob); free(p->arena);
  free(p);
}

int vmo_parse(const uint8_t *data, size_t len, uint32_t ew_ts, uint32_t mma_t, vmo_prog **out,
              char *err, size_t cap) {
  vmo_prog *p = (vmo_prog *)calloc(1, sizeof *p);
  if (!p) return failf(err, cap, "out of memory");
  p->ew_ts = ew_ts; p->mma_t = mma_t;
  p->blob = (uint8_t *)malloc(len ? len : 1);
  memcpy(p->blob, data, len);
  rd_t r = { p->blob, len, 0 };
#define PFAIL(...) do { vmo_free(p); return failf(err, cap, "VMProgram parse error: " __VA_ARGS__); } while (0)
  uint32_t magic, version, n_instrs, main_len, hpad;
  if (!rd_u32(&r, &magic) || !rd_u32(&r, &version)) PFAIL("truncated header");
  if (magic != 0x314D5056u) PFAIL("bad magic");
  if (version != 3) PFAIL("unsupported version %u (executor expects 3)", version);
  if (!rd_u32(&r, &p->n_buffers) || !rd_u32(&r, &n_instrs) || !rd_u32(&r, &p->n_consts) ||
      !rd_u32(&r, &main_len) || !rd_u32(&r, &p->n_inputs) || !rd_u32(&r, &p->n_outputs) ||
      !rd_u32(&r, &p->n_aux) || !rd_u32(&r, &hpad) || !rd_u64(&r, &p->arena_bytes))
    PFAIL("truncated header");
  if ((uint64_t)p->n_buffers * 24 > len) PFAIL("truncated buffer table");
  p->buffers = (vmo_buf *)calloc(p->n_buffers + 1, sizeof(vmo_buf));
  for (uint32_t i = 0; i < p->n_buffers; i++) {
    uint32_t pad;
    vmo_buf *b = &p->buffers[i];
    if (!rd_u64(&r, &b->off) || !rd_u64(&r, &b->size) || !rd_u32(&r, &b->dtype) || !rd_u32(&r, &pad))
      PFAIL("truncated buffer table");
    if (b->dtype > DT_MAX) PFAIL("unsupported dtype %u", b->dtype);
    if (b->off % 4 || b->off + b->size > p->arena_bytes) PFAIL("buffer outside arena / misaligned");
  }
  p->inputs = (uint32_t *)calloc(p->n_inputs + 1, 4);
  p->outputs = (uint32_t *)calloc(p->n_outputs + 1, 4);
  for (uint32_t i = 0; i < p->n_inputs; i++)
    if (!rd_u32(&r, &p->inputs[i]) || p->inputs[i] >= p->n_buffers) PFAIL("bad input map");
  if (!rd_align8(&r)) PFAIL("bad input map");
  for (uint32_t i = 0; i < p->n_outputs; i++)
    if (!rd_u32(&r, &p->outputs[i]) || p->outputs[i] >= p->n_buffers) PFAIL("bad output map");
  if (!rd_align8(&r)) PFAIL("bad output map");
  for (uint32_t i = 0; i < p->n_inputs + p->n_outputs; i++) {
    uint32_t rank, pad;
    if (!rd_u32(&r, &rank) || !rd_u32(&r, &pad) || rank > 16) PFAIL("bad io shapes");
    for (uint32_t d = 0; d < rank; d++) { uint64_t u; if (!rd_u64(&r, &u)) PFAIL("bad io shapes"); }
    if (!rd_align8(&r)) PFAIL("bad io shapes");
  }
  if ((uint64_t)p->n_aux * 4 > len - r.pos) PFAIL("truncated aux");
  p->aux = (int32_t *)calloc(p->n_aux + 1, 4);
  memcpy(p->aux, r.d + r.pos, (size_t)p->n_aux * 4);
  r.pos += (size_t)p->n_aux * 4;
  if (!rd_align8(&r)) PFAIL("aux align");
  p->const_id = (uint32_t *)calloc(p->n_consts + 1, 4);
  p->const_len = (uint32_t *)calloc(p->n_consts + 1, 4);
  p->const_data = (const uint8_t **)calloc(p->n_consts + 1, sizeof(void *));
  for (uint32_t i = 0; i < p->n_consts; i++) {
    if (!rd_u32(&r, &p->const_id[i]) || !rd_u32(&r, &p->const_len[i]) || p->const_id[i] >= p->n_buffers)
      PFAIL("bad const entry");
    if (p->const_len[i] > p->buffers[p->const_id[i]].size) PFAIL("const too big");
    if (r.pos + p->const_len[i] > len) PFAIL("truncated const data");
    p->const_data[i] = r.d + r.pos;
    r.pos += p->const_len[i];
    if (!rd_align8(&r)) PFAIL("truncated const data");
  }
  if (main_len > n_instrs) PFAIL("main_len > n_instrs");
  if ((uint64_t)n_instrs * 32 > len - r.pos) PFAIL("truncated instructions");
  r.pos += (size_t)n_instrs * 32; /* the tensor ISA is not what the device executes */
  if (!rd_align8(&r)) PFAIL("instr align");
  uint32_t n_flags;
  if (!rd_u32(&r, &p->n_tasks) || !rd_u32(&r, &p->n_entries) || !rd_u32(&r, &n_flags) || !rd_u32(&r, &p->n_lanes))
    PFAIL("truncated sched header");
  if (p->n_lanes == 0 || p->n_lanes > 4096) PFAIL("bad n_lanes");
  if ((uint64_t)p->n_tasks * 48 > len - r.pos) PFAIL("truncated tasks");
  p->tasks = (vmo_task *)calloc(p->n_tasks + 1, sizeof(vmo_task));
  memcpy(p->tasks, r.d + r.pos, (size_t)p->n_tasks * 48);
  r.pos += (size_t)p->n_tasks * 48;
  p->lanes = (vmo_lane *)calloc(p->n_lanes, sizeof(vmo_lane));
  for (uint32_t i = 0; i < p->n_lanes; i++) {
    vmo_lane *l = &p->lanes[i];
    if (!rd_u32(&r, &l->off) || !rd_u32(&r, &l->count) || !rd_u32(&r, &l->root_len) || !rd_u32(&r, &l->pad) ||
        l->root_len > l->count)
      PFAIL("truncated/bad lane tab");
  }
  if (!rd_align8(&r)) PFAIL("lane tab align");
  if ((uint64_t)p->n_entries * 32 > len - r.pos) PFAIL("truncated entries");
  p->entries = (vmo_entry *)calloc(p->n_entries + 1, sizeof(vmo_entry));
  memcpy(p->entries, r.d + r.pos, (size_t)p->n_entries * 32);
  r.pos += (size_t)p->n_entries * 32;
  if (r.pos != len) PFAIL("trailing bytes: parsed %zu of %zu", r.pos, len);

  for (uint32_t i = 0; i < p->n_tasks; i++) {
    const vmo_task *t = &p->tasks[i];
    uint32_t op = t->tile_op & 0xFF, dt = (t->tile_op >> 8) & 0xFF;
    if (op > TOP_MAX) PFAIL("unknown tile_op %u", op);
    if (dt > DT_MAX) PFAIL("unknown dtype %u", dt);
    if (t->dst >= p->n_buffers || t->a >= p->n_buffers || t->b >= p->n_buffers)
      PFAIL("task buffer id out of range");
    if (op == TOP_MAP_REGION &&
        (t->p2 >= p->n_buffers || t->p3 >= p->n_buffers || t->p4 >= p->n_buffers ||
         t->p5 >= p->n_buffers || t->p6 >= p->n_buffers || t->p7 >= p->n_buffers))
      PFAIL("region input buffer id out of range");
    if (op == TOP_EW && t->p0 == SUB_SELECT && t->p3 >= p->n_buffers) PFAIL("select pred id out of range");
    if ((op == TOP_GATHER || op == TOP_IOTA_DIM || op == TOP_DYN_GATHER || op == TOP_DYN_SCATTER ||
         op == TOP_RED_WINDOW || op == TOP_GATHER_INDEX || op == TOP_SCATTER_INDEX || op == TOP_SCATTER ||
         op == TOP_CONV) && t->p0 >= p->n_aux)
      PFAIL("task aux offset out of range");
    if (op == TOP_MMA && (t->p4 > p->n_aux || t->p5 > p->n_aux)) PFAIL("mma view aux offset out of range");
    if (op == TOP_FLASH_ATTN && (t->p0 >= p->n_buffers || (uint64_t)t->p3 + 9 > p->n_aux))
      PFAIL("flash-attn V id / aux offset out of range");
  }
  uint32_t ref_barriers = 0;
  for (uint32_t l = 0; l < p->n_lanes; l++) {
    uint32_t off = p->lanes[l].off, count = p->lanes[l].count, barriers = 0;
    if ((uint64_t)off + count > p->n_entries) PFAIL("lane range oob");
    for (uint32_t e = off; e < off + count; e++) {
      const vmo_entry *en = &p->entries[e];
      if (en->task == ENT_BARRIER) barriers++;
      else if (en->task == ENT_WHILE || en->task == ENT_IF) {
        if (en->signal_flag >= p->n_buffers) PFAIL("control cond buffer id out of range");
        if ((uint64_t)en->tile_lo + en->tile_hi > count || (uint64_t)en->wait_flag + en->wait_count > count)
          PFAIL("control sub-range out of lane stream");
      } else if (en->task == ENT_FOR) {
        if ((uint64_t)en->tile_lo + en->tile_hi > count) PFAIL("control sub-range out of lane stream");
      } else if (en->task != ENT_NOP && en->task >= p->n_tasks) PFAIL("entry task index out of range");
    }
    if (l == 0) ref_barriers = barriers;
    else if (barriers != ref_barriers) PFAIL("non-uniform top-level barrier counts across lanes");
  }
#undef PFAIL
  p->arena = (uint8_t *)calloc(p->arena_bytes ? p->arena_bytes : 8, 1);
  if (!p->arena) { vmo_free(p); return failf(err, cap, "arena alloc of %llu bytes failed", (unsigned long long)p->arena_bytes); }
  for (uint32_t i = 0; i < p->n_consts; i++)
    memcpy(p->arena + p->buffers[p->const_id[i]].off, p->const_data[i], p->const_len[i]);
  *out = p;
  return 0;
}

uint32_t vmo_n_inputs(const vmo_prog *p) { return p->n_inputs; }
uint32_t vmo_n_outputs(const vmo_prog *p) { return p->n_outputs; }
uint32_t vmo_n_lanes(const vmo_prog *p) { return p->n_lanes; }
uint64_t vmo_input_bytes(const vmo_prog *p, uint32_t i) { return p->buffers[p->inputs[i]].size; }
uint64_t vmo_output_bytes(const vmo_prog *p, uint32_t i) { return p->buffers[p->outputs[i]].size; }
uint32_t vmo_input_dtype(const vmo_prog *p, uint32_t i) { return p->buffers[p->inputs[i]].dtype; }
uint32_t vmo_output_dtype(const vmo_prog *p, uint32_t i) { return p->buffers[p->outputs[i]].dtype; }
uint64_t vmo_arena_bytes(const vmo_prog *p) { return p->arena_bytes; }

/* ---- tile ops ------------------------------------------------------------ */
#define BUF(p, id) ((p)->arena + (p)->buffers[id].off)

/* strided VIEW index (ew.cl:174-185; shared by gather / viewed EW / MMA / flash) */
static int64_t view_idx(const int32_t *aux, uint32_t off, int64_t i) {
  const int32_t *x = aux + off;
  int rank = x[0];
  const int32_t *dims = x + 1, *strides = x + 1 + rank;
  int64_t rem = i, o = x[1 + 2 * rank];
  for (int e = rank - 1; e >= 0; --e) {
    o += (rem % dims[e]) * (int64_t)strides[e];
    rem /= dims[e];
  }
  return o;
}

static float np_max(float x, float y) { return (x != x || y != y) ? NAN : (x > y ? x : y); }
static float np_min(float x, float y) { return (x != x || y != y) ? NAN : (x < y ? x : y); }
static float gelu_f(float x) {
  float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}
static int ew_is_bin(uint32_t s) { return s <= SUB_POW || (s >= SUB_ATAN2 && s <= SUB_REMAINDER); }
static int ew_is_un(uint32_t s) { return (s >= SUB_COPY && s <= SUB_SIGN) || (s >= SUB_LOG1P && s <= SUB_ROUND) || s == SUB_GELU; }

static float alu_bin(uint32_t sub, float x, float y) {
  switch (sub) {
    case SUB_ADD: return x + y;
    case SUB_MUL: return x * y;
    case SUB_SUB: return x - y;
    case SUB_DIV: return x / y;
    case SUB_MAX: return np_max(x, y);
    case SUB_MIN: return np_min(x, y);
    case SUB_POW: return powf(x, y);
    case SUB_ATAN2: return atan2f(x, y);
    case SUB_REMAINDER: return fmodf(x, y);
    default: return 0.0f;
  }
}
static float alu_un(uint32_t sub, float x) {
  switch (sub) {
    case SUB_COPY: return x;
    case SUB_NEG: return -x;
    case SUB_EXP: return expf(x);
    case SUB_LOG: return logf(x);
    case SUB_SQRT: return sqrtf(x);
    case SUB_RSQRT: return 1.0f / sqrtf(x);
    case SUB_TANH: return tanhf(x);
    case SUB_ABS: return fabsf(x);
    case SUB_FLOOR: return floorf(x);
    case SUB_CEIL: return ceilf(x);
    case SUB_SIGN: return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : x);
    case SUB_LOG1P: return log1pf(x);
    case SUB_EXPM1: return expm1f(x);
    case SUB_CBRT: return cbrtf(x);
    case SUB_SIN: return sinf(x);
    case SUB_COS: return cosf(x);
    case SUB_TAN: return tanf(x);
    case SUB_RINT: return rintf(x);
    case SUB_ROUND: return roundf(x);
    case SUB_GELU: return gelu_f(x);
    default: return 0.0f;
  }
}
/* the straight-line map ALU shared by MAP_REGION and the matmul epilogue
 * (vm_common.cl:173-196; ops/region.py:44-60; ops/dot.py:206-224) */
static float micro_alu(uint32_t kind, float x, float y, float s, float t) {
  switch (kind) {
    case SUB_ADD: return x + y;
    case SUB_MUL: return x * y;
    case SUB_SUB: return x - y;
    case SUB_DIV: return x / y;
    case SUB_MAX: return np_max(x, y);
    case SUB_MIN: return np_min(x, y);
    case SUB_NEG: return -x;
    case SUB_EXP: return expf(x);
    case SUB_LOG: return logf(x);
    case SUB_SQRT: return sqrtf(x);
    case SUB_RSQRT: return 1.0f / sqrtf(x);
    case SUB_TANH: return tanhf(x);
    case SUB_ABS: return fabsf(x);
    case SUB_AFFINE: { volatile float m = x * s; return m + t; }
    case SUB_GELU: return gelu_f(x);
    default: return x;
  }
}

#define CMP(pr, x, y) ((pr) == 0 ? (x) == (y) : (pr) == 1 ? (x) != (y) : (pr) == 2 ? (x) < (y) : \
                       (pr) == 3 ? (x) <= (y) : (pr) == 4 ? (x) > (y) : (x) >= (y))

static int64_t ld_int(const void *p, uint32_t dt, size_t i) {
  switch (dt) {
    case DT_I32: return ((const int32_t *)p)[i];
    case DT_U32: return ((const uint32_t *)p)[i];
    case DT_I64: return ((const int64_t *)p)[i];
    case DT_BOOL: return ((const uint8_t *)p)[i];
    default: return 0;
  }
}
static void st_int(void *p, uint32_t dt, size_t i, int64_t v) {
  switch (dt) {
    case DT_I32: ((int32_t *)p)[i] = (int32_t)(uint32_t)(uint64_t)v; break;
    case DT_U32: ((uint32_t *)p)[i] = (uint32_t)(uint64_t)v; break;
    case DT_I64: ((int64_t *)p)[i] = v; break;
    case DT_BOOL: ((uint8_t *)p)[i] = (uint8_t)v; break;
    default: break;
  }
}

static int ew_range(vmo_prog *p, const vmo_task *t, int64_t lo, int64_t hi, char *err, size_t cap) {
  const uint32_t sub = t->p0, dt = (t->tile_op >> 8) & 0xFF, adt = (t->tile_op >> 16) & 0xFF;
  uint8_t *d = BUF(p, t->dst);
  const uint8_t *a = BUF(p, t->a), *b = BUF(p, t->b);
  if (sub == SUB_CMP) { /* ew.cl:71-94; operands adt -> 1-byte bool */
    const uint32_t pr = t->p2;
    for (int64_t i = lo; i < hi; i++) {
      int r;
      if (is_float_dt(adt)) { float x = ldf(a, adt, i), y = ldf(b, adt, i); r = CMP(pr, x, y); }
      else if (adt == DT_F64) { double x = ((const double *)a)[i], y = ((const double *)b)[i]; r = CMP(pr, x, y); }
      else if (adt == DT_U32) { uint32_t x = ((const uint32_t *)a)[i], y = ((const uint32_t *)b)[i]; r = CMP(pr, x, y); }
      else { int64_t x = ld_int(a, adt, i), y = ld_int(b, adt, i); r = CMP(pr, x, y); }
      d[i] = r ? 1 : 0;
    }
    return 0;
  }
  if (sub == SUB_SELECT) { /* ew.cl:97-127; pred p3 is 1-byte */
    const uint8_t *pr = BUF(p, t->p3);
    size_t es = dt_size(dt);
    for (int64_t i = lo; i < hi; i++) memcpy(d + i * es, (pr[i] ? a : b) + i * es, es);
    return 0;
  }
  if (sub == SUB_BITCAST) { /* ew.cl:594-612 */
    size_t es = dt_size(dt);
    memmove(d + lo * es, a + lo * es, (size_t)(hi - lo) * es);
    return 0;
  }
  if (sub == SUB_ISFINITE) { /* ew.cl:616-636 */
    for (int64_t i = lo; i < hi; i++) {
      double x = adt == DT_F64 ? ((const double *)a)[i] : (double)ldf(a, adt, i);
      d[i] = isfinite(x) ? 1 : 0;
    }
    return 0;
  }
  if (sub == SUB_CONVERT) { /* ew.cl:532-588; ops/making.py:146-160 */
    for (int64_t i = lo; i < hi; i++) {
      if (is_float_dt(adt) || adt == DT_F64) {
        double x = adt == DT_F64 ? ((const double *)a)[i] : (double)ldf(a, adt, i);
        if (is_float_dt(dt)) stf(d, dt, i, (float)x);
        else if (dt == DT_F64) ((double *)d)[i] = x;
        else if (dt == DT_U32) ((uint32_t *)d)[i] = (uint32_t)(int64_t)trunc(x);
        else if (dt == DT_BOOL) d[i] = (uint8_t)(int64_t)trunc(x);
        else st_int(d, dt, i, (int64_t)trunc(x));
      } else {
        if (is_float_dt(dt)) {
          float f = adt == DT_I64 ? (float)((const int64_t *)a)[i]
                  : adt == DT_U32 ? (float)((const uint32_t *)a)[i]
                  : adt == DT_I32 ? (float)((const int32_t *)a)[i] : (float)((const uint8_t *)a)[i];
          stf(d, dt, i, f);
        } else if (dt == DT_F64) ((double *)d)[i] = (double)ld_int(a, adt, i);
        else st_int(d, dt, i, ld_int(a, adt, i));
      }
    }
    return 0;
  }
  if (is_float_dt(dt)) { /* ew.cl:226-353 (f32) and :494-511 (f16/bf16: f32 compute, round on store) */
    const int viewable = ew_is_bin(sub) || ew_is_un(sub);
    const uint32_t av = viewable ? t->p2 : 0, bv = viewable ? t->p3 : 0;
    for (int64_t i = lo; i < hi; i++) {
      float r;
      if (ew_is_bin(sub)) {
        float x = ldf(a, dt, av ? view_idx(p->aux, av - 1, i) : i);
        float y = ldf(b, dt, bv ? view_idx(p->aux, bv - 1, i) : i);
        r = alu_bin(sub, x, y);
      } else if (ew_is_un(sub)) {
        r = alu_un(sub, ldf(a, dt, av ? view_idx(p->aux, av - 1, i) : i));
      } else if (sub == SUB_AFFINE) {
        volatile float m = ldf(a, dt, i) * bits_f32(t->p2);
        r = m + bits_f32(t->p3);
      } else if (sub == SUB_FILL) r = bits_f32(t->p2);
      else if (sub == SUB_IOTA_FLAT) r = (float)i;
      else if (sub == SUB_LTS) { if (i == 0) stf(d, dt, 0, ldf(a, dt, 0) < ldf(b, dt, 0) ? 1.0f : 0.0f); continue; }
      else return failf(err, cap, "EW float: unsupported subop %u", sub);
      stf(d, dt, i, r);
    }
    return 0;
  }
  if (dt == DT_F64) { /* ew.cl:356-391 */
    for (int64_t i = lo; i < hi; i++) {
      double x = ((const double *)a)[i], y = ew_is_bin(sub) ? ((const double *)b)[i] : 0.0, r;
      switch (sub) {
        case SUB_ADD: r = x + y; break; case SUB_MUL: r = x * y; break; case SUB_SUB: r = x - y; break;
        case SUB_DIV: r = x / y; break;
        case SUB_MAX: r = (x != x || y != y) ? NAN : (x > y ? x : y); break;
        case SUB_MIN: r = (x != x || y != y) ? NAN : (x < y ? x : y); break;
        case SUB_POW: r = pow(x, y); break; case SUB_COPY: r = x; break; case SUB_NEG: r = -x; break;
        case SUB_EXP: r = exp(x); break; case SUB_LOG: r = log(x); break; case SUB_SQRT: r = sqrt(x); break;
        case SUB_RSQRT: r = 1.0 / sqrt(x); break; case SUB_TANH: r = tanh(x); break; case SUB_ABS: r = fabs(x); break;
        case SUB_FLOOR: r = floor(x); break; case SUB_CEIL: r = ceil(x); break;
        case SUB_SIGN: r = x > 0 ? 1.0 : (x < 0 ? -1.0 : x); break;
        case SUB_FILL: r = bits_f32(t->p2); break; case SUB_IOTA_FLAT: r = (double)i; break;
        default: return failf(err, cap, "EW f64: unsupported subop %u", sub);
      }
      ((double *)d)[i] = r;
    }
    return 0;
  }
  if (dt == DT_BOOL) { /* ew.cl:469-490 */
    for (int64_t i = lo; i < hi; i++) {
      uint8_t x = a[i], y = b[i], r;
      switch (sub) {
        case SUB_AND: r = x & y; break; case SUB_OR: r = x | y; break; case SUB_XOR: r = x ^ y; break;
        case SUB_NOT: r = x == 0; break; case SUB_COPY: r = x; break;
        case SUB_FILL: r = (uint8_t)t->p2; break;
        case SUB_MAX: r = x > y ? x : y; break; case SUB_MIN: r = x < y ? x : y; break;
        default: return failf(err, cap, "EW bool: unsupported subop %u", sub);
      }
      d[i] = r;
    }
    return 0;
  }
  /* integers: ew.cl:394-463; arithmetic wraps, u32 compares unsigned */
  const int is64 = dt == DT_I64, isu = dt == DT_U32;
  const unsigned smask = is64 ? 63u : 31u;
  for (int64_t i = lo; i < hi; i++) {
    if (sub == SUB_FILL) { st_int(d, dt, i, (int64_t)(int32_t)t->p2); continue; }
    if (sub == SUB_IOTA_FLAT) { st_int(d, dt, i, i); continue; }
    int64_t x = ld_int(a, dt, i);
    const int needs_y = sub <= SUB_POW || sub == SUB_AND || sub == SUB_OR || sub == SUB_XOR ||
                        sub == SUB_SHL || sub == SUB_SHR_L || sub == SUB_SHR_A;
    int64_t y = needs_y ? ld_int(b, dt, i) : 0, r;
    uint64_t ux = (uint64_t)x, uy = (uint64_t)y;
    switch (sub) {
      case SUB_ADD: r = (int64_t)(ux + uy); break;
      case SUB_MUL: r = (int64_t)(ux * uy); break;
      case SUB_SUB: r = (int64_t)(ux - uy); break;
      case SUB_DIV: r = y ? (isu ? (int64_t)(ux / uy) : ((x == INT64_MIN && y == -1) ? x : x / y)) : 0; break;
      case SUB_MAX: r = x > y ? x : y; break;   /* ld_int zero-extends u32, so this is unsigned for u32 */
      case SUB_MIN: r = x < y ? x : y; break;
      case SUB_COPY: r = x; break;
      case SUB_NEG: r = (int64_t)(0 - ux); break;
      case SUB_ABS: r = x < 0 ? (int64_t)(0 - ux) : x; break;
      case SUB_SIGN: r = x > 0 ? 1 : (x < 0 ? -1 : 0); break;
      case SUB_AND: r = x & y; break; case SUB_OR: r = x | y; break; case SUB_XOR: r = x ^ y; break;
      case SUB_NOT: r = ~x; break;
      case SUB_SHL: r = is64 ? (int64_t)(ux << (uy & smask)) : (int64_t)(uint32_t)((uint32_t)ux << (uy & smask)); break;
      case SUB_SHR_L: r = is64 ? (int64_t)(ux >> (uy & smask)) : (int64_t)((uint32_t)ux >> (uy & smask)); break;
      case SUB_SHR_A: r = is64 ? (x >> (uy & smask)) : (int64_t)((int32_t)(uint32_t)ux >> (uy & smask)); break;
      default: return failf(err, cap, "EW int: unsupported subop %u", sub);
    }
    st_int(d, dt, i, r);
  }
  return 0;
}

static void copy_elem(uint8_t *d, int64_t di, const uint8_t *s, int64_t si, size_t es) {
  memcpy(d + di * (int64_t)es, s + si * (int64_t)es, es);
}

/* reductions: kinds of ops/reduce.py:56; float accumulates in double */
typedef struct { double f; int64_t i; uint64_t u; } acc_t;
static void acc_init(acc_t *a, uint32_t kind, uint32_t dt) {
  a->f = kind == K_SUM ? 0.0 : kind == K_PROD ? 1.0 : kind == K_MAX ? -INFINITY : INFINITY;
  if (dt == DT_U32) {
    a->u = kind == K_PROD ? 1 : kind == K_MIN ? 0xFFFFFFFFull : kind == K_AND ? 0xFFFFFFFFull : 0;
  } else if (dt == DT_BOOL) {
    a->u = (kind == K_AND || kind == K_MIN || kind == K_PROD) ? 1 : 0;
  } else {
    a->i = kind == K_SUM ? 0 : kind == K_PROD ? 1
         : kind == K_MAX ? (dt == DT_I64 ? INT64_MIN : INT32_MIN)
         : kind == K_MIN ? (dt == DT_I64 ? INT64_MAX : INT32_MAX) : kind == K_AND ? -1 : 0;
  }
}
static void acc_step(acc_t *a, uint32_t kind, uint32_t dt, const void *src, int64_t i, int *nan) {
  if (is_float_dt(dt) || dt == DT_F64) {
    double v = dt == DT_F64 ? ((const double *)src)[i] : (double)ldf(src, dt, i);
    switch (kind) {
      case K_SUM: a->f += v; break;
      case K_PROD: a->f *= v; break;
      case K_MAX: if (v != v) *nan = 1; else if (v > a->f) a->f = v; break;
      default: if (v != v) *nan = 1; else if (v < a->f) a->f = v; break;
    }
  } else if (dt == DT_U32 || dt == DT_BOOL) {
    uint64_t v = dt == DT_U32 ? ((const uint32_t *)src)[i] : ((const uint8_t *)src)[i];
    switch (kind) {
      case K_SUM: a->u += v; break; case K_PROD: a->u *= v; break;
      case K_MAX: if (v > a->u) a->u = v; break; case K_MIN: if (v < a->u) a->u = v; break;
      case K_AND: a->u &= v; break; case K_OR: a->u |= v; break; default: a->u ^= v; break;
    }
  } else {
    int64_t v = ld_int(src, dt, i);
    switch (kind) {
      case K_SUM: a->i = (int64_t)((uint64_t)a->i + (uint64_t)v); break;
      case K_PROD: a->i = (int64_t)((uint64_t)a->i * (uint64_t)v); break;
      case K_MAX: if (v > a->i) a->i = v; break; case K_MIN: if (v < a->i) a->i = v; break;
      case K_AND: a->i &= v; break; case K_OR: a->i |= v; break; default: a->i ^= v; break;
    }
  }
}
static void acc_store(const acc_t *a, uint32_t kind, uint32_t dt, void *dst, int64_t o, int nan) {
  (void)kind;
  if (is_float_dt(dt)) stf(dst, dt, o, nan ? NAN : (float)a->f);
  else if (dt == DT_F64) ((double *)dst)[o] = nan ? NAN : a->f;
  else if (dt == DT_U32) ((uint32_t *)dst)[o] = (uint32_t)a->u;
  else if (dt == DT_BOOL) ((uint8_t *)dst)[o] = (uint8_t)a->u;
  else st_int(dst, dt, o, a->i);
}

static int64_t dyn_base(vmo_prog *p, const int32_t *x) { /* dynslice.cl:28-42; ops/dynslice.py:144-150 */
  int rank = x[0];
  const int32_t *strides = x + 1 + rank, *cmax = x + 1 + 2 * rank, *bufid = x + 1 + 4 * rank;
  int is64 = x[1 + 5 * rank];
  int64_t base = 0;
  for (int d = 0; d < rank; d++) {
    const uint8_t *ip = BUF(p, (uint32_t)bufid[d]);
    int64_t s = is64 ? *(const int64_t *)ip : *(const int32_t *)ip;
    s = s < 0 ? 0 : (s > cmax[d] ? cmax[d] : s);
    base += s * strides[d];
  }
  return base;
}

static int exec_tiles(vmo_prog *p, const vmo_task *t, uint32_t tlo, uint32_t thi, char *err, size_t cap) {
  const uint32_t op = t->tile_op & 0xFF, dt = (t->tile_op >> 8) & 0xFF, adt = (t->tile_op >> 16) & 0xFF;
  const int64_t TS = p->ew_ts;
  uint8_t *dst = BUF(p, t->dst);
  const uint8_t *a = BUF(p, t->a), *b = BUF(p, t->b);
  const size_t es = dt_size(dt);
  switch (op) {
    case TOP_EW: {
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
      if (lo >= hi) return 0;
      int rc = 0;
      if (t->p0 == SUB_LTS) return ew_range(p, t, lo, hi, err, cap);
      const int64_t CH = 8192;
      int64_t nch = (hi - lo + CH - 1) / CH;
#pragma omp parallel for schedule(static) if (nch > 4)
      for (int64_t c = 0; c < nch; c++) {
        int64_t l = lo + c * CH, h = l + CH < hi ? l + CH : hi;
        if (ew_range(p, t, l, h, err, cap)) rc = 1;
      }
      return rc;
    }
    case TOP_GATHER: { /* gather.cl:9-82; ops/shape.py:196-217 */
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
#pragma omp parallel for schedule(static) if (hi - lo > 65536)
      for (int64_t i = lo; i < hi; i++) copy_elem(dst, i, a, view_idx(p->aux, t->p0, i), es);
      return 0;
    }
    case TOP_SCATTER: { /* scatter.cl:9-50; ops/concat.py:214-236 */
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
      for (int64_t i = lo; i < hi; i++) copy_elem(dst, view_idx(p->aux, t->p0, i), a, i, es);
      return 0;
    }
    case TOP_IOTA_DIM: { /* iota.cl:4-29; ops/making.py:85-117 */
      const int32_t *x = p->aux + t->p0;
      int rank = x[0], dim = x[1 + rank];
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
      for (int64_t i = lo; i < hi; i++) {
        int64_t rem = i, val = 0;
        for (int e = rank - 1; e >= 0; --e) { int64_t c = rem % x[1 + e]; rem /= x[1 + e]; if (e == dim) val = c; }
        if (is_float_dt(dt)) stf(dst, dt, i, (float)val);
        else if (dt == DT_F64) ((double *)dst)[i] = (double)val;
        else st_int(dst, dt, i, val);
      }
      return 0;
    }
    case TOP_DYN_GATHER: case TOP_DYN_SCATTER: { /* dynslice.cl:57-166 */
      const int32_t *x = p->aux + t->p0;
      int rank = x[0];
      int64_t base = dyn_base(p, x), n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
      for (int64_t i = lo; i < hi; i++) {
        int64_t rem = i, o = base;
        for (int e = rank - 1; e >= 0; --e) { o += (rem % x[1 + e]) * (int64_t)x[1 + rank + e]; rem /= x[1 + e]; }
        if (op == TOP_DYN_GATHER) copy_elem(dst, i, a, o, es); else copy_elem(dst, o, a, i, es);
      }
      return 0;
    }
    case TOP_RED_PART: { /* reduce.cl:90-153; ops/reduce.py:307-317 */
      int64_t n = t->p0, chunk = t->p1; uint32_t kind = t->p2;
#pragma omp parallel for schedule(static)
      for (int64_t tile = tlo; tile < (int64_t)thi; tile++) {
        int64_t lo = tile * chunk, hi = lo + chunk < n ? lo + chunk : n;
        if (lo >= hi) continue;
        acc_t acc; int nan = 0;
        acc_init(&acc, kind, dt);
        for (int64_t i = lo; i < hi; i++) acc_step(&acc, kind, dt, a, i, &nan);
        acc_store(&acc, kind, dt, dst, tile, nan);
      }
      return 0;
    }
    case TOP_RED_COMB: { /* reduce.cl:529-549 */
      if (!(tlo == 0 && thi > 0)) return 0;
      acc_t acc; int nan = 0;
      acc_init(&acc, t->p1, dt);
      for (int64_t i = 0; i < (int64_t)t->p0; i++) acc_step(&acc, t->p1, dt, a, i, &nan);
      acc_store(&acc, t->p1, dt, dst, 0, nan);
      return 0;
    }
    case TOP_RED_SEG: { /* reduce.cl:165-281; ops/reduce.py:372-382 */
      int64_t n_out = t->p0, seg = t->p1; uint32_t kind = t->p2;
      int64_t hi = thi < n_out ? thi : n_out;
#pragma omp parallel for schedule(static) if ((hi - (int64_t)tlo) * seg > 65536)
      for (int64_t o = tlo; o < hi; o++) {
        if (t->p3) { /* dot mode: out[o] = sum_j A[o*seg+j] * x[j] */
          double s = 0;
          for (int64_t j = 0; j < seg; j++) s += (double)(ldf(a, adt, o * seg + j) * ldf(b, adt, j));
          stf(dst, dt, o, (float)s);
        } else {
          acc_t acc; int nan = 0;
          acc_init(&acc, kind, dt);
          for (int64_t j = 0; j < seg; j++) acc_step(&acc, kind, dt, a, o * seg + j, &nan);
          acc_store(&acc, kind, dt, dst, o, nan);
        }
      }
      return 0;
    }
    case TOP_RED_STRIDED: { /* reduce.cl:488-527; ops/reduce.py:432-444 */
      int64_t n_out = t->p0, red = t->p1, inner = t->p2; uint32_t kind = t->p3;
      int64_t lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n_out) hi = n_out;
#pragma omp parallel for schedule(static) if ((hi - lo) * red > 65536)
      for (int64_t g = lo; g < hi; g++) {
        int64_t o = g / inner, i = g % inner, base = o * red * inner + i;
        acc_t acc; int nan = 0;
        acc_init(&acc, kind, dt);
        for (int64_t r = 0; r < red; r++) acc_step(&acc, kind, dt, a, base + r * inner, &nan);
        acc_store(&acc, kind, dt, dst, g, nan);
      }
      return 0;
    }
    case TOP_SOFTMAX_SEG: { /* reduce.cl:304-392; ops/reduce.py:464-468 */
      int64_t n_out = t->p0, seg = t->p1, hi = thi < n_out ? thi : n_out;
#pragma omp parallel for schedule(static)
      for (int64_t o = tlo; o < hi; o++) {
        float m = -INFINITY;
        for (int64_t j = 0; j < seg; j++) m = np_max(m, ldf(a, adt, o * seg + j));
        double s = 0;
        for (int64_t j = 0; j < seg; j++) s += (double)expf(ldf(a, adt, o * seg + j) - m);
        float sf = (float)s;
        for (int64_t j = 0; j < seg; j++) stf(dst, dt, o * seg + j, expf(ldf(a, adt, o * seg + j) - m) / sf);
      }
      return 0;
    }
    case TOP_LAYERNORM_SEG: { /* reduce.cl:399-479; ops/reduce.py:471-475: one-pass variance */
      int64_t n_out = t->p0, seg = t->p1, hi = thi < n_out ? thi : n_out;
      float eps = bits_f32(t->p2);
#pragma omp parallel for schedule(static)
      for (int64_t o = tlo; o < hi; o++) {
        double s = 0, s2 = 0;
        for (int64_t j = 0; j < seg; j++) { float x = ldf(a, adt, o * seg + j); s += x; s2 += (double)(x * x); }
        float mu = (float)(s / (double)seg), ex2 = (float)(s2 / (double)seg);
        float var = ex2 - mu * mu;
        float den = sqrtf(var + eps);
        for (int64_t j = 0; j < seg; j++) stf(dst, dt, o * seg + j, (ldf(a, adt, o * seg + j) - mu) / den);
      }
      return 0;
    }
    case TOP_MAP_REGION: { /* region.cl:43-98; ops/region.py:63-84 */
      const int32_t *x = p->aux + t->p0;
      uint32_t n_in = (uint32_t)x[0], out_slot = (uint32_t)x[1], n_micro = (uint32_t)x[2];
      if (n_in > 8) return failf(err, cap, "map-region with %u inputs", n_in);
      const uint32_t ids[8] = { t->a, t->b, t->p2, t->p3, t->p4, t->p5, t->p6, t->p7 };
      const uint8_t *in[8];
      for (uint32_t k = 0; k < n_in; k++) in[k] = BUF(p, ids[k]);
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
      const int32_t *mp = x + 3 + n_in;
#pragma omp parallel for schedule(static) if (hi - lo > 32768)
      for (int64_t i = lo; i < hi; i++) {
        float R[64];
        for (uint32_t k = 0; k < n_in; k++) R[(uint32_t)x[3 + k] & 63] = ldf(in[k], adt, i);
        for (uint32_t m = 0; m < n_micro; m++) {
          const int32_t *q = mp + 6 * m;
          R[(uint32_t)q[1] & 63] = micro_alu((uint32_t)q[0], R[(uint32_t)q[2] & 63], R[(uint32_t)q[3] & 63],
                                             bits_f32((uint32_t)q[4]), bits_f32((uint32_t)q[5]));
        }
        stf(dst, dt, i, R[out_slot & 63]);
      }
      return 0;
    }
    case TOP_MMA: { /* mma.cl:136-434; ops/dot.py:262-293 */
      const int64_t M = t->p0, N = t->p1, K = t->p2, G = t->p3 ? t->p3 : 1, T = p->mma_t;
      const int64_t tn = (N + T - 1) / T, tm = (M + T - 1) / T, per = tm * tn;
      const uint8_t *res = t->p6 ? BUF(p, t->p7) : NULL;
      const uint32_t rdt = t->p6 ? p->buffers[t->p7].dtype : DT_F32;
#pragma omp parallel for schedule(dynamic, 1)
      for (int64_t tile = tlo; tile < (int64_t)thi; tile++) {
        int64_t g = tile / per, loc = tile % per, tr = loc / tn, tc = loc % tn;
        int64_t r0 = tr * T, r1 = r0 + T < M ? r0 + T : M, c0 = tc * T, c1 = c0 + T < N ? c0 + T : N;
        if (g >= G || r0 >= r1 || c0 >= c1) continue;
        int64_t w = c1 - c0;
        float *accv = (float *)malloc((size_t)w * sizeof(float));
        float *brow = (float *)malloc((size_t)w * sizeof(float));
        for (int64_t r = r0; r < r1; r++) {
          for (int64_t c = 0; c < w; c++) accv[c] = 0.0f;
          for (int64_t k = 0; k < K; k++) {
            int64_t ai = (g * M + r) * K + k;
            float av = ldf(a, adt, t->p4 ? view_idx(p->aux, t->p4 - 1, ai) : ai);
            if (t->p5) for (int64_t c = 0; c < w; c++) brow[c] = ldf(b, adt, view_idx(p->aux, t->p5 - 1, (g * K + k) * N + c0 + c));
            else for (int64_t c = 0; c < w; c++) brow[c] = ldf(b, adt, (g * K + k) * N + c0 + c);
            for (int64_t c = 0; c < w; c++) accv[c] += av * brow[c];
          }
          for (int64_t c = 0; c < w; c++) {
            float v = accv[c];
            if (t->p6) { /* store epilogue: mma.cl:74-96 */
              const int32_t *e = p->aux + (t->p6 - 1);
              int nm = e[0];
              for (int m = 0; m < nm; m++) {
                const int32_t *q = e + 1 + 4 * m;
                float y = v;
                if (q[1] == 1) y = ldf(res, rdt, (g * M + r) * N + c0 + c);
                else if (q[1] == 2) y = ldf(res, rdt, c0 + c);
                v = micro_alu((uint32_t)q[0], v, y, bits_f32((uint32_t)q[2]), bits_f32((uint32_t)q[3]));
              }
            }
            stf(dst, dt, (g * M + r) * N + c0 + c, v);
          }
        }
        free(accv); free(brow);
      }
      return 0;
    }
    case TOP_FLASH_ATTN: { /* attention.cl:49-159; ops/attention.py:52-66 */
      const int32_t *x = p->aux + t->p3;
      const int64_t H = x[0], T_ = x[1], C = x[2], hd = x[3];
      const float scale = bits_f32((uint32_t)x[4]);
      const int causal = x[5];
      const uint32_t qv = (uint32_t)x[6], kv = (uint32_t)x[7], vv = (uint32_t)x[8];
      const uint8_t *v = BUF(p, t->p0);
      int64_t hi = (int64_t)thi < H * T_ ? (int64_t)thi : H * T_;
#pragma omp parallel for schedule(dynamic, 8)
      for (int64_t tile = tlo; tile < hi; tile++) {
        int64_t g = tile / T_, m = tile % T_, qpos = m + (C - T_);
        float *sc = (float *)malloc((size_t)C * sizeof(float));
        float mx = -INFINITY;
        for (int64_t c = 0; c < C; c++) {
          float s = 0;
          for (int64_t d = 0; d < hd; d++) {
            int64_t qi = (g * T_ + m) * hd + d, ki = (g * hd + d) * C + c;
            s += ldf(a, adt, qv ? view_idx(p->aux, qv - 1, qi) : qi) * ldf(b, adt, kv ? view_idx(p->aux, kv - 1, ki) : ki);
          }
          s *= scale;
          if (causal && c > qpos) s = -INFINITY;
          sc[c] = s;
          if (s > mx) mx = s;
        }
        double den = 0;
        for (int64_t c = 0; c < C; c++) { sc[c] = expf(sc[c] - mx); den += sc[c]; }
        for (int64_t d = 0; d < hd; d++) {
          double o = 0;
          for (int64_t c = 0; c < C; c++) {
            int64_t vi = (g * C + c) * hd + d;
            o += (double)((sc[c] / (float)den) * ldf(v, adt, vv ? view_idx(p->aux, vv - 1, vi) : vi));
          }
          stf(dst, dt, (g * T_ + m) * hd + d, (float)o);
        }
        free(sc);
      }
      return 0;
    }
    case TOP_RED_WINDOW: { /* reduce_window.cl:19-70; ops/reduce_window.py:160-200 */
      const int32_t *x = p->aux + t->p0;
      const int kind = x[0], rank = x[1];
      const int32_t *od = x + 2, *wd = od + rank, *ws = wd + rank, *pl = ws + rank, *id = pl + rank, *is = id + rank;
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS, wcount = 1;
      if (hi > n) hi = n;
      if (rank > 16) return failf(err, cap, "reduce_window rank %d", rank);
      for (int d = 0; d < rank; d++) wcount *= wd[d];
#pragma omp parallel for schedule(static) if ((hi - lo) * wcount > 65536)
      for (int64_t i = lo; i < hi; i++) {
        int64_t oc[16], rem = i;
        for (int d = rank - 1; d >= 0; --d) { oc[d] = rem % od[d]; rem /= od[d]; }
        acc_t acc; int nan = 0;
        acc_init(&acc, (uint32_t)kind, dt);   /* kinds 0 sum, 1 max, 2 min: the reduce kinds */
        for (int64_t w = 0; w < wcount; w++) {
          int64_t rw = w, off = 0; int inb = 1;
          for (int d = rank - 1; d >= 0; --d) {
            int64_t wc = rw % wd[d]; rw /= wd[d];
            int64_t ic = oc[d] * ws[d] + wc - pl[d];
            if (ic < 0 || ic >= id[d]) inb = 0;
            off += ic * is[d];
          }
          if (inb) acc_step(&acc, (uint32_t)kind, dt, a, off, &nan);   /* padding = the identity: skipped */
        }
        acc_store(&acc, (uint32_t)kind, dt, dst, i, nan);
      }
      return 0;
    }
    case TOP_GATHER_INDEX: case TOP_SCATTER_INDEX: {
      /* gather.cl:84-152, scatter.cl:81-179; ops/gather_index.py:154-186, ops/scatter_index.py:216-260 */
      const int scat = op == TOP_SCATTER_INDEX;
      const int32_t *x = p->aux + t->p0;
      const int rank = x[0], nidx = x[1], vstride = x[2], is64 = x[3], kind = scat ? x[6] : 0;
      const uint32_t idx_buf = (uint32_t)x[5];
      const int32_t *dims = x + (scat ? 7 : 6), *ops = dims + rank, *sis = ops + rank, *ios = sis + rank, *cmax = ios + nidx;
      if (idx_buf >= p->n_buffers) return failf(err, cap, "index buffer id out of range");
      const uint8_t *ib = BUF(p, idx_buf);
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
      /* sequential on purpose: with duplicate indices the update order is the element order
         (np.add.at / maximum.at / minimum.at; plain assignment keeps the last writer) */
      for (int64_t i = lo; i < hi; i++) {
        int64_t rem = i, off = 0, sb = 0;
        for (int e = rank - 1; e >= 0; --e) { int64_t c = rem % dims[e]; rem /= dims[e]; off += c * ops[e]; sb += c * sis[e]; }
        for (int k = 0; k < nidx; k++) {
          int64_t at = sb + (int64_t)k * vstride;
          int64_t sv = is64 ? ((const int64_t *)ib)[at] : ((const int32_t *)ib)[at];
          sv = sv < 0 ? 0 : (sv > cmax[k] ? cmax[k] : sv);
          off += sv * ios[k];
        }
        if (!scat) { copy_elem(dst, i, a, off, es); continue; }
        if (kind == 0) { copy_elem(dst, off, a, i, es); continue; }
        if (dt == DT_F32) {
          float *d = (float *)dst; const float v = ((const float *)a)[i];
          d[off] = kind == 1 ? d[off] + v : kind == 2 ? np_max(d[off], v) : np_min(d[off], v);
        } else if (dt == DT_U32) {
          uint32_t *d = (uint32_t *)dst; const uint32_t v = ((const uint32_t *)a)[i];
          d[off] = kind == 1 ? d[off] + v : kind == 2 ? (d[off] > v ? d[off] : v) : (d[off] < v ? d[off] : v);
        } else if (dt == DT_I32) {
          int32_t *d = (int32_t *)dst; const int32_t v = ((const int32_t *)a)[i];
          d[off] = kind == 1 ? (int32_t)((uint32_t)d[off] + (uint32_t)v) : kind == 2 ? (d[off] > v ? d[off] : v) : (d[off] < v ? d[off] : v);
        } else {
          return failf(err, cap, "scatter combine on dtype %u", dt);
        }
      }
      return 0;
    }
    case TOP_CONV: { /* conv.cl:23-72; ops/conv.py:160-208: f32, accumulate in double */
      const int32_t *x = p->aux + t->p0;
      const int sdim = x[0], Cin = x[1], Cout = x[2];
      const int32_t *osp = x + 3, *win = osp + sdim, *st = win + sdim, *pl = st + sdim, *dil = pl + sdim, *isp = dil + sdim;
      if (sdim < 1 || sdim > 4) return failf(err, cap, "conv spatial rank %d", sdim);
      int64_t istr[4], acc = Cin, wcount = 1;
      for (int d = sdim - 1; d >= 0; --d) { istr[d] = acc; acc *= isp[d]; }
      const int64_t ibatch = acc;
      for (int d = 0; d < sdim; d++) wcount *= win[d];
      int64_t n = t->p1, lo = (int64_t)tlo * TS, hi = (int64_t)thi * TS;
      if (hi > n) hi = n;
      const float *in = (const float *)a, *wt = (const float *)b;
#pragma omp parallel for schedule(static) if ((hi - lo) * wcount * Cin > 65536)
      for (int64_t i = lo; i < hi; i++) {
        int64_t rem = i, oc[4];
        const int64_t co = rem % Cout; rem /= Cout;
        for (int d = sdim - 1; d >= 0; --d) { oc[d] = rem % osp[d]; rem /= osp[d]; }
        const int64_t bi = rem;
        double sum = 0.0;
        for (int64_t w = 0; w < wcount; w++) {
          int64_t rw = w, ioff = bi * ibatch; int inb = 1;
          for (int d = sdim - 1; d >= 0; --d) {
            int64_t wc = rw % win[d]; rw /= win[d];
            int64_t ic = oc[d] * st[d] + wc * dil[d] - pl[d];
            if (ic < 0 || ic >= isp[d]) inb = 0;
            ioff += ic * istr[d];
          }
          if (!inb) continue;
          const int64_t wb = w * Cin * Cout + co;
          for (int c = 0; c < Cin; c++) sum += (double)(in[ioff + c] * wt[wb + (int64_t)c * Cout]);
        }
        ((float *)dst)[i] = (float)sum;
      }
      return 0;
    }
    default:
      return failf(err, cap, "tile op %u is not covered by the oracle", op);
  }
}

/* ---- control walk (vm_main.cl:147-257; vmreader.py:655-773) -------------- */
typedef struct { uint32_t pc, end, widx, phase; } frame_t;
enum { TOK_DONE = 0, TOK_BAR, TOK_FOR_BODY, TOK_WHILE_COND, TOK_WHILE_BODY };

static int cond_is_true(vmo_prog *p, uint32_t buf) {
  uint32_t bits;
  memcpy(&bits, BUF(p, buf), 4);
  return bits != 0u; /* vm_main.cl:178-179 reads the 4-byte word */
}

int vmo_execute(vmo_prog *p, const void *const *inputs, void *const *outputs, int nthreads,
                char *err, size_t cap) {
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#else
  (void)nthreads;
#endif
  for (uint32_t i = 0; i < p->n_inputs; i++)
    memcpy(BUF(p, p->inputs[i]), inputs[i], p->buffers[p->inputs[i]].size);
  const uint32_t L = p->n_lanes;
  frame_t *st = (frame_t *)calloc((size_t)L * (MAX_DEPTH + 1), sizeof(frame_t));
  int *sp = (int *)calloc(L, sizeof(int));
  int *tok = (int *)calloc(L, sizeof(int));
  int rc = 0;
  uint64_t guard = 0;
  for (uint32_t l = 0; l < L; l++) {
    frame_t *f = &st[(size_t)l * (MAX_DEPTH + 1)];
    f->pc = 0; f->end = p->lanes[l].root_len; f->widx = 0xFFFFFFFFu; f->phase = 0;
  }
  for (;;) {
    for (uint32_t l = 0; l < L && !rc; l++) {
      const vmo_entry *stream = p->entries + p->lanes[l].off;
      frame_t *base = &st[(size_t)l * (MAX_DEPTH + 1)];
      for (;;) {
        frame_t *f = &base[sp[l]];
        if (f->pc >= f->end) {
          if (f->widx == 0xFFFFFFFFu) { tok[l] = TOK_DONE; break; }
          const vmo_entry *w = &stream[f->widx];
          if (w->task == ENT_IF) { sp[l]--; base[sp[l]].pc++; continue; }
          if (w->task == ENT_FOR) { tok[l] = TOK_FOR_BODY; break; }
          tok[l] = f->phase == 0 ? TOK_WHILE_COND : TOK_WHILE_BODY;
          break;
        }
        const vmo_entry *e = &stream[f->pc];
        if (e->task == ENT_BARRIER) { tok[l] = TOK_BAR; break; }
        if (e->task == ENT_WHILE || e->task == ENT_FOR || e->task == ENT_IF) {
          uint32_t start, len, phase;
          if (e->task == ENT_WHILE) { start = e->tile_lo; len = e->tile_hi; phase = 0; }
          else if (e->task == ENT_FOR) {
            if (e->wait_flag == 0) { f->pc++; continue; }
            start = e->tile_lo; len = e->tile_hi; phase = e->wait_flag;
          } else {
            int c = cond_is_true(p, e->signal_flag);
            start = c ? e->tile_lo : e->wait_flag; len = c ? e->tile_hi : e->wait_count; phase = 2;
            if (len == 0) { f->pc++; continue; }
          }
          if (sp[l] + 1 > MAX_DEPTH) { rc = failf(err, cap, "control nesting exceeds %d", MAX_DEPTH); break; }
          uint32_t widx = f->pc;
          sp[l]++;
          frame_t *nf = &base[sp[l]];
          nf->pc = start; nf->end = start + len; nf->widx = widx; nf->phase = phase;
          continue;
        }
        if (e->task != ENT_NOP) {
          if (exec_tiles(p, &p->tasks[e->task], e->tile_lo, e->tile_hi, err, cap)) { rc = 1; break; }
        }
        f->pc++;
      }
    }
    if (rc) break;
    int all_done = 1, uniform = 1;
    for (uint32_t l = 0; l < L; l++) { if (tok[l] != TOK_DONE) all_done = 0; if (tok[l] != tok[0]) uniform = 0; }
    if (all_done) break;
    if (!uniform) { rc = failf(err, cap, "non-uniform control across lanes"); break; }
    if (++guard > (1ull << 32)) { rc = failf(err, cap, "runaway loop"); break; }
    for (uint32_t l = 0; l < L; l++) {
      const vmo_entry *stream = p->entries + p->lanes[l].off;
      frame_t *base = &st[(size_t)l * (MAX_DEPTH + 1)];
      frame_t *f = &base[sp[l]];
      const vmo_entry *w = f->widx == 0xFFFFFFFFu ? NULL : &stream[f->widx];
      switch (tok[l]) {
        case TOK_BAR: f->pc++; break;
        case TOK_WHILE_COND:
          if (cond_is_true(p, w->signal_flag)) { f->pc = w->wait_flag; f->end = w->wait_flag + w->wait_count; f->phase = 1; }
          else { sp[l]--; base[sp[l]].pc++; }
          break;
        case TOK_FOR_BODY:
          if (--f->phase != 0) { f->pc = w->tile_lo; f->end = w->tile_lo + w->tile_hi; }
          else { sp[l]--; base[sp[l]].pc++; }
          break;
        default: /* WHILE_BODY -> recheck cond */
          f->pc = w->tile_lo; f->end = w->tile_lo + w->tile_hi; f->phase = 0;
          break;
      }
    }
  }
  free(st); free(sp); free(tok);
  if (rc) return rc;
  for (uint32_t i = 0; i < p->n_outputs; i++)
    memcpy(outputs[i], BUF(p, p->outputs[i]), p->buffers[p->outputs[i]].size);
  return 0;
}
