/* b2vm - C ABI of the B200 device backend for VMProgram v3 bytecode.
 *
 * This is the boundary the reference's PJRT plugin (pjrt_plugin/src/plugin.cc)
 * would bind in place of its OpenCL runtime classes (pjrt_plugin/src/runtime.h).
 * Plain pointers and sizes only; no C++ or torch types cross it; nothing throws.
 * Every function that can fail returns a b2_status (0 = ok) and writes a
 * NUL-terminated message into `err` (may be NULL) of capacity `err_cap`.
 *
 * Ownership follows the reference (runtime.h:309-334): a parsed program is
 * moved into the loaded program by b2_program_load; a loaded program borrows
 * its runtime, which must outlive it; inputs are borrowed for the call; device
 * outputs returned by b2_execute_device belong to the caller and go back to the
 * runtime's size-keyed pool through b2_free.
 *
 * Threading follows the reference (runtime.h:233,301): one mutex per runtime
 * serialises Execute and host<->device copies; the pool has its own lock.
 */
#ifndef B2VM_H_
#define B2VM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; values are the PJRT_Error_Code values plugin.cc maps the
 * reference's bool+string errors onto (plugin.cc:634,754-761,784-790,945-972). */
typedef enum {
  B2_OK = 0,
  B2_INVALID_ARGUMENT = 3,    /* malformed blob, wrong argument count/size */
  B2_DEADLINE_EXCEEDED = 4,   /* a bounded device wait (grid barrier) ran out */
  B2_RESOURCE_EXHAUSTED = 8,  /* device allocation failed */
  B2_FAILED_PRECONDITION = 9, /* no CUDA device, lanes exceed co-residency */
  B2_UNIMPLEMENTED = 12,      /* tile op / dtype outside the backend's coverage */
  B2_INTERNAL = 13            /* CUDA runtime error */
} b2_status;

typedef struct b2_runtime b2_runtime; /* replaces pjrt_ocl::OclRuntime   (runtime.h:120-305) */
typedef struct b2_program b2_program; /* replaces pjrt_ocl::VmProgram    (runtime.h:77-104)  */
typedef struct b2_loaded b2_loaded;   /* replaces pjrt_ocl::LoadedProgram (runtime.h:309-435) */

/* What plugin.cc reads from OclRuntime::info(), ngroups(), ew_ts(), mma_t()
 * (plugin.cc:328,771-773) to describe the device and to tell the lowering
 * subprocess the tile geometry (PJRT_OCL_NLANES / PJRT_OCL_EW_TS / PJRT_OCL_MMA_T). */
typedef struct {
  char device_name[128];
  int device_ordinal;
  int sm_count;
  int cc_major, cc_minor;
  uint64_t total_mem_bytes;
  uint32_t lanes;         /* co-resident CTAs = scheduler lanes to compile for */
  uint32_t ew_ts;         /* elementwise tile size (elements) */
  uint32_t mma_t;         /* matmul output tile edge */
  uint32_t threads_per_lane;
} b2_device_info;

/* Device-side outcome of the last execute of a loaded program. */
typedef struct {
  uint32_t code;          /* 0 ok, 1 barrier wait ran out, 2 control stack overflow,
                             3 unsupported tile op reached, 4 tensor-core wait ran out */
  uint32_t lane;          /* lane that recorded it */
  uint32_t where;         /* barrier index / entry index */
  uint32_t detail;        /* tile op or extra information */
  uint64_t barriers;      /* grid barriers executed by lane 0 */
  uint64_t device_ns;     /* lane 0: globaltimer at exit minus at entry */
} b2_exec_status;

/* ---- runtime (OclRuntime::Create, runtime.cc:255-662) -------------------- */
b2_status b2_runtime_create(int device_ordinal, b2_runtime **out, char *err, size_t err_cap);
void b2_runtime_destroy(b2_runtime *rt);
b2_status b2_runtime_info(const b2_runtime *rt, b2_device_info *out);

/* AllocDevice / PoolAlloc / PoolFree (runtime.cc:2244-2277) and the blocking
 * WriteToDevice / ReadFromDevice (runtime.cc:2279-2301). */
b2_status b2_alloc(b2_runtime *rt, size_t bytes, void **dev_ptr, char *err, size_t err_cap);
b2_status b2_free(b2_runtime *rt, void *dev_ptr, size_t bytes);
b2_status b2_h2d(b2_runtime *rt, void *dev_dst, const void *host_src, size_t bytes, char *err, size_t err_cap);
b2_status b2_d2h(b2_runtime *rt, void *host_dst, const void *dev_src, size_t bytes, char *err, size_t err_cap);

/* ---- program (VmProgram::Parse, runtime.cc:90-251) ----------------------- */
/* Host-only: needs no CUDA device. Applies the same validation as the reference
 * parser and rejects trailing bytes like vmreader.parse (vmreader.py:314-315). */
b2_status b2_program_parse(const uint8_t *blob, size_t len, b2_program **out, char *err, size_t err_cap);
void b2_program_destroy(b2_program *prog);
uint32_t b2_program_num_inputs(const b2_program *prog);
uint32_t b2_program_num_outputs(const b2_program *prog);
uint32_t b2_program_num_lanes(const b2_program *prog);
uint32_t b2_program_num_tasks(const b2_program *prog);
uint64_t b2_program_arena_bytes(const b2_program *prog);
/* is_output: 0 = argument i, 1 = result i. dtype uses the VMProgram enum
 * (f32 0, i32 1, u32 2, bool 3, i64 4, f64 5, f16 6, bf16 7). */
uint64_t b2_program_io_bytes(const b2_program *prog, int is_output, uint32_t i);
uint32_t b2_program_io_dtype(const b2_program *prog, int is_output, uint32_t i);
uint32_t b2_program_io_rank(const b2_program *prog, int is_output, uint32_t i);
int64_t b2_program_io_dim(const b2_program *prog, int is_output, uint32_t i, uint32_t d);

/* ---- loaded program (LoadedProgram::Load, runtime.cc:735-1074) ------------ */
/* Consumes `prog` on success (it is moved into the loaded program). */
b2_status b2_program_load(b2_runtime *rt, b2_program *prog, b2_loaded **out, char *err, size_t err_cap);
void b2_loaded_destroy(b2_loaded *lp);
const b2_program *b2_loaded_program(const b2_loaded *lp);

/* LoadedProgram::Execute (runtime.cc:1103-1177): host arguments to host results,
 * synchronous; inputs[i] holds b2_program_io_bytes(prog, 0, i) bytes. */
b2_status b2_execute_host(b2_loaded *lp, const void *const *inputs, size_t n_inputs,
                          void *const *outputs, size_t n_outputs, char *err, size_t err_cap);

/* LoadedProgram::ExecuteDevice (runtime.cc:2107-2242): device arguments, device
 * results freshly taken from the pool (caller owns, returns them with b2_free);
 * synchronous like the reference's clFinish. */
b2_status b2_execute_device(b2_loaded *lp, void *const *dev_inputs, size_t n_inputs,
                            void **dev_outputs, size_t n_outputs, char *err, size_t err_cap);

/* Same, but the results are written into caller-provided device buffers and the
 * launch is enqueued on `cuda_stream` (a cudaStream_t; NULL = the runtime's own
 * stream) WITHOUT waiting for it: the asynchronous form a CUDA-stream-aware
 * caller uses to overlap copies, collectives and execution. b2_loaded_status
 * waits for that stream and reports the device status of the last launch.
 * A loaded program owns ONE arena and ONE barrier block: its launches must run
 * one after another (enqueue them on one stream, or order the streams with
 * events); two launches of the same loaded program in flight at once corrupt
 * each other. Launches may be queued back to back without fetching the status;
 * if one of them fails on the device (a wait ran out), the launches queued
 * behind it find the abort flag set, return at their first barrier without
 * writing results, and b2_loaded_status reports the first failure - so fetch
 * the status before trusting the results of a pipelined batch.
 * In/out buffers: a program buffer that is one argument and one result and that
 * the program writes (a cache updated in place; the reference copies such donated
 * buffers through its arena, runtime.cc:799-801) is updated in the RESULT's memory.
 * Pass the same address as that argument and that result and nothing is copied;
 * pass different ones and the argument is first copied into the result. */
b2_status b2_execute_device_async(b2_loaded *lp, void *const *dev_inputs, size_t n_inputs,
                                  void *const *dev_outputs, size_t n_outputs,
                                  void *cuda_stream, char *err, size_t err_cap);
b2_status b2_loaded_status(b2_loaded *lp, b2_exec_status *out, char *err, size_t err_cap);
/* The result that argument `input` shares its buffer with when that buffer is an
 * in/out buffer (see b2_execute_device_async), else -1. */
int b2_loaded_in_out_result(const b2_loaded *lp, uint32_t input);
/* Number of kernels launched by this loaded program so far. */
uint64_t b2_loaded_launch_count(const b2_loaded *lp);
/* Load-time facts about how the program was mapped to the device, for tests and
 * logs (no counterpart in the reference). `which`: 0 fused elementwise chains,
 * 1 operands forwarded in registers, 2 intermediate stores elided, 3 matmul
 * tasks, 4 matmul tasks on the tensor-core path, 5 floating-point operations of
 * all matmul tasks per execute (2 G M N K each; a task inside a loop body counts
 * once), 6 flash-attention tasks, 7 flash-attention tasks on the tensor-core path,
 * 8 strided-reduction phases whose few output tiles were re-cut by rows over all
 * lanes, 9 index of the megakernel build the program runs on (0 = the smallest;
 * the library carries several builds, each holding a subset of the tile-op
 * families, and a program runs on the smallest one that has all it uses),
 * 10 bit mask of the tile-op families the program uses, 11 full reductions
 * (RED_PART + RED_COMB) re-cut evenly over all lanes with the combine folded into
 * the same phase, 12 flash-attention tasks on the decode path (few query rows; K and
 * V rows read with 16-byte loads), 13 in/out ports, 14 phases whose units (matmuls of
 * different depth, regions, elementwise chains) were re-cut evenly over all lanes,
 * 15 groups of neighbouring row-local phases (row norms and elementwise chains over
 * the same rows) run as one pipeline per lane with the barriers between them removed,
 * 16 converts from a 16-bit dtype to f32 folded into the full sum that follows them,
 * 17 full sums taken from the row op (softmax / layer norm) that wrote their input,
 * 18 grid barriers between such a row op and its sum that were dropped (they ordered nothing any more),
 * 19 decomposed RMS norms over bf16 rows (convert, square, row sum, scalar region, two broadcast multiplies,
 * convert) run as one row op, 20 barriers dropped because the phase they closed holds nothing after that.
 * Unknown `which` returns 0. */
uint64_t b2_loaded_stat(const b2_loaded *lp, int which);
/* Per-wait budget of device-side bounded waits, in nanoseconds (default 2e9). */
void b2_loaded_set_wait_budget_ns(b2_loaded *lp, uint64_t ns);
/* The time, in ns since kernel entry, at which each of the first grid barriers of
 * the last execute released (every lane had arrived, seen from lane 0) (what the reference prints under
 * PJRT_OCL_PHASE_TS, runtime.cc:2196-2240). Writes at most `cap` values and
 * returns how many were written. */
size_t b2_loaded_phase_ns(const b2_loaded *lp, uint64_t *out, size_t cap);
/* Per-lane timing, off by default (the reference's per-lane barrier timestamps,
 * VMO_TS_REC in vm_common.cl:258-282, read back and summarised by
 * runtime.cc:2196-2240). When on, every lane records its start, its exit and its
 * ARRIVAL at each of the first 64 grid barriers (globaltimer nanoseconds), which
 * is what shows straggler idle: a phase ends at its last arrival, every other
 * lane waited since its own. b2_loaded_lane_times waits for the last launch and
 * copies lanes x 66 values, lane-major: [start, exit, arrival 0 .. arrival 63];
 * returns the number of values written (0 when timing is off). */
b2_status b2_loaded_lane_timing(b2_loaded *lp, int on, char *err, size_t err_cap);
size_t b2_loaded_lane_times(b2_loaded *lp, uint64_t *out, size_t cap);

/* ---- allocation-free full sum (no counterpart in the reference) ------------ */
/* out[0] = sum of the n_elems f32 values at dev_in, for hosts that cannot
 * allocate device memory: a process whose own allocator already holds all of
 * HBM (cudaMalloc - hence b2_program_load - fails there), or a latency path that
 * cannot take the device-wide stall of cudaMalloc / cudaFree. The caller passes
 * input and output; the partial sums live in a fixed 16.3 KB array inside the
 * library (held by every GPU that loads it, until exit), which limits n_elems to
 * b2_sum_f32_static_max_elems() = 536 870 912; more is B2_INVALID_ARGUMENT.
 * Calls no cudaMalloc / cudaFree. Enqueued on `cuda_stream` (NULL = the default
 * stream) and waited for before returning. All calls on one GPU share the array:
 * calls that overlap on the GPU (other threads, other streams) race. The first
 * call on each GPU looks the array's device address up; make it before any
 * stream capture begins. Buffers 4-byte aligned (16-byte aligned input is
 * fastest). */
b2_status b2_sum_f32_static(int device_ordinal, const void *dev_in, uint64_t n_elems, void *dev_out,
                            void *cuda_stream, char *err, size_t err_cap);
uint64_t b2_sum_f32_static_max_elems(void);

#ifdef __cplusplus
}
#endif
#endif /* B2VM_H_ */
