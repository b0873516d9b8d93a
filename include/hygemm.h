/*
 * C ABI of the B200 (sm_100a) hybrid MXFP4/MXFP8 output-channel linear layer.
 *
 * Every symbol the reference's Python binds through ctypes is exported with
 * the same name, argument order and error convention, so the reference's
 * `hygemm_vllm/native.py`, `producer.py` and `fused.py` can load this library
 * unchanged (HYGEMM_LIBRARY / HYGEMM_PRODUCER_LIBRARY / HYGEMM_FUSED_LIBRARY
 * may all point at the one shared object).  The reference's entry points keep
 * their IEEE-half meaning; `_bf16` / `_dtype` twins add bfloat16, the primary
 * type of this build.
 *
 * Ownership: the caller owns every tensor; the library borrows pointers for
 * the duration of the enqueued work and owns only a handle's workspace.
 * Errors: `int` status, 0 = ok, -1 = failure with a thread-local message in
 * hg_last_error() (hg_silu_pack returns a cudaError_t value instead, as the
 * reference does).  No C++ exception crosses the boundary.  All pointers are
 * device pointers unless stated; `stream` is a cudaStream_t.
 *
 * Citations name the reference interface each declaration replaces
 * (paths relative to the reference project root).
 */
#ifndef HYGEMM_B200_H_
#define HYGEMM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One precision partition of a hybrid linear.
 * Replaces hygemm::oc::DeviceProblem (src/kernel/output_channel_gemm.h:14-22)
 * == ctypes `Problem` (integrations/vllm/hygemm_vllm/native.py:7-9).
 * output[token * outputs + ids[row]] = dot(W[row], X[token]). */
typedef struct hg_problem {
  int rows;                      /* weight rows in this partition (0 = partition absent) */
  int tokens;                    /* M */
  int k;                         /* input channels, multiple of 128 */
  int outputs;                   /* N of the full layer (row stride of output) */
  const void* weight;            /* packed E2M1 [rows,k/2] (low) or E4M3 [rows,k] (high) */
  const void* activation;        /* E4M3 [tokens,k], shared by both partitions */
  const void* weight_scales;     /* E8M0, 512-byte atoms of 128 rows x 4 K32 groups */
  const void* activation_scales; /* E8M0, same layout, hg_scale_size(tokens,k) bytes */
  const void* ids;               /* int32 [rows] output channel of each row */
  void* output;                  /* 16-bit float [tokens,outputs] */
} hg_problem;

enum { HG_DTYPE_F16 = 0, HG_DTYPE_BF16 = 1 };

/* Launch policies accepted by hg_run (integrations/vllm/hygemm_vllm/native.py:14-15).
 * 0..3 (serial, concurrent, high_first, high_main) all map to the single
 * tcgen05 launch that covers both partitions; 4..6 select the SIMT pair kernel. */
enum { HG_POLICY_SERIAL = 0, HG_POLICY_CONCURRENT = 1, HG_POLICY_HIGH_FIRST = 2, HG_POLICY_HIGH_MAIN = 3,
       HG_POLICY_GEMV_PAIR1 = 4, HG_POLICY_GEMV_PAIR2 = 5, HG_POLICY_GEMV_PAIR4 = 6 };

/* Schedule ids accepted as low_id/high_id by hg_create (the reference's
 * variant ids, src/kernel/output_channel_gemm.h:41, select CUTLASS tile
 * shapes; here they select the tile schedule of the one tcgen05 kernel). */
enum { HG_SCHEDULE_AUTO = 0,        /* chosen from the shape and the SM count */
       HG_SCHEDULE_DATA_PARALLEL = 1, /* one work unit per output tile */
       HG_SCHEDULE_SPLIT_K = 2,     /* fixed split of K, deterministic fix-up */
       HG_SCHEDULE_STREAM_K = 3,    /* equal k-block share per CTA */
       HG_SCHEDULE_SIMT = 28 };     /* SIMT kernel: the reference's ids 28-34 (output_channel_gemv.cu) all select it */
/* The reference's other variant ids (4-27, 35-44: CUTLASS and cp.async tile shapes) are accepted and run with
 * HG_SCHEDULE_AUTO, so a plan file tuned on the reference's GPU still loads; ids of 45 and above are refused. */

/* integrations/vllm/native/runtime.cu:116 */
const char* hg_last_error(void);

/* integrations/vllm/native/runtime.cu:117-119 — bytes of the padded scale buffer. */
int64_t hg_scale_size(int rows, int k);

/* integrations/vllm/native/runtime.cu:120-134 — quantise IEEE-half [rows,k] to
 * E4M3 (fp4=0) or packed E2M1 (fp4=1) codes plus E8M0 scales; all padding bytes 0x7f. */
int hg_pack(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream);
/* integrations/vllm/native/runtime.cu:135-145 — mode only picks a kernel; bytes are identical. */
int hg_pack_mode(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream, int mode);
/* bfloat16 twins of the two above. */
int hg_pack_bf16(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream);
int hg_pack_mode_bf16(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream, int mode);

/* integrations/vllm/native/producer.cu:46-54 — SwiGLU + MXFP8 quantisation of
 * [rows,2k] gate||up; debug (optional) receives the 16-bit product.  Returns a
 * cudaError_t value (0 = ok). */
int hg_silu_pack(const void* in, void* q, void* sf, void* debug, int rows, int k, void* stream, int math);
int hg_silu_pack_bf16(const void* in, void* q, void* sf, void* debug, int rows, int k, void* stream, int math);

/* integrations/vllm/native/runtime.cu:146-147 — build the schedule and workspace
 * for this exact shape (IEEE-half output).  A partition with rows==0 is skipped. */
int hg_create(int low_id, int high_id, const hg_problem* low, const hg_problem* high, void* stream, void** handle);
/* Same with an explicit output type (HG_DTYPE_*). */
int hg_create_dtype(int low_id, int high_id, const hg_problem* low, const hg_problem* high, void* stream,
                    int dtype, void** handle);
/* integrations/vllm/native/runtime.cu:148-149 — rebind pointers (same shape) and
 * enqueue on `stream`; allocates nothing; may be captured in a CUDA graph.  The kernel starts reading
 * weights, weight scales and ids before it waits for the kernel in front of it in the stream, so those must be
 * complete (not still being written by work queued just before) when the first hg_run on a stream is issued. */
int hg_run(void* handle, const hg_problem* low, const hg_problem* high, void* stream, int policy);
/* hg_pack + hg_run in ONE launch for decode sizes (tokens <= 16): `x` is the 16-bit activation matrix
 * [tokens,k] (x_dtype = HG_DTYPE_*); dedicated quantiser warps of the GEMM kernel convert each CTA's K slice with
 * the arithmetic of hg_pack, so the output equals hg_pack followed by hg_run bit for bit, without the
 * quantiser launch and without the codes and scales passing through HBM.  The problems' `activation` and
 * `activation_scales` are ignored (may be null).  No counterpart in the reference, which always runs its
 * pack kernel first (integrations/vllm/hygemm_vllm/native.py:69-73). */
int hg_run_x(void* handle, const hg_problem* low, const hg_problem* high, const void* x, int x_dtype, void* stream);
/* integrations/vllm/native/runtime.cu:151-161 — 10 ints per partition: id, tile_m,
 * tile_n, tile_k, stages, registers, shared bytes, local bytes, fp8, pingpong (-1 if absent). */
int hg_info(void* handle, int* out20);
/* integrations/vllm/native/runtime.cu:162 */
void hg_destroy(void* handle);
/* Device-side status of the last launches of this handle: 0 = ok, otherwise the
 * code a bounded in-kernel wait recorded before giving up.  status[3] = {error,
 * K128 blocks issued, work units stored} since the last call; clears them and
 * synchronises `stream`.
 * (The reference has no counterpart; its kernels cannot report a stuck wait.) */
int hg_status(void* handle, void* stream, int* status);
/* Host-only view of the tile schedule hg_create would build for a shape on a
 * device with `sms` SMs (no GPU needed; no counterpart in the reference, whose
 * schedules live inside CUTLASS).  header[12] = schedule, grid, n_tile,
 * token_tiles, stages, shared bytes, TMEM columns, workspace slots, counters,
 * units, separate reduce launch (0/1), MMA-issuing threads; units (optional) receives 9 ints per unit: cta, tile, token_tile,
 * kb_begin, kb_end, split, nsplit, ws_slot, counter. */
int hg_plan(int rows_low, int rows_high, int tokens, int k, int sms, int schedule, int* header, int* units,
            int max_units);
/* Diagnostic, only in a library built with -DHG_TRACE (build.py --trace; ordinary builds return -1 with an
 * error): per-CTA time stamps of the handle's last tensor-core launch, 16 per CTA in nanoseconds of the GPU's
 * global timer (0 = point not reached): entry, set-up done, dependency wait released, first full stage, the
 * first four units' last commit, start and end of the first three epilogues.  *values = words written.
 * Synchronises `stream`.  (No counterpart in the reference; `bench.py --timeline` prints the distribution.) */
int hg_trace(void* handle, void* stream, unsigned long long* out, int max_values, int* values);

/* Bytes of the fixed scratch array behind hg_run_static (held on every GPU that loads the library). */
#define HG_STATIC_SCRATCH_BYTES (8u << 20)

/* The hybrid GEMM of hg_create + hg_run in one call that allocates no device memory (no counterpart in
 * the reference, whose handles always own a workspace).  It is for callers that cannot call cudaMalloc
 * where a layer runs: an engine whose memory pool owns the whole device, a latency-critical loop that
 * cannot afford the device-wide synchronisation an allocation implies, or code that meets a shape only
 * when it has to run it and so cannot warm a handle.  The tile schedule, split-K partial sums, arrival
 * counters and status words live in one array of HG_STATIC_SCRATCH_BYTES inside the library image.
 *   - `schedule` is an HG_SCHEDULE_* id 0..3, `dtype` an HG_DTYPE_*; inputs and outputs as for hg_run.
 *   - The first call on a device looks up the array's device address and raises the kernel's
 *     shared-memory limit.
 *   - NOT for stream capture: whenever the array holds another shape's schedule the call copies this
 *     shape's schedule into it from host memory (a copy from pageable memory, which also waits for the
 *     stream), and a captured copy would replay from memory a later call rewrites.  A capturing stream
 *     is refused with -1.  Repeating the shape of the previous call on a device copies nothing.
 *   - Every call uses the same array.  Calls on one stream are safe; calls that overlap on the GPU
 *     (different streams or threads) race.  Arrival counters are cleared at the start of each call.
 *   - A shape whose schedule and partial sums exceed the array returns -1 with a message naming both
 *     sizes; nothing is launched.  Use hg_create/hg_run for such shapes. */
int hg_run_static(int schedule, const hg_problem* low, const hg_problem* high, void* stream, int dtype);
/* hg_status for the hg_run_static calls on the current device since the last read: status[3] = {error code of
 * a bounded in-kernel wait that gave up (0 = none), K128 blocks issued, work units stored}; clears them and
 * synchronises `stream`.  Without it an expired wait on this path would go unseen, as there is no handle to ask. */
int hg_static_status(void* stream, int* status);

/* ---- Row-parallel tensor parallelism: the GEMM writes its partial sums into a peer-mapped buffer and a second
 * kernel pulls and adds the partials of all ranks over NVLink.  No counterpart in the reference, which refuses
 * tensor_parallel_size > 1 (integrations/vllm/hygemm_vllm/quantization.py:81-83).
 *
 * Every rank owns an exchange buffer of 2 x half_bytes and a flag array of `world` ints, both mapped on
 * every peer (CUDA IPC / symmetric memory), plus three private ints of `state` (exchange count, block ticket,
 * status), all zeroed once.  One exchange is two calls on every rank:
 *
 *   hg_run_partial   the GEMM of hg_run (or hg_run_x when `x` is not null), whose scatter epilogue stores this
 *                    rank's partial [tokens,outputs] into one half of its OWN buffer: 16-bit elements, or fp32
 *                    when `f32` is set (decode sizes: the sum is then rounded once, not once per rank).
 *                    `output` of the problems is ignored.
 *   hg_tp_allreduce  publishes "my partial is written" to every peer's flag array, waits (bounded:
 *                    HYGEMM_TP_WAIT_MS, default one second; then status = 1000 + rank waited for, readable
 *                    with hg_tp_status, and `out` is filled with NaN) for all `world` flags in the own array,
 *                    loads the partials of all ranks (`buffers[w]` = rank w's buffer as mapped here, 16-byte
 *                    loads over NVLink, all in flight together) and adds them in rank order into `out`:
 *                    identical bits on every rank.  It then advances `state[0]`.
 *
 * The two halves of a buffer are used alternately (by the parity of state[0] + 1): a rank can only reach the
 * GEMM that overwrites a half after every peer has published the exchange in between, i.e. after every peer
 * has finished reading that half.  Both calls allocate nothing and are graph-capturable: the exchange count
 * lives in device memory.  world <= 8.  Callers poll hg_tp_status at step boundaries. */
#define HG_TP_MAX_WORLD 8
int hg_run_partial(void* handle, const hg_problem* low, const hg_problem* high, const void* x, int x_dtype,
                   void* buffer, int64_t half_bytes, int f32, const int* state, void* stream);
int hg_tp_allreduce(void* const* buffers, void* out, int64_t elems, int64_t half_bytes, int f32, int world, int rank,
                    int* const* flags, int* state, int dtype, void* stream);
/* Reads and clears state[2] (0 = every wait was satisfied). */
int hg_tp_status(int* state, void* stream, int* status);

/* Offline MXFP4 quantiser with an exponent search (integrations/vllm/allocation/fp4_quant.py:28-58,
 * `quantize`; there a chain of torch ops, here one kernel).  `in` is [rows,k] 16-bit (HG_DTYPE_*), `importance`
 * null or k non-negative floats weighting the squared error per input channel.  Per K32 group the
 * round-to-nearest codes and scale of hg_pack(fp4) are the baseline; each non-zero entry of `offsets` (at most
 * 8, in order) moves the scale byte, clamped to [0,254], re-rounds the group (saturating) and wins if its
 * weighted squared error is strictly smaller.  Writes packed codes [rows,k/2] (even k in the low nibble) and
 * LOGICAL scale bytes [rows,k/32] (offline_weights.physical_scales lays them out in atoms). */
int hg_clip_pack(const void* in, const float* importance, void* q4, void* scales, int rows, int k,
                 const int* offsets, int n_offsets, int dtype, void* stream);

/* Single-kernel path kept for binding compatibility
 * (integrations/vllm/native/fused_probe.cu:7-28).  The tcgen05 kernel already
 * covers both partitions in one launch, so these wrap the same implementation
 * with operands fixed at creation. */
const char* hg_fused_error(void);
int hg_fused_create(int id, const hg_problem* low, const hg_problem* high, void* stream, void** handle);
int hg_fused_create_dtype(int id, const hg_problem* low, const hg_problem* high, void* stream, int dtype,
                          void** handle);
int hg_fused_update(void* handle, const hg_problem* low, const hg_problem* high);
int hg_fused_run(void* handle, void* stream);
int hg_fused_info(void* handle, int* out11);
void hg_fused_destroy(void* handle);

#ifdef __cplusplus
}
#endif
#endif /* HYGEMM_B200_H_ */
