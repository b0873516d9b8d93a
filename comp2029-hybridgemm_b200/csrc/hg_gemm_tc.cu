// Hybrid MXFP4xMXFP8 + MXFP8xMXFP8 output-channel GEMM for sm_100a.
//
// One persistent launch covers BOTH precision partitions of a hybrid linear
// (the reference runs two CUTLASS SM120 kernels on two streams,
// integrations/vllm/native/runtime.cu:31-43, or a single-kernel precision
// switch, src/kernel/output_channel_switch_collective.cuh:146-172):
//
//   out[t, ids[r]] = sum_g 2^(sw[r,g]+sx[t,g]-254) * sum_{k in g} W[r,k] * X[t,k]
//
// * MMA shape: tcgen05.mma kind::mxf8f6f4.block_scale, M = 128 weight rows,
//   N = n_tile tokens (16..128), K = 32 per instruction, fp32 accumulators in
//   TMEM.  The A format (E2M1 or E4M3) is chosen per tile, so low and high
//   tiles share one pipeline (stage = two K128 blocks).
// * Operands: activations, MXFP8 weight tiles and both scale streams by TMA
//   (cp.async.bulk.tensor with 128B swizzle, 1-D bulk copies for the scale
//   atoms).  MXFP4 weight tiles by 8-byte cp.async from dedicated loader warps:
//   every 16 packed codes land in the first half of their swizzled 16-byte
//   chunk, which is the 8-bit container the f8f6f4 kinds read, so HBM carries
//   0.5 B/element and every request is a full 128-byte line.
// * Scales: the 512-byte atoms (128 rows x 4 K32 groups) go to TMEM with
//   tcgen05.cp 32x128b.warpx4; the byte of the current K32 block is selected
//   with the a_sf_id/b_sf_id descriptor fields.
// * Issue: up to four MMA-issuing threads in separate warps (two by default),
//   each with its own accumulator: a tcgen05 instruction costs its issuing
//   thread 50-430 cycles whatever its shape (MMA 90, scale copy 51, commit 432)
//   and threads issue in parallel.  Up to 64-token tiles issuer q owns every
//   I-th pipeline stage; wider tiles have a three-stage ring, and there both
//   issuers read every stage, issuer q its K128 block q.
// * Decode sizes (at most 16 tokens) can quantise their activations in the
//   launch: the FUSED instantiation adds four quantiser warps (hg_run_x).
// * Row-parallel tensor parallelism: the epilogue can store the partial result
//   (fp32 for decode sizes) into this rank's half of a peer-mapped exchange
//   buffer (hg_run_partial); hg_tp.cu holds the kernel that pulls every rank's
//   partial over NVLink and adds them.
// * Schedule: a host-built list of work units (row tile, token tile, K range)
//   per CTA: data-parallel, split-K or stream-K.  Tiles cut along K write fp32
//   partials to a workspace; up to 48-token tiles the LAST unit to arrive
//   (one acq_rel ticket, no spinning) sums the partials in K order, wider
//   tiles are summed by splitk_reduce_kernel; either way deterministic.
// * Epilogue: tcgen05.ld 32x32b.x16 (the next sixteen columns in flight while
//   the current ones are stored), accumulators added in a fixed order, fp32 ->
//   bf16/fp16 (RNE), scattered straight to out[t*N + ids[r]] along one running
//   address per sixteen tokens; consecutive lanes own consecutive rows, so
//   sorted maps give contiguous 64-byte runs.  Two accumulator slots (where
//   TMEM holds them: up to 96-token tiles) let the epilogue of one unit overlap
//   the next main loop; MXFP8 tiles, whose stores scatter over the whole row,
//   run first in their CTA for the same reason.
// * Every mbarrier wait is bounded; on expiry the CTA records a code in the
//   status word, lets copies in flight land, frees TMEM and exits.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>

#include "hg_gemm_tc.cuh"

namespace hg {

// ---------------------------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------------------------

// Where the epilogue stores: `ptr` is [tokens, outputs] of 16-bit elements, or of fp32 when `f32` is set.
// For a row-parallel partial (hg_run_partial) `ptr` is this rank's exchange buffer, `epoch` the device word
// that counts finished exchanges and `parity_bytes` the distance between the two halves of the buffer; the
// half written is the one of exchange `*epoch + 1`.
struct OutTargets {
  void* ptr;
  int f32;
  const int* epoch;
  int64_t parity_bytes;
};

// Per-CTA start of the schedule, passed BY VALUE as a kernel parameter: a CTA learns its first work unit
// from the constant bank instead of from two dependent global loads (about a microsecond before the first
// weight request can leave).  Grids larger than kMaxHeads fall back to the arrays in global memory.
constexpr int kMaxHeads = 160;
struct CtaHeads {
  int valid;                   // 0: read cta_begin / units from global memory
  int begin[kMaxHeads + 1];
  WorkUnit first[kMaxHeads];
};

struct TcParams {
  int rows[2];
  int tiles[2];
  const uint8_t* sfa[2];
  const int32_t* ids[2];
  const uint8_t* sfb;
  OutTargets out;
  int outputs, tokens, k, kblocks;
  int n_tile, stages, dtype;
  int issuers;    // MMA-issuing threads = independent accumulators per unit (1, 2 or 4)
  int acc_slots;  // accumulator buffers: 2 lets the epilogue of a unit overlap the next main loop
  int split_blocks;  // 1: both issuers consume every stage, issuer q its K128 block q (wide token tiles)
  int external_reduce;  // cut tiles only store partial sums; splitk_reduce_kernel adds them
  int staged_fixup;     // the last piece of a cut tile sums the pieces from shared memory (bulk copies) when its ring is idle
  const uint8_t* weight_low;
  const uint16_t* x;  // fused mode: 16-bit activations [tokens,k], quantised in the kernel (tokens <= 16); else null
  int x_bf16;
  uint32_t tmem_cols;
  const WorkUnit* units;
  const int* cta_begin;
  float* workspace;
  int* counters;
  int* status;
#ifdef HG_TRACE
  unsigned long long* trace;   // 16 time stamps per CTA, see HG_STAMP
#endif
};

enum : int { kErrProducer = 1, kErrMmaFull = 2, kErrMmaAcc = 3, kErrEpilogue = 4, kErrDrain = 5, kErrLoader = 6 };
// Builds with -DHG_TRACE record, per CTA, the global timer at sixteen points of the kernel (hg_trace reads them
// back; `bench.py --timeline` prints their distribution over the grid).  Slots: 0 entry, 1 set-up done, 2 dependency
// wait released (TMA thread), 3 first full stage seen by issuer 0, 4-7 issuer 0's commit of its first four units,
// 8/9, 10/11, 12/13 start and end of the first three epilogues (thread 64).  Ordinary builds compile none of it.
#ifdef HG_TRACE
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define HG_STAMP(slot) do { if (p.trace) p.trace[blockIdx.x * 16 + (slot)] = global_timer_ns(); } while (0)
#else
#define HG_STAMP(slot) do { } while (0)
#endif

constexpr long long kWaitLimitCycles = 4000000000ll;  // about 2 s at the boost clock, per wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the limit expired or another role of this
// CTA already gave up (abort flag in shared memory).  The clock is only read on
// the slow path, every 256 failed polls (each poll itself blocks in hardware for
// a short, implementation-defined time).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
  for (int burst = 0; burst < 256; ++burst)
    if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
#pragma unroll 1
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - start > kWaitLimitCycles) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_scales(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
__device__ __forceinline__ void tc_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
}
// A register filled by a tcgen05.ld issued before the last tc_wait_ld(): passing it through this (empty)
// volatile statement keeps every use behind that wait, however far ahead the load was issued.
__device__ __forceinline__ uint32_t tc_loaded(uint32_t v) {
  asm volatile("" : "+r"(v));
  return v;
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (tcgen05 format, version 1).
//   bits [0,14) start address >> 4, [16,30) leading byte offset >> 4,
//   [32,46) stride byte offset >> 4, [46,48) version = 1, [61,64) swizzle mode.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  return uint64_t((addr & 0x3ffffu) >> 4) | (uint64_t(lbo >> 4) << 16) | (uint64_t(sbo >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(layout) << 61);
}
constexpr uint32_t kSwizzle128B = 2, kSwizzleNone = 0;

// Instruction descriptor of kind::mxf8f6f4.block_scale:
//   [4,6) B scale id, [7,10) A format (0 E4M3, 5 E2M1), [10,13) B format, [15] A major, [16] B major
//   (0 = K-major), [17,23) N>>3, [23] scale format (1 = UE8M0), [24,29) M>>4, [29,31) A scale id.
__device__ __forceinline__ uint32_t instr_desc(bool a_is_fp4, int n_tile) {
  return (a_is_fp4 ? 5u << 7 : 0u) | (0u << 10) | (uint32_t(n_tile >> 3) << 17) | (1u << 23) |
         (uint32_t(kTileRows >> 4) << 24);
}

__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.b32 p, %1, 0;\n"
      "barrier.cta.red.and.pred q, 1, 128, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}"
      : "=r"(r)
      : "r"(uint32_t(ok))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("barrier.cta.sync 1, 128;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ void scatter_store(const OutTargets& out, char* base, int64_t index, float v) {
  if (out.f32) reinterpret_cast<float*>(base)[index] = v;
  else reinterpret_cast<uint16_t*>(base)[index] = from_float<T>(v);
}

// Start of the output this launch writes: the plain output, or the half of the exchange buffer that belongs
// to the coming exchange.  Read after pdl_wait(): the word is advanced by the kernel that ends the previous exchange.
__device__ __forceinline__ char* out_base(const OutTargets& out) {
  char* base = static_cast<char*>(out.ptr);
  if (!out.epoch) return base;
  const int e = *reinterpret_cast<const volatile int*>(out.epoch) + 1;
  return base + int64_t(e & 1) * out.parity_bytes;
}

// Shared-memory plan.  One pipeline stage covers up to two K128 blocks (K256):
//   A   2 x 16 KiB  weight tiles, 128 rows x 128 B each, 128B-swizzled, K-major
//   B   2 x n_tile x 128 B activation tiles, same layout
//   SFA 2 x 512 B, SFB 2 x 512 B scale atoms
struct SmemLayout {
  uint32_t a, b, sfa, sfb, bars;  // byte offsets from the 1024-aligned base
  uint32_t b_tile;                // bytes of one K128 activation tile
};
__host__ __device__ inline SmemLayout smem_layout(int stages, int n_tile) {
  SmemLayout s;
  s.b_tile = uint32_t(n_tile) * 128u;
  s.a = 0;
  s.b = s.a + uint32_t(stages) * 32768u;
  s.sfa = s.b + uint32_t(stages) * 2u * s.b_tile;
  s.sfb = s.sfa + uint32_t(stages) * 1024u;
  s.bars = s.sfb + uint32_t(stages) * 1024u;
  return s;
}
constexpr int kScaleSets = 2;  // TMEM scale-factor buffers, alternated per K128 block
constexpr int kBarrierBytes = (2 * kMaxStages + 5) * 8 + 32;
constexpr int kLoaderThreads = 128;  // warps 6..9
constexpr int kQuantThreads = 128;   // warps 13..16 (fused activation quantisation)

// 8-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros instead.
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// One arrival on `bar` once every cp.async this thread issued so far has landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// FUSED = true adds the activation-quantiser warps (hg_run_x); the plain instantiation has none, so the
// decode GEMMs on prepacked activations do not carry their threads and registers.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(FUSED ? kTcThreads : kTcThreads - kQuantThreads, 1)
hybrid_gemm_tc_kernel(const __grid_constant__ TcParams p, const __grid_constant__ CUtensorMap map_high,
                      const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CtaHeads heads) {
  pdl_trigger();  // the next kernel in the stream may start its own set-up
  if (threadIdx.x == 0) HG_STAMP(0);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const SmemLayout lay = smem_layout(p.stages, p.n_tile);

  // Barrier block: full[stages], empty[stages], acc_full[2], acc_empty[2], drain, fix-up, then three words.
  const uint32_t bars = base + lay.bars;
  auto full_bar = [&](int s) { return bars + uint32_t(s) * 8u; };
  auto empty_bar = [&](int s) { return bars + uint32_t(p.stages + s) * 8u; };
  auto acc_full_bar = [&](int s) { return bars + uint32_t(2 * p.stages + s) * 8u; };
  auto acc_empty_bar = [&](int s) { return bars + uint32_t(2 * p.stages + 2 + s) * 8u; };
  const uint32_t drain_bar = bars + uint32_t(2 * p.stages + 4) * 8u;
  const uint32_t fix_bar = bars + uint32_t(2 * p.stages + 5) * 8u;   // partial sums of a cut tile landed in shared memory
  volatile int* words = reinterpret_cast<volatile int*>(base_ptr + lay.bars + (2 * p.stages + 6) * 8);
  volatile int* tmem_slot = words;       // TMEM base address written by tcgen05.alloc
  volatile int* abort_flag = words + 1;  // set by the first role whose wait expired
  volatile int* ticket_slot = words + 2; // split-K arrival ticket broadcast

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // The schedule of this CTA is fetched before the set-up barrier so its latency overlaps the set-up.
  int unit_begin, unit_end;
  WorkUnit first_unit{};
  if (heads.valid) {
    unit_begin = heads.begin[blockIdx.x];
    unit_end = heads.begin[blockIdx.x + 1];
    first_unit = heads.first[blockIdx.x];
  } else {
    unit_begin = p.cta_begin[blockIdx.x];
    unit_end = p.cta_begin[blockIdx.x + 1];
    if (unit_begin < unit_end) first_unit = p.units[unit_begin];
  }

  if (threadIdx.x == 0) {
    // a map the launch does not use (no MXFP8 rows; activations quantised in the kernel) arrives as zeros
    if (p.rows[1]) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_high)) : "memory");
    if (!FUSED) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_act)) : "memory");
    for (int s = 0; s < p.stages; ++s) {
      // TMA thread (with the byte count) + every loader thread (+ every quantiser thread in fused mode)
      mbar_init(full_bar(s), 1 + kLoaderThreads + (FUSED ? kQuantThreads : 0));
      mbar_init(empty_bar(s), p.split_blocks ? 2 : 1);   // released by the commit of every issuer that reads the stage
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full_bar(s), uint32_t(p.issuers));
      mbar_init(acc_empty_bar(s), 4);
    }
    mbar_init(drain_bar, uint32_t(p.issuers));
    mbar_init(fix_bar, 1);
    *abort_flag = 0;
    *ticket_slot = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(const_cast<int*>(tmem_slot))), "r"(p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = uint32_t(*tmem_slot);
  if (threadIdx.x == 0) HG_STAMP(1);

  // TMEM columns: acc_slots accumulator slots of issuers x acc_cols columns, then per issuer kScaleSets
  // sets of (SFA, SFB), 4 columns each.
  const uint32_t acc_cols = uint32_t((p.n_tile + 31) & ~31);
  const uint32_t acc_stride = acc_cols * uint32_t(p.issuers);
  const uint32_t sf_cols = tmem_base + uint32_t(p.acc_slots) * acc_stride;

  int error = 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // Activations, both scale streams and MXFP8 weight tiles (128-byte rows).  MXFP4 weight
    // tiles are brought in by the loader warps below.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      // Activations and their scales come from the previous kernel; the MXFP4 weight stream of the loader
      // warps does not and is already running.  (Fused mode: this thread only moves weights and their scales.)
      if (!FUSED) pdl_wait();
      HG_STAMP(2);
      for (int u = unit_begin; u < unit_end && !error; ++u) {
        const WorkUnit wu = u == unit_begin ? first_unit : p.units[u];
        const int part = wu.tile >= p.tiles[0];
        const int tile = part ? wu.tile - p.tiles[0] : wu.tile;
        const int token0 = wu.token_tile * p.n_tile;
        const uint8_t* sfa_src = p.sfa[part] + (int64_t(tile) * p.kblocks) * 512;
        const uint8_t* sfb_src = p.sfb + (int64_t(token0 / 128) * p.kblocks) * 512;
        for (int kb = wu.kb_begin; kb < wu.kb_end; kb += 2) {
          const int nkb = min(2, wu.kb_end - kb);
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { error = kErrProducer; break; }
          const uint32_t bar = full_bar(stage);
          constexpr bool fused = FUSED;  // activations and their scales are then produced by the quantiser warps
          mbar_expect_tx(bar, uint32_t(nkb) * ((part ? 16384u : 0u) + (fused ? 512u : lay.b_tile + 1024u)));
          for (int i = 0; i < nkb; ++i) {
            if (part)
              tma_load_2d(base + lay.a + uint32_t(stage) * 32768u + uint32_t(i) * 16384u, &map_high, bar,
                          (kb + i) * kTileK, tile * kTileRows);
            if (!fused)
              tma_load_2d(base + lay.b + (uint32_t(stage) * 2u + uint32_t(i)) * lay.b_tile, &map_act, bar,
                          (kb + i) * kTileK, token0);
          }
          bulk_load(base + lay.sfa + uint32_t(stage) * 1024u, sfa_src + int64_t(kb) * 512, uint32_t(nkb) * 512u, bar);
          if (!fused)
            bulk_load(base + lay.sfb + uint32_t(stage) * 1024u, sfb_src + int64_t(kb) * 512, uint32_t(nkb) * 512u, bar);
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ------------------------------------------------------------------ MXFP4 weight loaders (warps 6..9)
    // The f8f6f4 MMA kinds read 4-bit operands from an 8-bit container: every 16-byte chunk of a
    // shared-memory row holds 16 codes in its first 8 bytes and 8 bytes of padding.  Each thread copies
    // 8-byte granules of the packed rows (16 codes) straight to the first half of their swizzled chunk
    // with cp.async, so HBM carries 0.5 B/element, requests are full 128-byte lines (sixteen
    // consecutive lanes cover one row's K256 slice) and no register or staging buffer is involved.
    // Thread t owns granule m = t % 16 of rows t / 16 + 8 i; row % 8 is constant per thread, so the
    // swizzle term is too.
    const int t = threadIdx.x - 192;
    const int m = t & 15, rsub = t >> 4;
    const int blk = m >> 3, j = m & 7;
    const uint32_t dst_off = uint32_t(blk) * 16384u + uint32_t(rsub) * 128u + (uint32_t(j ^ rsub) << 4);
    const int64_t pitch = p.k >> 1;  // bytes per packed row
    int stage = 0;
    uint32_t phase = 0;
    for (int u = unit_begin; u < unit_end && !error; ++u) {
      const WorkUnit wu = u == unit_begin ? first_unit : p.units[u];
      const int part = wu.tile >= p.tiles[0];
      const int row0 = wu.tile * kTileRows + rsub;  // first row of this thread (low partition only)
      const uint8_t* src0 = p.weight_low + int64_t(row0) * pitch + m * 8;
      for (int kb = wu.kb_begin; kb < wu.kb_end; kb += 2) {
        const int nkb = min(2, wu.kb_end - kb);
        bool ok = true;
        if (lane == 0) ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
        if (!ok) { error = kErrLoader; break; }
        if (!part && blk < nkb) {
          const uint32_t dst = base + lay.a + uint32_t(stage) * 32768u + dst_off;
          const uint8_t* src = src0 + int64_t(kb) * 64;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const bool valid = row0 + 8 * i < p.rows[0];
            cp_async_8(dst + uint32_t(i) * 1024u, valid ? src + int64_t(8 * i) * pitch : p.weight_low, valid ? 8u : 0u);
          }
        }
        cp_async_arrive(full_bar(stage));
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
      }
    }
    // Copies still in flight must land before shared memory is released.
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (FUSED && warp >= 13) {
    // ------------------------------------------------------------------ activation quantisers (warps 13..16)
    // Fused mode only (decode, at most 16 tokens; p.x != null).  Thread tq owns one K32 group (tq % 8) of
    // token tq / 8 in each K256 stage: same arithmetic as mx_quant_kernel, so codes and
    // scales are the bytes hg_pack would have produced; they go straight to the swizzled activation tile and
    // to the scale atom in shared memory and never touch HBM.  These warps issue no weight copies, so their
    // global loads do not queue behind HBM-latency cp.async traffic, and the NEXT stage's 64 bytes are
    // requested before the current ones are converted.
    if constexpr (FUSED) {
      const int tq = threadIdx.x - 416;
      const int token = tq >> 3, blk_x = (tq & 7) >> 2, g = tq & 3;
      const uint16_t* x_row = p.x + int64_t(token) * p.k + g * 32;
      auto load_x = [&](int kb, int nkb, uint4 (&r)[4]) {
        if (blk_x < nkb && token < p.tokens) {
          const uint4* src = reinterpret_cast<const uint4*>(x_row + int64_t(kb + blk_x) * 128);
#pragma unroll
          for (int c = 0; c < 4; ++c) r[c] = src[c];
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) r[c] = make_uint4(0u, 0u, 0u, 0u);
        }
      };
      uint4 cur[4], nxt[4];
      int stage = 0;
      uint32_t phase = 0;
      int u = unit_begin;
      WorkUnit wu = first_unit;
      int kb = wu.kb_begin;
      pdl_wait();   // x is the previous kernel's output
      if (u < unit_end) load_x(kb, min(2, wu.kb_end - kb), cur);
      while (u < unit_end && !error) {
        const int nkb = min(2, wu.kb_end - kb);
        int next_u = u, next_kb = kb + 2;
        WorkUnit next_wu = wu;
        if (next_kb >= wu.kb_end) {
          ++next_u;
          if (next_u < unit_end) { next_wu = p.units[next_u]; next_kb = next_wu.kb_begin; }
        }
        if (next_u < unit_end) load_x(next_kb, min(2, next_wu.kb_end - next_kb), nxt);
        bool ok = true;
        if (lane == 0) ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
        if (!ok) { error = kErrLoader; break; }
        if (blk_x < nkb) {
          const uint32_t row_base = base + lay.b + (uint32_t(stage) * 2u + uint32_t(blk_x)) * lay.b_tile + uint32_t(token) * 128u;
          const uint32_t sw = uint32_t(token & 7);
          {
            float v[32];
            float amax = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 raw = cur[c];
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const uint16_t bits = uint16_t(w[i >> 1] >> ((i & 1) * 16));
                v[c * 8 + i] = p.x_bf16 ? to_float<__nv_bfloat16>(bits) : to_float<__half>(bits);
                amax = fmaxf(amax, fabsf(v[c * 8 + i]));
              }
            }
            const int e = mx_exponent<false>(amax);
            const float inv = mx_inverse_scale(e);
            uint32_t codes[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              codes[i] = cvt_e4m3x2(v[4 * i] * inv, v[4 * i + 1] * inv) | (cvt_e4m3x2(v[4 * i + 2] * inv, v[4 * i + 3] * inv) << 16);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((uint32_t(2 * g) ^ sw) << 4)),
                         "r"(codes[0]), "r"(codes[1]), "r"(codes[2]), "r"(codes[3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((uint32_t(2 * g + 1) ^ sw) << 4)),
                         "r"(codes[4]), "r"(codes[5]), "r"(codes[6]), "r"(codes[7]) : "memory");
            const uint32_t sf_addr = base + lay.sfb + uint32_t(stage) * 1024u + uint32_t(blk_x) * 512u +
                                     uint32_t(token & 31) * 16u + uint32_t(token >> 5) * 4u + uint32_t(g);
            asm volatile("st.shared.u8 [%0], %1;" ::"r"(sf_addr), "r"(uint32_t(e + 127)) : "memory");
          }
        }
        mbar_arrive(full_bar(stage));   // release: the stores above are visible to whoever acquires the barrier
#pragma unroll
        for (int c = 0; c < 4; ++c) cur[c] = nxt[c];
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        u = next_u; wu = next_wu; kb = next_kb;
      }
    }
  } else if (warp == 1 || (warp >= 10 && warp < 13)) {
    // ------------------------------------------------------------------ MMA issuers (warps 1, 10, 11, 12)
    // A tcgen05 instruction costs its issuing thread on the order of a hundred cycles (descriptor set-up
    // through the uniform datapath) whatever its shape, far more than a 128 x n_tile x 32 MMA occupies the
    // tensor core.  So up to four threads in four warps issue independent streams: issuer q takes every I-th
    // pipeline stage (or, with split_blocks, its K128 block of every stage) and accumulates into its own TMEM
    // accumulator; the epilogue adds the accumulators in a fixed order, which keeps the result deterministic.
    const int q = warp == 1 ? 0 : warp - 9;
    if (lane == 0 && q < p.issuers) {
      uint32_t issued = 0;
      int acc_it = 0;
      uint32_t ring = 0;                                   // pipeline stages consumed by earlier units
      const uint32_t issuer_mask = uint32_t(p.issuers) - 1u;
      int ring_slot = 0;
      uint32_t ring_round = 0;
      const uint32_t sf_base = sf_cols + uint32_t(q) * (8u * kScaleSets);
      uint32_t sf_flip = 0;
      for (int u = unit_begin; u < unit_end && !error; ++u, ++acc_it) {
        const WorkUnit wu = u == unit_begin ? first_unit : p.units[u];
        const int part = wu.tile >= p.tiles[0];
        const int slot = acc_it % p.acc_slots;
        const uint32_t unit_stages = uint32_t(wu.kb_end - wu.kb_begin + 1) >> 1;
        if (!mbar_wait(acc_empty_bar(slot), (uint32_t(acc_it / p.acc_slots) & 1u) ^ 1u, abort_flag)) { error = kErrMmaAcc; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + uint32_t(slot) * acc_stride + uint32_t(q) * acc_cols;
        const uint32_t idesc = instr_desc(part == 0, p.n_tile);
        // SFB of token tile t0 sits in column (t0 % 128) / 32 of its 128-token atom.
        const uint32_t sfb_col = uint32_t((wu.token_tile * p.n_tile) % 128) / 32u;
        // Ownership follows the ring SLOT of the global stage number g: issuer (g % stages) % issuers.  Each
        // ring slot, and with it each full/empty barrier, then has exactly one consumer that sees every round
        // in turn, so parity waits stay unambiguous however short units are.
        // The ring depth is a multiple of the issuer count (1, 2 or 4), so (g % stages) % issuers is g % issuers.
        bool fresh = true;   // this issuer's accumulator has not been written in this unit yet
        for (uint32_t l = 0; l < unit_stages && !error; ++l, ring_slot = ring_slot + 1 == p.stages ? (ring_round ^= 1u, 0) : ring_slot + 1) {
          if (!p.split_blocks && ((ring + l) & issuer_mask) != uint32_t(q)) continue;
          const int kb = wu.kb_begin + 2 * int(l);
          const int nkb = min(2, wu.kb_end - kb);
          const int stage = ring_slot;   // (ring + l) % stages, kept incrementally with its round parity
          if (!mbar_wait(full_bar(stage), ring_round, abort_flag)) { error = kErrMmaFull; break; }
          if (q == 0 && issued == 0) HG_STAMP(3);
          // The MXFP4 rows were written through the generic proxy (cp.async); the tensor core reads
          // shared memory through the async proxy.
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          tc_fence_after();
          for (int i = 0; i < nkb; ++i) {
            if (p.split_blocks && i != q) continue;
            const uint32_t sf_set = sf_base + (sf_flip ^= 1u) * 8u;
            tc_cp_scales(sf_set, smem_desc(base + lay.sfa + uint32_t(stage) * 1024u + uint32_t(i) * 512u, 0, 128, kSwizzleNone));
            tc_cp_scales(sf_set + 4, smem_desc(base + lay.sfb + uint32_t(stage) * 1024u + uint32_t(i) * 512u, 0, 128, kSwizzleNone));
            const uint64_t desc_a = smem_desc(base + lay.a + uint32_t(stage) * 32768u + uint32_t(i) * 16384u, 0, 1024, kSwizzle128B);
            const uint64_t desc_b = smem_desc(base + lay.b + (uint32_t(stage) * 2u + uint32_t(i)) * lay.b_tile, 0, 1024, kSwizzle128B);
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              // 32 K-elements = 32 bytes further along the swizzled row: start address field += 2.
              tc_mma(tmem_d, desc_a + 2 * j, desc_b + 2 * j, idesc | (j << 29) | (j << 4),
                     (!fresh || j > 0) ? 1u : 0u, sf_set, sf_set + 4 + sfb_col);
            }
            fresh = false;
            ++issued;
          }
          // A stage whose second block lies beyond the unit gives the second issuer nothing to read.
          if (p.split_blocks && q >= nkb) mbar_arrive(empty_bar(stage));
          else tc_commit(empty_bar(stage));
        }
        ring += unit_stages;
        // Every issuer reports, also one that had no stage in this unit (its accumulator is then skipped).
        if (!error) tc_commit(acc_full_bar(slot));
        if (q == 0 && acc_it < 4) HG_STAMP(4 + acc_it);
      }
      // Let every MMA issued by this thread retire before TMEM is released.
      tc_commit(drain_bar);
      if (q == 0 && !mbar_wait(drain_bar, 0, abort_flag) && !error) error = kErrDrain;
      if (issued) atomicAdd(p.status + 1, int(issued));
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;                 // TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    int acc_it = 0, stored = 0;
    uint32_t ring = 0;
    pdl_wait();  // nothing is written to global memory before every earlier kernel has finished
    char* const out = out_base(p.out);
    const bool out_f32 = p.out.f32 != 0;
    for (int u = unit_begin; u < unit_end; ++u, ++acc_it) {
      const WorkUnit wu = u == unit_begin ? first_unit : p.units[u];
      const int part = wu.tile >= p.tiles[0];
      const int tile = part ? wu.tile - p.tiles[0] : wu.tile;
      const int slot = acc_it % p.acc_slots;
      const int row = tile * kTileRows + row_in_tile;
      const bool row_ok = row < p.rows[part];
      const int channel = row_ok ? p.ids[part][row] : 0;   // fetched while the main loop runs
      const bool ok = mbar_wait(acc_full_bar(slot), uint32_t(acc_it / p.acc_slots) & 1u, abort_flag);
      if (!epilogue_all(ok)) { error = kErrEpilogue; break; }
      tc_fence_after();
      if (threadIdx.x == 64 && acc_it < 3) HG_STAMP(8 + 2 * acc_it);
      const int token0 = wu.token_tile * p.n_tile;
      // Issuers that owned a stage of this unit (global stages ring .. ring + unit_stages - 1, by ring slot).
      const uint32_t unit_stages = uint32_t(wu.kb_end - wu.kb_begin + 1) >> 1;
      uint32_t owners = 0;
      if (p.split_blocks) owners = wu.kb_end - wu.kb_begin >= 2 ? 3u : 1u;
      else
        for (uint32_t l = 0; l < unit_stages && l < uint32_t(p.issuers); ++l)
          owners |= 1u << ((ring + l) & (uint32_t(p.issuers) - 1u));
      ring += unit_stages;
      const uint32_t taddr = tmem_base + lane_addr + uint32_t(slot) * acc_stride;
      float* ws = wu.nsplit > 1
                      ? p.workspace + (int64_t(wu.ws_slot) + wu.split) * (int64_t(p.n_tile) * kTileRows) + row_in_tile
                      : nullptr;
      // Sixteen columns (tokens) of this thread's row: to the split-K workspace, or scattered to the output.
      // The row stride and the number of valid tokens live in registers: the sixteen addresses are one running sum.
      const int64_t row_stride = p.outputs;
      const int tokens_left = p.tokens - token0;
      auto emit = [&](int c0, const float (&r)[16]) {
        const int valid = tokens_left - c0;
        if (ws) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < valid) ws[int64_t(c0 + i) * kTileRows] = r[i];   // columns nobody will read are skipped
        } else if (row_ok) {
          if (!out_f32) {
            uint16_t* at = reinterpret_cast<uint16_t*>(out) + channel + int64_t(token0 + c0) * row_stride;
#pragma unroll
            for (int i = 0; i < 16; ++i, at += row_stride)
              if (i < valid) *at = from_float<T>(r[i]);
          } else {
            float* at = reinterpret_cast<float*>(out) + channel + int64_t(token0 + c0) * row_stride;
#pragma unroll
            for (int i = 0; i < 16; ++i, at += row_stride)
              if (i < valid) *at = r[i];
          }
        }
      };
      if (!FUSED && p.issuers <= 2 && p.n_tile > 16) {
        // Wide tiles: the TMEM read of the next sixteen columns is in flight while the current sixteen are
        // stored.  The issuers' accumulators are added in the same fixed order as below.
        const bool own0 = owners & 1u, own1 = (owners >> 1) & 1u;
        uint32_t a[16], b[16];
        auto fetch = [&](int c0) {
          if (own0) tc_load16(taddr + uint32_t(c0), a);
          if (own1) tc_load16(taddr + acc_cols + uint32_t(c0), b);
        };
        fetch(0);
        for (int c0 = 0; c0 < p.n_tile; c0 += 16) {
          tc_wait_ld();
          float r[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            r[i] = 0.f;
            if (own0) r[i] += __uint_as_float(tc_loaded(a[i]));
            if (own1) r[i] += __uint_as_float(tc_loaded(b[i]));
          }
          if (c0 + 16 < p.n_tile) fetch(c0 + 16);
          emit(c0, r);
        }
      } else {
        for (int c0 = 0; c0 < p.n_tile; c0 += 16) {
          float r[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = 0.f;
          for (int a = 0; a < p.issuers; ++a) {   // add the issuers' accumulators in a fixed order
            if (!((owners >> a) & 1u)) continue;
            uint32_t e[16];
            tc_load16(taddr + uint32_t(a) * acc_cols + uint32_t(c0), e);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] += __uint_as_float(e[i]);
          }
          emit(c0, r);
        }
      }
      // Accumulator buffer may be overwritten by the next-but-one unit.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(slot));
      if (threadIdx.x == 64 && acc_it < 3) HG_STAMP(9 + 2 * acc_it);

      if (wu.nsplit > 1 && !p.external_reduce) {
        // Deterministic split-K fix-up: the last unit of the tile to arrive sums
        // all partials in K order.  No unit ever waits for another.
        epilogue_sync();
        if (threadIdx.x == 64) {
          // Release (cumulative over the partials of all epilogue threads, which the barrier ordered before
          // this thread) and acquire in one instruction; the barrier below hands the acquired view on.
          int ticket_value;
          asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(ticket_value) : "l"(p.counters + wu.counter) : "memory");
          *ticket_slot = ticket_value;
        }
        epilogue_sync();
        const int ticket = *ticket_slot;
        if (ticket == wu.nsplit - 1) {
          const float* src = p.workspace + int64_t(wu.ws_slot) * (int64_t(p.n_tile) * kTileRows) + row_in_tile;
          // The CTA's last unit: its ring is idle (every stage consumed), so one thread asks for all pieces'
          // partial tiles with bulk copies into it, every byte in flight at once, and the 128 threads add them
          // from shared memory in K order: one memory round trip per batch of columns, and one batch unless
          // the pieces are many and the tile wide.
          const int cols = min(p.n_tile, p.tokens - token0);
          const int batch = min(cols, int((uint32_t(p.stages) * 32768u) / (uint32_t(wu.nsplit) * 512u)));
          // Measured (B200, cold graph burst): above 16 tokens the staged sum wins (o_proj at 32 tokens 14.4 ->
          // 13.8 us, qkv 13.8 -> 12.4, down 19.1 -> 18.2); up to 16 tokens the register path below needs one or
          // two rounds anyway and the extra fence, barrier and copy issue cost 0.2-0.4 us, so it keeps that path.
          if (p.staged_fixup && cols > 16 && u + 1 == unit_end && batch > 0) {
            const float* piece0 = src - row_in_tile;
            uint32_t fix_phase = 0;
            for (int cbase = 0; cbase < cols && !error; cbase += batch) {
              const int nc = min(batch, cols - cbase);
              if (threadIdx.x == 64) {
                // the other pieces were written through the generic proxy and acquired by the ticket above;
                // the bulk copies read them through the async proxy
                asm volatile("fence.proxy.async;" ::: "memory");
                mbar_expect_tx(fix_bar, uint32_t(wu.nsplit * nc) * 512u);
                for (int s = 0; s < wu.nsplit; ++s)
                  bulk_load(base + lay.a + uint32_t(s * nc) * 512u,
                            piece0 + (int64_t(s) * p.n_tile + cbase) * kTileRows, uint32_t(nc) * 512u, fix_bar);
              }
              const bool landed = mbar_wait(fix_bar, fix_phase, abort_flag);
              fix_phase ^= 1u;
              if (!epilogue_all(landed)) { error = kErrEpilogue; break; }
              if (row_ok) {
                // four columns x four pieces per round: sixteen independent shared-memory loads in flight,
                // additions in K order
                const uint32_t piece_stride = uint32_t(nc) * 512u;
                const uint32_t row_addr = base + lay.a + uint32_t(row_in_tile) * 4u;
                for (int c = 0; c < nc; c += 4) {
                  float sum[4] = {0.f, 0.f, 0.f, 0.f};
                  for (int s0 = 0; s0 < wu.nsplit; s0 += 4) {
                    float v[4][4];
#pragma unroll
                    for (int ds = 0; ds < 4; ++ds)
#pragma unroll
                      for (int j = 0; j < 4; ++j) {
                        v[ds][j] = 0.f;
                        if (s0 + ds < wu.nsplit && c + j < nc)
                          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[ds][j])
                                       : "r"(row_addr + uint32_t(s0 + ds) * piece_stride + uint32_t(c + j) * 512u));
                      }
#pragma unroll
                    for (int ds = 0; ds < 4; ++ds)
                      if (s0 + ds < wu.nsplit) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) sum[j] += v[ds][j];
                      }
                  }
#pragma unroll
                  for (int j = 0; j < 4; ++j)
                    if (c + j < nc)
                      scatter_store<T>(p.out, out, int64_t(token0 + cbase + c + j) * p.outputs + channel, sum[j]);
                }
              }
              if (cbase + batch < cols) epilogue_sync();   // everyone has read this batch before the next one lands
            }
            if (error) break;
          } else if (row_ok) {
            // Eight columns x four pieces per round: all loads of a round are in flight together (each is an
            // L2 round trip), the additions keep K order.  Columns beyond the token count are not read.
            for (int c = 0; c < p.n_tile && token0 + c < p.tokens; c += 8) {
              float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              for (int s0 = 0; s0 < wu.nsplit; s0 += 4) {
                float v[4][8];
#pragma unroll
                for (int ds = 0; ds < 4; ++ds)
#pragma unroll
                  for (int i = 0; i < 8; ++i)
                    v[ds][i] = (s0 + ds < wu.nsplit && token0 + c + i < p.tokens)
                                   ? __ldcg(src + (int64_t(s0 + ds) * p.n_tile + c + i) * kTileRows) : 0.f;
#pragma unroll
                for (int ds = 0; ds < 4; ++ds)
                  if (s0 + ds < wu.nsplit) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) sum[i] += v[ds][i];
                  }
              }
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (token0 + c + i < p.tokens)
                  scatter_store<T>(p.out, out, int64_t(token0 + c + i) * p.outputs + channel, sum[i]);
            }
          }
          if (threadIdx.x == 64) p.counters[wu.counter] = 0;  // ready for the next launch
        }
        epilogue_sync();  // ticket_slot is reused by the next unit
      }
      ++stored;
    }
    if (threadIdx.x == 64 && stored) atomicAdd(p.status + 2, stored);
  }

  if (error) {
    *abort_flag = 1;
    atomicCAS(p.status, 0, error * 1000000 + int(blockIdx.x));
    // Give copies and MMAs in flight time to land before shared memory and TMEM are released.
    const long long start = clock64();
    while (clock64() - start < 400000ll) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
  }

}

// Fixed-order sum of the partial tiles of every cut (tile, token tile) for wide token tiles
// (the counterpart of the reference's reduce kernel, src/kernel/output_channel_gemv.cu:73-81).
// One block per (cut tile, 8 token columns), one thread per weight row.
struct ReduceParams {
  int rows[2];
  int tiles[2];
  const int32_t* ids[2];
  OutTargets out;
  int outputs, tokens, n_tile;
  const float* workspace;
  const int* cut_tiles;   // 4 ints each: tile, token_tile, ws_slot, nsplit
};

template <typename T>
__global__ void __launch_bounds__(kTileRows)
splitk_reduce_kernel(const ReduceParams rp) {
  pdl_trigger();
  pdl_wait();  // the partial sums come from the GEMM launched just before
  const int column_blocks = rp.n_tile >> 3;
  const int cut = blockIdx.x / column_blocks, c0 = (blockIdx.x % column_blocks) * 8;
  const int tile_v = rp.cut_tiles[4 * cut], token_tile = rp.cut_tiles[4 * cut + 1];
  const int slot = rp.cut_tiles[4 * cut + 2], nsplit = rp.cut_tiles[4 * cut + 3];
  const int part = tile_v >= rp.tiles[0];
  const int row = (part ? tile_v - rp.tiles[0] : tile_v) * kTileRows + int(threadIdx.x);
  if (row >= rp.rows[part]) return;
  const int channel = rp.ids[part][row];
  char* const out = out_base(rp.out);
  const int token0 = token_tile * rp.n_tile + c0;
  const float* src = rp.workspace + int64_t(slot) * (int64_t(rp.n_tile) * kTileRows) + int64_t(c0) * kTileRows + threadIdx.x;
  float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < nsplit; ++s) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sum[i] += __ldcg(src + (int64_t(s) * rp.n_tile + i) * kTileRows);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (token0 + i < rp.tokens) scatter_store<T>(rp.out, out, int64_t(token0 + i) * rp.outputs + channel, sum[i]);
}

// ---------------------------------------------------------------------------------------------
// Host side: schedule
// ---------------------------------------------------------------------------------------------

static int round_up(int v, int m) { return (v + m - 1) / m * m; }
// HYGEMM_TC_STAGED_FIXUP=0: the last piece of a cut tile always sums the pieces with loads from global memory.
static bool staged_fixup() {
  static const bool value = [] { const char* t = std::getenv("HYGEMM_TC_STAGED_FIXUP"); return !(t && t[0] == '0'); }();
  return value;
}
constexpr int kMaxDynamicSmem = 232448;  // 227 KiB, the per-CTA limit of sm_100

Plan make_plan(int rows_low, int rows_high, int tokens, int k, int sms, int schedule) {
  Plan plan;
  const int tiles_low = (rows_low + kTileRows - 1) / kTileRows, tiles_high = (rows_high + kTileRows - 1) / kTileRows;
  const int tiles = tiles_low + tiles_high, kblocks = k / kTileK;
  plan.n_tile = tokens >= 128 ? 128 : std::max(16, round_up(tokens, 16));
  // 65..128 tokens on a layer with few row tiles: two 64-token tiles instead of one wide one.  The work
  // items double (qkv 36 -> 72, o_proj 28 -> 56), each moves a third fewer bytes through its SM and two MMA
  // issuers fit (qkv / o_proj at 128 tokens: 19.6 -> 13.1 us, down 33.7 -> 30.7 us).  Wide layers keep the
  // 128-token tile: the weights would be streamed twice (gate_up: 32.3 -> 37.6 us).
  if (tokens > 64 && tokens <= 128 && 2 * tiles <= sms) plan.n_tile = 64;
  if (const char* cap = std::getenv("HYGEMM_TC_NTILE")) {  // tuning aid: cap the token tile (a multiple of 16)
    const int capped = std::max(16, std::min(plan.n_tile, std::atoi(cap) / 16 * 16));
    // Several token tiles per 128-token scale atom are only laid out for 64-token tiles (the activation
    // scale columns of a tile must start on an even TMEM column); narrower caps apply to a single tile only.
    if (capped >= 64 || tokens <= capped) plan.n_tile = capped;
  }
  plan.token_tiles = (tokens + plan.n_tile - 1) / plan.n_tile;
  // A tile's activation scales sit in TMEM column (token0 % 128) / 32 of their atom; an odd column there made
  // the MMA raise "misaligned address", so token tiles narrower than 64 must be alone in the call.
  if (plan.n_tile < 64 && plan.token_tiles > 1) throw std::runtime_error("Token tiles narrower than 64 cannot share a scale atom");
  const int stage_bytes = 32768 + 2 * plan.n_tile * 128 + 2048;  // one K256 stage: weights, activations, scales
  plan.stages = std::min(kMaxStages, (kMaxDynamicSmem - 1024 - kBarrierBytes) / stage_bytes);
  if (const char* cap = std::getenv("HYGEMM_TC_STAGES"))  // tuning aid: cap the pipeline depth
    plan.stages = std::max(2, std::min(plan.stages, std::atoi(cap)));
  plan.smem_bytes = 1024 + plan.stages * stage_bytes + kBarrierBytes;
  // MMA-issuing threads: two.  Up to n_tile = 64 they own alternate stages and TMEM (512 columns) holds two
  // double-buffered accumulators per issuer; the pipeline depth is then kept a multiple of the issuer count
  // so that the issuers own equally many ring slots and each stage barrier has one consumer (five stages
  // shared 3:2 measured slower than four shared 2:2).
  plan.issuers = plan.n_tile <= 64 ? 2 : 1;
  if (const char* cap = std::getenv("HYGEMM_TC_ISSUERS"))  // tuning aid: 1, 2 or 4
    plan.issuers = std::max(1, std::min(plan.n_tile <= 32 ? 4 : plan.n_tile <= 64 ? 2 : 2, std::atoi(cap)));
  if (plan.issuers == 3) plan.issuers = 2;
  // Wider tiles have a three-stage ring, so the two issuers share EVERY stage instead, issuer q taking its K128
  // block q: each stage barrier keeps both consumers in every round, so the depth need not be a multiple of
  // the issuer count.  At n_tile = 128 TMEM then holds one accumulator per issuer (the epilogue is no longer
  // overlapped); the halved issue time per stage outweighs that (gate_up at 128 tokens 32.6 -> 30.6 us, at 96
  // tokens, where two accumulator slots still fit, 30.5 -> 25.6 us).
  plan.split_blocks = 0;
  const char* split_text = std::getenv("HYGEMM_TC_SPLIT_BLOCKS");   // tuning aid: 0 never, 1 above 64 tokens, 2 always
  const int split_mode = split_text ? std::atoi(split_text) : 1;
  if (plan.n_tile > 64 && plan.issuers == 1 && split_mode != 0) { plan.split_blocks = 1; plan.issuers = 2; }
  else if (plan.issuers == 2 && split_mode == 2) plan.split_blocks = 1;
  plan.acc_slots = plan.issuers * 2 * round_up(plan.n_tile, 32) + plan.issuers * 8 * kScaleSets <= 512 ? 2 : 1;
  if (!plan.split_blocks) plan.stages = std::max(plan.issuers, plan.stages / plan.issuers * plan.issuers);
  plan.smem_bytes = 1024 + plan.stages * stage_bytes + kBarrierBytes;
  int cols = plan.issuers * (plan.acc_slots * round_up(plan.n_tile, 32) + 8 * kScaleSets), pow2 = 32;
  while (pow2 < cols) pow2 *= 2;
  plan.tmem_cols = pow2;

  // Cost of one K128 block of a tile in HBM bytes (weights dominate): E2M1 8 KiB, E4M3 16 KiB.
  auto weight = [&](int tile) { return tile < tiles_low ? 1 : 2; };
  const int items = tiles * plan.token_tiles;
  int64_t total_cost = 0;
  for (int t = 0; t < tiles; ++t) total_cost += int64_t(weight(t)) * kblocks * plan.token_tiles;
  plan.grid = int(std::min<int64_t>(sms, std::max<int64_t>(1, items)));

  auto greedy = [&](std::vector<WorkUnit> units, std::vector<int64_t> cost) {
    // Longest-processing-time assignment of whole units to CTAs.
    std::vector<int> order(units.size());
    for (size_t i = 0; i < order.size(); ++i) order[i] = int(i);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
    const int grid = int(std::min<size_t>(size_t(sms), std::max<size_t>(1, units.size())));
    std::vector<std::vector<int>> per(grid);
    std::vector<int64_t> load(grid, 0);
    for (int i : order) {
      int best = int(std::min_element(load.begin(), load.end()) - load.begin());
      per[best].push_back(i);
      load[best] += cost[i];
    }
    plan.grid = grid;
    plan.units.clear();
    plan.cta_begin.assign(1, 0);
    for (auto& list : per) {
      // Costlier units first, then by position.  An MXFP8 tile scatters its outputs to channels all over the
      // row (one sector per element); run first, that epilogue hides under the next unit's main loop instead
      // of ending the CTA.
      std::sort(list.begin(), list.end(), [&](int a, int b) { return cost[a] != cost[b] ? cost[a] > cost[b] : a < b; });
      for (int i : list) plan.units.push_back(units[i]);
      plan.cta_begin.push_back(int(plan.units.size()));
    }
    return *std::max_element(load.begin(), load.end());
  };

  // Data-parallel candidate.
  std::vector<WorkUnit> dp;
  std::vector<int64_t> dp_cost;
  for (int t = 0; t < tiles; ++t)
    for (int tt = 0; tt < plan.token_tiles; ++tt) {
      dp.push_back(WorkUnit{t, tt, 0, kblocks, 0, 1, 0, 0});
      dp_cost.push_back(int64_t(weight(t)) * kblocks);
    }

  auto split_k = [&](int splits) {
    std::vector<WorkUnit> units;
    std::vector<int64_t> cost;
    int slots = 0, counters = 0;
    for (int t = 0; t < tiles; ++t)
      for (int tt = 0; tt < plan.token_tiles; ++tt) {
        const int s_tile = std::min(splits * weight(t), kblocks);
        for (int s = 0; s < s_tile; ++s) {
          const int b = int(int64_t(kblocks) * s / s_tile), e = int(int64_t(kblocks) * (s + 1) / s_tile);
          units.push_back(WorkUnit{t, tt, b, e, s, s_tile, slots, counters});
          cost.push_back(int64_t(weight(t)) * (e - b));
        }
        if (s_tile > 1) { slots += s_tile; ++counters; }
        else units.back().nsplit = 1;
      }
    plan.ws_slots = slots;
    plan.counters = counters;
    return greedy(units, cost);
  };

  auto stream_k = [&]() {
    // Equal share of cost per CTA.  The ideal cut points (in cost units) are mapped
    // to (item, K128 block) positions and snapped to the item boundary when they
    // would leave a piece shorter than kMinBlocks (short pieces only add fix-up
    // traffic), so every CTA's load is within about one block of the ideal share.
    const int kMinBlocks = 2;
    plan.grid = int(std::max<int64_t>(1, std::min<int64_t>(sms, total_cost / (2 * kMinBlocks))));
    std::vector<int64_t> start(items + 1, 0);   // cumulative cost at the start of each (tile, token tile)
    for (int i = 0; i < items; ++i) start[i + 1] = start[i] + int64_t(weight(i / plan.token_tiles)) * kblocks;
    std::vector<int64_t> cut(plan.grid + 1, 0);  // positions in blocks: item * kblocks + kb
    cut[plan.grid] = int64_t(items) * kblocks;
    int item = 0;
    for (int c = 1; c < plan.grid; ++c) {
      const int64_t v = total_cost * c / plan.grid;
      while (item + 1 < items && start[item + 1] <= v) ++item;
      const int w = weight(item / plan.token_tiles);
      int kb = int((v - start[item] + w / 2) / w);
      if (kb < kMinBlocks) kb = 0;
      if (kblocks - kb < kMinBlocks) kb = kblocks;
      cut[c] = std::max(cut[c - 1], int64_t(item) * kblocks + kb);
    }
    plan.units.clear();
    plan.cta_begin.assign(1, 0);
    std::vector<int> pieces(items, 0);
    for (int c = 0; c < plan.grid; ++c) {
      for (int64_t pos = cut[c]; pos < cut[c + 1];) {
        const int i = int(pos / kblocks), kb = int(pos % kblocks);
        const int end = int(std::min<int64_t>(kblocks, cut[c + 1] - int64_t(i) * kblocks));
        plan.units.push_back(WorkUnit{i / plan.token_tiles, i % plan.token_tiles, kb, end, pieces[i]++, 1, 0, 0});
        pos = int64_t(i) * kblocks + end;
      }
      plan.cta_begin.push_back(int(plan.units.size()));
    }
    int slots = 0, counters = 0;
    std::vector<int> slot_of(items, 0), counter_of(items, 0);
    for (int i = 0; i < items; ++i)
      if (pieces[i] > 1) { slot_of[i] = slots; counter_of[i] = counters++; slots += pieces[i]; }
    for (auto& unit : plan.units) {
      const int i = unit.tile * plan.token_tiles + unit.token_tile;
      unit.nsplit = pieces[i];
      unit.ws_slot = slot_of[i];
      unit.counter = counter_of[i];
    }
    plan.ws_slots = slots;
    plan.counters = counters;
  };

  if (schedule == HG_SCHEDULE_AUTO) {
    // Measured on B200 (Qwen2.5-7B layer shapes, M = 1..128): whole tiles win once there are about
    // 1.5 tiles per SM, and also for wide token tiles unless K is long, because the fix-up traffic of a
    // cut tile grows with n_tile (n_tile x 128 fp32 partials written and read per piece); otherwise
    // stream-K, which keeps every SM streaming.
    const bool many_tiles = 2 * items >= 3 * sms;
    const bool wide_short = plan.n_tile >= 64 && kblocks < 64;
    schedule = (many_tiles || wide_short) ? HG_SCHEDULE_DATA_PARALLEL : HG_SCHEDULE_STREAM_K;
  }
  plan.ws_slots = 0;
  plan.counters = 0;
  if (schedule == HG_SCHEDULE_DATA_PARALLEL) {
    greedy(dp, dp_cost);
  } else if (schedule == HG_SCHEDULE_SPLIT_K) {
    const int splits = std::max<int>(1, std::min<int64_t>(kblocks, (2 * int64_t(sms) * kblocks + total_cost - 1) / std::max<int64_t>(1, total_cost)));
    split_k(splits);
  } else if (schedule == HG_SCHEDULE_STREAM_K) {
    stream_k();
  } else {
    throw std::runtime_error("Unknown tile schedule id");
  }
  plan.schedule = schedule;
  // With wide token tiles the partial sums of a cut tile are large (n_tile x 128 fp32 per piece) and only
  // one CTA per tile, the last to arrive, would sum them while the others sit idle: measured 68 us for
  // down at M = 128.  From n_tile = 64 on, a second, fully parallel kernel does the fixed-order sum.
  plan.external_reduce = plan.n_tile >= 64 && plan.ws_slots > 0;
  plan.cut_tiles.clear();
  if (plan.external_reduce) {
    std::vector<char> seen(size_t(tiles) * plan.token_tiles, 0);
    for (const WorkUnit& unit : plan.units) {
      const size_t item = size_t(unit.tile) * plan.token_tiles + unit.token_tile;
      if (unit.nsplit > 1 && !seen[item]) {
        seen[item] = 1;
        plan.cut_tiles.insert(plan.cut_tiles.end(), {unit.tile, unit.token_tile, unit.ws_slot, unit.nsplit});
      }
    }
  }
  return plan;
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor maps, handle, launch
// ---------------------------------------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(ptr);
  });
  if (!fn) throw std::runtime_error("cuTensorMapEncodeTiled is not available from this driver");
  return fn;
}

// 2-D K-major tensor map over E4M3 bytes: dim0 = K, dim1 = rows; box = 128 x box_rows, 128B swizzle.
static CUtensorMap make_map(const void* ptr, int rows, int k, int box_rows) {
  CUtensorMap map;
  std::memset(&map, 0, sizeof(map));
  const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(k)};
  const cuuint32_t box[2] = {128u, cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult r = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box,
                                    elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return map;
}

static CtaHeads make_heads(const Plan& plan) {
  CtaHeads heads{};
  static const bool enabled = [] { const char* t = std::getenv("HYGEMM_TC_HEADS"); return !t || std::atoi(t) != 0; }();
  if (plan.grid > kMaxHeads || !enabled) return heads;
  heads.valid = 1;
  for (int c = 0; c <= plan.grid; ++c) heads.begin[c] = plan.cta_begin[c];
  for (int c = 0; c < plan.grid; ++c)
    if (plan.cta_begin[c] < plan.cta_begin[c + 1]) heads.first[c] = plan.units[plan.cta_begin[c]];
  return heads;
}

struct TcGemm {
  Plan plan;
  CtaHeads heads{};
  int rows[2] = {0, 0}, tokens = 0, k = 0, outputs = 0, dtype = HG_DTYPE_BF16;
  WorkUnit* d_units = nullptr;
  int* d_cta_begin = nullptr;
  float* d_workspace = nullptr;
  int* d_counters = nullptr;
  int* d_status = nullptr;
  int* d_cut = nullptr;
#ifdef HG_TRACE
  unsigned long long* d_trace = nullptr;
#endif
  // Tensor maps of recent operand pointers (the shape is fixed per handle): a serving loop alternates among
  // a few activation buffers and one weight pointer, so the driver call is paid once per pointer.
  struct CachedMap { const void* ptr = nullptr; CUtensorMap map; };
  CachedMap act_maps[4], high_map;
  int act_next = 0;
};

void validate(const hg_problem& l, const hg_problem& h, bool fused) {
  const hg_problem& any = l.rows ? l : h;
  if (l.rows < 0 || h.rows < 0 || l.rows + h.rows == 0) throw std::runtime_error("Hybrid GEMM needs at least one weight row");
  if (any.tokens <= 0 || any.k <= 0 || any.k % 128 || any.outputs <= 0) throw std::runtime_error("Invalid hybrid GEMM shape");
  if (l.rows && h.rows &&
      (l.tokens != h.tokens || l.k != h.k || l.outputs != h.outputs || l.output != h.output ||
       (!fused && (l.activation != h.activation || l.activation_scales != h.activation_scales))))
    throw std::runtime_error("Low and high partitions must share activation, scales and output");
  auto misaligned = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  for (const hg_problem* q : {&l, &h}) {
    if (!q->rows) continue;
    if (!q->weight || (!fused && (!q->activation || !q->activation_scales)) || !q->weight_scales || !q->ids || !q->output)
      throw std::runtime_error("Null pointer in hybrid GEMM problem");
    if (misaligned(q->weight, 32) || misaligned(q->activation, 16) || misaligned(q->weight_scales, 16) ||
        misaligned(q->activation_scales, 16) || misaligned(q->ids, 4) || misaligned(q->output, 2))
      throw std::runtime_error("Hybrid GEMM operands must be aligned (weights 32 B, codes and scales 16 B)");
  }
}

// The limit is a property of the function, not of a handle: always raise it to the device maximum so
// handles with different stage counts can coexist.
template <typename T>
static void configure_kernel() {
  check(cudaFuncSetAttribute(hybrid_gemm_tc_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem),
        "cudaFuncSetAttribute");
  check(cudaFuncSetAttribute(hybrid_gemm_tc_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem),
        "cudaFuncSetAttribute");
}

TcGemm* tc_create(const hg_problem& l, const hg_problem& h, int schedule, int dtype, cudaStream_t stream) {
  validate(l, h);
  if (dtype != HG_DTYPE_F16 && dtype != HG_DTYPE_BF16) throw std::runtime_error("Unknown output dtype");
  const hg_problem& any = l.rows ? l : h;
  int device = 0, sms = 0;
  check(cudaGetDevice(&device), "cudaGetDevice");
  check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "SM count");
  auto g = std::make_unique<TcGemm>();
  g->rows[0] = l.rows; g->rows[1] = h.rows;
  g->tokens = any.tokens; g->k = any.k; g->outputs = any.outputs; g->dtype = dtype;
  g->plan = make_plan(l.rows, h.rows, any.tokens, any.k, sms, schedule);
  g->heads = make_heads(g->plan);
  const Plan& plan = g->plan;
  check(cudaMalloc(&g->d_units, sizeof(WorkUnit) * std::max<size_t>(1, plan.units.size())), "cudaMalloc units");
  check(cudaMalloc(&g->d_cta_begin, sizeof(int) * plan.cta_begin.size()), "cudaMalloc schedule");
  check(cudaMalloc(&g->d_workspace, sizeof(float) * std::max<int64_t>(1, int64_t(plan.ws_slots) * plan.n_tile * kTileRows)), "cudaMalloc workspace");
  check(cudaMalloc(&g->d_counters, sizeof(int) * std::max(1, plan.counters)), "cudaMalloc counters");
    check(cudaMalloc(&g->d_status, sizeof(int) * 4), "cudaMalloc status");
  check(cudaMalloc(&g->d_cut, sizeof(int) * std::max<size_t>(4, plan.cut_tiles.size())), "cudaMalloc cut list");
#ifdef HG_TRACE
  check(cudaMalloc(&g->d_trace, sizeof(unsigned long long) * 16 * size_t(plan.grid)), "trace buffer");
  check(cudaMemsetAsync(g->d_trace, 0, sizeof(unsigned long long) * 16 * size_t(plan.grid), stream), "trace buffer");
#endif
  if (!plan.cut_tiles.empty())
    check(cudaMemcpyAsync(g->d_cut, plan.cut_tiles.data(), sizeof(int) * plan.cut_tiles.size(), cudaMemcpyHostToDevice, stream), "upload cut list");
  check(cudaMemcpyAsync(g->d_units, plan.units.data(), sizeof(WorkUnit) * plan.units.size(), cudaMemcpyHostToDevice, stream), "upload units");
  check(cudaMemcpyAsync(g->d_cta_begin, plan.cta_begin.data(), sizeof(int) * plan.cta_begin.size(), cudaMemcpyHostToDevice, stream), "upload schedule");
  check(cudaMemsetAsync(g->d_counters, 0, sizeof(int) * std::max(1, plan.counters), stream), "clear counters");
  check(cudaMemsetAsync(g->d_status, 0, sizeof(int) * 4, stream), "clear status");
  check(cudaStreamSynchronize(stream), "schedule upload");  // host vectors are pageable
  if (dtype == HG_DTYPE_BF16) configure_kernel<__nv_bfloat16>();
  else configure_kernel<__half>();
  return g.release();
}

// Second launch of a call whose cut tiles are summed outside the GEMM kernel.
static void launch_reduce(const Plan& plan, const TcParams& p, const int* cut_tiles, int dtype, cudaStream_t stream, bool pdl) {
  if (!plan.external_reduce || plan.cut_tiles.empty()) return;
  ReduceParams rp{};
  rp.rows[0] = p.rows[0]; rp.rows[1] = p.rows[1];
  rp.tiles[0] = p.tiles[0]; rp.tiles[1] = p.tiles[1];
  rp.ids[0] = p.ids[0]; rp.ids[1] = p.ids[1];
  rp.out = p.out; rp.outputs = p.outputs; rp.tokens = p.tokens; rp.n_tile = p.n_tile;
  rp.workspace = p.workspace; rp.cut_tiles = cut_tiles;
  const dim3 grid(unsigned(plan.cut_tiles.size() / 4 * size_t(plan.n_tile / 8))), block(kTileRows);
  if (pdl) {
    check(dtype == HG_DTYPE_BF16 ? launch_kernel(splitk_reduce_kernel<__nv_bfloat16>, grid, block, 0, stream, rp)
                                 : launch_kernel(splitk_reduce_kernel<__half>, grid, block, 0, stream, rp), "split-K reduce launch");
  } else {
    if (dtype == HG_DTYPE_BF16) splitk_reduce_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(rp);
    else splitk_reduce_kernel<__half><<<grid, block, 0, stream>>>(rp);
    check(cudaGetLastError(), "split-K reduce launch");
  }
}

// Everything of the kernel parameters that follows from the problems and the plan; the caller adds the
// output target, the fused activations and the schedule / scratch pointers.
static TcParams base_params(const Plan& plan, const hg_problem& l, const hg_problem& h, int dtype) {
  const hg_problem& any = l.rows ? l : h;
  TcParams p{};
  p.rows[0] = l.rows; p.rows[1] = h.rows;
  p.tiles[0] = (l.rows + kTileRows - 1) / kTileRows; p.tiles[1] = (h.rows + kTileRows - 1) / kTileRows;
  p.sfa[0] = static_cast<const uint8_t*>(l.weight_scales); p.sfa[1] = static_cast<const uint8_t*>(h.weight_scales);
  p.ids[0] = static_cast<const int32_t*>(l.ids); p.ids[1] = static_cast<const int32_t*>(h.ids);
  p.sfb = static_cast<const uint8_t*>(any.activation_scales);
  p.outputs = any.outputs; p.tokens = any.tokens; p.k = any.k; p.kblocks = any.k / kTileK;
  p.n_tile = plan.n_tile; p.stages = plan.stages; p.dtype = dtype; p.tmem_cols = uint32_t(plan.tmem_cols);
  p.issuers = plan.issuers;
  p.acc_slots = plan.acc_slots;
  p.split_blocks = plan.split_blocks;
  p.external_reduce = plan.external_reduce ? 1 : 0;
  p.staged_fixup = staged_fixup() ? 1 : 0;
  p.weight_low = static_cast<const uint8_t*>(l.weight);
  return p;
}

void tc_run(TcGemm* g, const hg_problem& l, const hg_problem& h, cudaStream_t stream, const void* x, int x_dtype,
            const PartialTarget* partial) {
  const bool fused = x != nullptr;
  validate(l, h, fused);
  if (fused) {
    if (g->plan.n_tile != 16) throw std::runtime_error("Fused activation quantisation serves at most 16 tokens");
    if (x_dtype != HG_DTYPE_F16 && x_dtype != HG_DTYPE_BF16) throw std::runtime_error("Unknown activation dtype");
    if (reinterpret_cast<uintptr_t>(x) & 15) throw std::runtime_error("Activations must be 16-byte aligned");
  }
  const hg_problem& any = l.rows ? l : h;
  if (l.rows != g->rows[0] || h.rows != g->rows[1] || any.tokens != g->tokens || any.k != g->k || any.outputs != g->outputs)
    throw std::runtime_error("Hybrid GEMM handle was created for a different shape");
  const Plan& plan = g->plan;
  TcParams p = base_params(plan, l, h, g->dtype);
  if (partial) {
    // This rank's exchange buffer (two halves); decode sizes travel as fp32 so the sum is rounded once.
    if (!partial->buffer || !partial->state) throw std::runtime_error("Null exchange buffer or state");
    if (reinterpret_cast<uintptr_t>(partial->buffer) & 15 || partial->half_bytes % 16) throw std::runtime_error("Exchange buffer halves must be 16-byte aligned");
    if (partial->half_bytes < int64_t(any.tokens) * any.outputs * (partial->f32 ? 4 : 2))
      throw std::runtime_error("Exchange buffer half smaller than tokens x outputs");
    p.out.ptr = partial->buffer;
    p.out.f32 = partial->f32 ? 1 : 0;
    p.out.epoch = partial->state;
    p.out.parity_bytes = partial->half_bytes;
  } else {
    p.out.ptr = any.output;
  }
  p.x = static_cast<const uint16_t*>(x);
  p.x_bf16 = x_dtype == HG_DTYPE_BF16;
  p.units = g->d_units; p.cta_begin = g->d_cta_begin;
  p.workspace = g->d_workspace; p.counters = g->d_counters; p.status = g->d_status;
#ifdef HG_TRACE
  p.trace = g->d_trace;
#endif
  // Tensor maps by operand pointer.  A map that the launch does not use (no MXFP8 rows; activations
  // quantised in the kernel) is passed as zeros and never touched by the kernel.
  static const CUtensorMap no_map{};
  const CUtensorMap* map_act = &no_map;
  if (!fused) {
    TcGemm::CachedMap* hit = nullptr;
    for (auto& entry : g->act_maps)
      if (entry.ptr == any.activation) hit = &entry;
    if (!hit) {
      hit = &g->act_maps[g->act_next];
      g->act_next = (g->act_next + 1) % 4;
      hit->map = make_map(any.activation, any.tokens, any.k, plan.n_tile);
      hit->ptr = any.activation;
    }
    map_act = &hit->map;
  }
  const CUtensorMap* map_high = &no_map;
  if (h.rows) {
    if (g->high_map.ptr != h.weight) {
      g->high_map.map = make_map(h.weight, h.rows, h.k, kTileRows);
      g->high_map.ptr = h.weight;
    }
    map_high = &g->high_map.map;
  }
  const dim3 grid(plan.grid), plain(kTcThreads - kQuantThreads), with_quantisers(kTcThreads);
  const bool bf16 = g->dtype == HG_DTYPE_BF16;
  cudaError_t launched;
  if (fused)
    launched = bf16 ? launch_kernel(hybrid_gemm_tc_kernel<__nv_bfloat16, true>, grid, with_quantisers, plan.smem_bytes, stream, p, *map_high, *map_act, g->heads)
                    : launch_kernel(hybrid_gemm_tc_kernel<__half, true>, grid, with_quantisers, plan.smem_bytes, stream, p, *map_high, *map_act, g->heads);
  else
    launched = bf16 ? launch_kernel(hybrid_gemm_tc_kernel<__nv_bfloat16, false>, grid, plain, plan.smem_bytes, stream, p, *map_high, *map_act, g->heads)
                    : launch_kernel(hybrid_gemm_tc_kernel<__half, false>, grid, plain, plan.smem_bytes, stream, p, *map_high, *map_act, g->heads);
  check(launched, "hybrid GEMM launch");
  launch_reduce(plan, p, g->d_cut, g->dtype, stream, true);
}

void tc_destroy(TcGemm* g) {
  if (!g) return;
  cudaFree(g->d_units); cudaFree(g->d_cta_begin); cudaFree(g->d_workspace); cudaFree(g->d_counters); cudaFree(g->d_status); cudaFree(g->d_cut);
#ifdef HG_TRACE
  cudaFree(g->d_trace);
#endif
  delete g;
}

const Plan& tc_plan(const TcGemm* g) { return g->plan; }

int tc_trace(TcGemm* g, cudaStream_t stream, unsigned long long* out, int max_values) {
#ifdef HG_TRACE
  const int values = std::min(max_values, 16 * g->plan.grid);
  check(cudaMemcpyAsync(out, g->d_trace, sizeof(unsigned long long) * size_t(values), cudaMemcpyDeviceToHost, stream), "trace read");
  check(cudaStreamSynchronize(stream), "trace read");
  return values;
#else
  (void)g; (void)stream; (void)out; (void)max_values;
  throw std::runtime_error("hg_trace needs a library built with -DHG_TRACE");
#endif
}

void tc_kernel_attributes(int* registers, int* local_bytes) {
  cudaFuncAttributes attr{};
  check(cudaFuncGetAttributes(&attr, hybrid_gemm_tc_kernel<__nv_bfloat16, false>), "cudaFuncGetAttributes");
  *registers = attr.numRegs;
  *local_bytes = int(attr.localSizeBytes);
}

void tc_status(TcGemm* g, cudaStream_t stream, int out[3]) {
  int host[4] = {0, 0, 0, 0};
  check(cudaMemcpyAsync(host, g->d_status, sizeof(host), cudaMemcpyDeviceToHost, stream), "status read");
  check(cudaMemsetAsync(g->d_status, 0, sizeof(host), stream), "status clear");
  check(cudaStreamSynchronize(stream), "status sync");
  out[0] = host[0]; out[1] = host[1]; out[2] = host[2];
}

// ---------------------------------------------------------------------------------------------
// hg_run_static: the hybrid GEMM for callers that must not allocate device memory
// ---------------------------------------------------------------------------------------------
//
// Some hosts of this library cannot call cudaMalloc on the path that runs a layer: a serving engine
// that has handed all device memory to its own pool, a latency-critical loop where an allocation
// (an implicit device-wide synchronisation) is not acceptable, or code that only ever sees shapes at
// the moment it must run them and so cannot warm a handle first.  For them the scratch memory the
// kernel needs — the tile schedule, the split-K partial sums, the arrival counters and the status
// words — lives in one fixed array inside the library image instead of in a handle.
//
// * The array is HG_STATIC_SCRATCH_BYTES long on every GPU that loads the library, until exit.
// * `g_static_scratch` is a device symbol.  Host code cannot use its name as a pointer; the device
//   address is looked up once per device with cudaGetSymbolAddress, with that device current.  That
//   look-up (and raising the kernel's shared-memory limit) happens in the first call on a device.
// * The call is NOT for stream capture: it copies the schedule of the shape from host memory into the
//   array whenever the array holds another shape's schedule, and a captured copy would replay from
//   host memory that a later call rewrites.  A capturing stream is refused with an error.
// * All calls share the array: two calls that overlap on the GPU (different streams) race on it.
//   Calls on one stream are ordered and safe.  Counters and status words are cleared at the start
//   of every call, whatever an earlier call left behind; hg_static_status reads the status words of
//   the calls since its last read.
// * A shape whose schedule and partial sums do not fit is rejected with an error; nothing is launched.

static __device__ __align__(256) unsigned char g_static_scratch[HG_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kStaticPlans = 8;   // schedules kept on the host, least recently used replaced

struct StaticPlan {
  int key[6] = {0, 0, 0, 0, 0, 0};
  uint64_t used = 0;             // 0 = empty
  Plan plan;
  CtaHeads heads{};
};

struct StaticState {
  std::mutex mutex;
  unsigned char* base[64] = {};   // device address of g_static_scratch, per device ordinal
  int sms[64] = {};
  const StaticPlan* resident[64] = {};   // whose schedule the array of that device holds
  uint64_t resident_stamp[64] = {};
  StaticPlan plans[kStaticPlans];
  uint64_t clock = 0;
};

StaticState& static_state() {
  static StaticState state;
  return state;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Where the three status words of the static path live: they are accumulated over calls (the kernel
// only ever adds to [1] and [2] and sets [0] once), so they sit apart from what each call clears.
constexpr size_t kStaticStatusOffset = 0, kStaticCountersOffset = 256;

unsigned char* static_base(StaticState& st, int device) {
  if (device < 0 || device >= 64) throw std::runtime_error("hg_run_static supports device ordinals 0..63");
  if (!st.base[device]) {
    // Once per device, with that device current: device address of the symbol, SM count, kernel limits.
    void* address = nullptr;
    check(cudaGetSymbolAddress(&address, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
    check(cudaDeviceGetAttribute(&st.sms[device], cudaDevAttrMultiProcessorCount, device), "SM count");
    configure_kernel<__nv_bfloat16>();
    configure_kernel<__half>();
    st.base[device] = static_cast<unsigned char*>(address);
  }
  return st.base[device];
}

}  // namespace

void tc_run_static(int schedule, const hg_problem& l, const hg_problem& h, int dtype, cudaStream_t stream) {
  validate(l, h);
  if (dtype != HG_DTYPE_F16 && dtype != HG_DTYPE_BF16) throw std::runtime_error("Unknown output dtype");
  if (schedule < HG_SCHEDULE_AUTO || schedule > HG_SCHEDULE_STREAM_K) throw std::runtime_error("Unknown tile schedule id");
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  check(cudaStreamIsCapturing(stream, &capturing), "cudaStreamIsCapturing");
  if (capturing != cudaStreamCaptureStatusNone)
    throw std::runtime_error("hg_run_static cannot be captured into a CUDA graph (it copies a schedule from host memory); "
                             "use hg_create/hg_run under capture");
  const hg_problem& any = l.rows ? l : h;
  StaticState& st = static_state();
  std::lock_guard<std::mutex> lock(st.mutex);
  int device = 0;
  check(cudaGetDevice(&device), "cudaGetDevice");
  unsigned char* base = static_base(st, device);
  const int key[6] = {l.rows, h.rows, any.tokens, any.k, schedule, st.sms[device]};
  StaticPlan* entry = nullptr;
  StaticPlan* oldest = &st.plans[0];
  for (StaticPlan& candidate : st.plans) {
    if (candidate.used && std::memcmp(key, candidate.key, sizeof(key)) == 0) entry = &candidate;
    if (candidate.used < oldest->used) oldest = &candidate;
  }
  if (!entry) {
    entry = oldest;
    for (auto& resident : st.resident)
      if (resident == entry) resident = nullptr;   // the array of that device holds a schedule that is going away
    entry->plan = make_plan(l.rows, h.rows, any.tokens, any.k, st.sms[device], schedule);
    entry->heads = make_heads(entry->plan);
    std::memcpy(entry->key, key, sizeof(key));
  }
  entry->used = ++st.clock;
  const Plan& plan = entry->plan;

  // Carve the array: status | counters | cta_begin | units | cut list | workspace.
  const size_t off_cta = align_up(kStaticCountersOffset + sizeof(int) * size_t(std::max(1, plan.counters)), 256);
  const size_t off_units = align_up(off_cta + sizeof(int) * plan.cta_begin.size(), 256);
  const size_t off_cut = align_up(off_units + sizeof(WorkUnit) * std::max<size_t>(1, plan.units.size()), 256);
  const size_t off_work = align_up(off_cut + sizeof(int) * std::max<size_t>(4, plan.cut_tiles.size()), 256);
  const size_t total = off_work + sizeof(float) * size_t(plan.ws_slots) * size_t(plan.n_tile) * kTileRows;
  if (total > size_t(HG_STATIC_SCRATCH_BYTES))
    throw std::runtime_error("hg_run_static: this shape needs " + std::to_string(total) +
                             " bytes of scratch (schedule and split-K partial sums) but the static buffer holds " +
                             std::to_string(size_t(HG_STATIC_SCRATCH_BYTES)) + "; use hg_create/hg_run");
  // Arrival counters start every call at zero; the status words are only cleared by hg_static_status.
  check(cudaMemsetAsync(base + kStaticCountersOffset, 0, off_cta - kStaticCountersOffset, stream), "clear static counters");
  if (st.resident[device] != entry) {
    // The schedule of another shape (or nothing) is in the array: copy this one in.  The vectors stay
    // alive in their cache entry; an entry is only rebuilt under the mutex, after which it is copied again.
    check(cudaMemcpyAsync(base + off_cta, plan.cta_begin.data(), sizeof(int) * plan.cta_begin.size(),
                          cudaMemcpyHostToDevice, stream), "upload schedule");
    check(cudaMemcpyAsync(base + off_units, plan.units.data(), sizeof(WorkUnit) * plan.units.size(),
                          cudaMemcpyHostToDevice, stream), "upload units");
    if (!plan.cut_tiles.empty())
      check(cudaMemcpyAsync(base + off_cut, plan.cut_tiles.data(), sizeof(int) * plan.cut_tiles.size(),
                            cudaMemcpyHostToDevice, stream), "upload cut list");
    st.resident[device] = entry;
  }

  TcParams p = base_params(plan, l, h, dtype);
  p.out.ptr = any.output;
  p.status = reinterpret_cast<int*>(base + kStaticStatusOffset);
  p.counters = reinterpret_cast<int*>(base + kStaticCountersOffset);
  p.cta_begin = reinterpret_cast<const int*>(base + off_cta);
  p.units = reinterpret_cast<const WorkUnit*>(base + off_units);
  p.workspace = reinterpret_cast<float*>(base + off_work);
  static const CUtensorMap no_map{};
  const CUtensorMap map_act = make_map(any.activation, any.tokens, any.k, plan.n_tile);
  const CUtensorMap map_high = h.rows ? make_map(h.weight, h.rows, h.k, kTileRows) : no_map;
  // Plain launches (no programmatic overlap): the clears and copies above are ordered before the kernel.
  if (dtype == HG_DTYPE_BF16)
    hybrid_gemm_tc_kernel<__nv_bfloat16, false><<<plan.grid, kTcThreads - kQuantThreads, plan.smem_bytes, stream>>>(p, map_high, map_act, entry->heads);
  else
    hybrid_gemm_tc_kernel<__half, false><<<plan.grid, kTcThreads - kQuantThreads, plan.smem_bytes, stream>>>(p, map_high, map_act, entry->heads);
  check(cudaGetLastError(), "hybrid GEMM launch (static scratch)");
  launch_reduce(plan, p, reinterpret_cast<const int*>(base + off_cut), dtype, stream, false);
}

void tc_static_status(cudaStream_t stream, int out[3]) {
  StaticState& st = static_state();
  std::lock_guard<std::mutex> lock(st.mutex);
  int device = 0;
  check(cudaGetDevice(&device), "cudaGetDevice");
  unsigned char* base = static_base(st, device);
  int host[3] = {0, 0, 0};
  check(cudaMemcpyAsync(host, base + kStaticStatusOffset, sizeof(host), cudaMemcpyDeviceToHost, stream), "status read");
  check(cudaMemsetAsync(base + kStaticStatusOffset, 0, sizeof(host), stream), "status clear");
  check(cudaStreamSynchronize(stream), "status sync");
  out[0] = host[0]; out[1] = host[1]; out[2] = host[2];
}

}  // namespace hg

extern "C" int hg_run_static(int schedule, const hg_problem* low, const hg_problem* high, void* stream, int dtype) {
  HG_TRY
  if (!low || !high) throw std::runtime_error("Null argument to hg_run_static");
  hg::tc_run_static(schedule, *low, *high, dtype, static_cast<cudaStream_t>(stream));
  HG_CATCH
}

extern "C" int hg_static_status(void* stream, int* status) {
  HG_TRY
  if (!status) throw std::runtime_error("Null argument to hg_static_status");
  hg::tc_static_status(static_cast<cudaStream_t>(stream), status);
  HG_CATCH
}
