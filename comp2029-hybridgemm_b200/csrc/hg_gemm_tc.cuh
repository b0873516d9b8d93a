// Host-side interface of the tcgen05 hybrid GEMM (see hg_gemm_tc.cu).
#pragma once
#include <vector>

#include "hg_common.cuh"

namespace hg {

constexpr int kTileRows = 128;  // weight rows per output tile (MMA M)
constexpr int kTileK = 128;     // K elements per pipeline stage
constexpr int kMaxStages = 12;
constexpr int kTcThreads = 544; // warp 0 TMA, 1 and 10-12 MMA issuers, 2-5 epilogue, 6-9 MXFP4 loaders, 13-16 activation quantisers

// One contiguous run of K128 blocks of one (row tile, token tile).
struct WorkUnit {
  int tile;        // virtual row tile: [0,tiles_low) low partition, then the high partition
  int token_tile;  // index of the token tile (n_tile tokens each)
  int kb_begin, kb_end;
  int split;       // position of this unit among the tile's units, in K order
  int nsplit;      // units the tile is cut into (1 = direct scatter, no workspace)
  int ws_slot;     // first workspace slot of the tile (valid when nsplit > 1)
  int counter;     // arrival counter of the tile (valid when nsplit > 1)
};

struct Plan {
  int n_tile = 0;          // tokens per tile = MMA N
  int token_tiles = 0;
  int stages = 0;
  int grid = 0;
  int schedule = 0;        // HG_SCHEDULE_* actually used
  int smem_bytes = 0;
  int tmem_cols = 0;
  int issuers = 1;         // MMA-issuing threads, each with its own TMEM accumulator
  int acc_slots = 2;       // accumulator buffers per issuer
  int split_blocks = 0;    // both issuers read every stage, one K128 block each (token tiles wider than 64)
  int ws_slots = 0;        // fp32 [n_tile][128] slots
  int counters = 0;
  bool external_reduce = false;  // cut tiles are summed by splitk_reduce_kernel instead of the last arriver
  std::vector<int> cut_tiles;    // 4 ints per cut (tile, token tile): tile, token_tile, ws_slot, nsplit
  std::vector<WorkUnit> units;
  std::vector<int> cta_begin;  // grid + 1 offsets into units
};

// Builds the tile schedule for one shape.  `sms` is the SM count of the device,
// `schedule` one of HG_SCHEDULE_{AUTO,DATA_PARALLEL,SPLIT_K,STREAM_K}.
Plan make_plan(int rows_low, int rows_high, int tokens, int k, int sms, int schedule);

struct TcGemm;  // opaque device-side state (plan buffers, workspace, counters, status)
TcGemm* tc_create(const hg_problem& l, const hg_problem& h, int schedule, int dtype, cudaStream_t stream);
// `x` (optional): 16-bit activations [tokens,k] to quantise inside the GEMM kernel (at most 16 tokens);
// the problems' activation / activation_scales pointers are then ignored.
// `partial` (optional): row-parallel tensor parallelism; the result goes to this rank's half of a peer-mapped
// exchange buffer (see hg_run_partial) instead of the problems' `output`.
struct PartialTarget {
  void* buffer;        // this rank's exchange buffer: two halves of half_bytes
  int64_t half_bytes;
  int f32;             // store fp32 partial sums instead of 16-bit ones
  const int* state;    // device word counting finished exchanges
};
void tc_run(TcGemm*, const hg_problem& l, const hg_problem& h, cudaStream_t stream, const void* x = nullptr,
            int x_dtype = HG_DTYPE_BF16, const PartialTarget* partial = nullptr);
void tc_destroy(TcGemm*);
const Plan& tc_plan(const TcGemm*);
// Per-CTA time stamps of the handle's last launch (16 per CTA, nanoseconds of the global timer; 0 = not reached).
// Only in builds with -DHG_TRACE; other builds throw.
int tc_trace(TcGemm*, cudaStream_t stream, unsigned long long* out, int max_values);
void tc_kernel_attributes(int* registers, int* local_bytes);
// Reads (and clears) the device status words: [0] error code of a bounded wait
// that gave up, [1] K128 blocks issued to the tensor core, [2] work units stored.
void tc_status(TcGemm*, cudaStream_t stream, int out[3]);
// Same three words for the launches of hg_run_static on the current device since the last read.
void tc_static_status(cudaStream_t stream, int out[3]);
// Argument rule shared by every GEMM path (tensor-core and SIMT): shapes, shared operands, null and
// misaligned pointers throw.  `fused`: activations are quantised in the kernel, the problems' activation
// pointers are ignored.
void validate(const hg_problem& l, const hg_problem& h, bool fused = false);

void run_simt_pair(const hg_problem& l, const hg_problem& h, cudaStream_t stream, int tokens_per_pass, int dtype);

}  // namespace hg
