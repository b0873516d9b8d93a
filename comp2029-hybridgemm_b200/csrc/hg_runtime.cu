// C ABI of the GEMM half of the library: handles, rebinding, launch policies.
// Mirrors integrations/vllm/native/runtime.cu:20-44,146-163 and
// integrations/vllm/native/fused_probe.cu:7-28 of the reference.
#include <algorithm>
#include <memory>

#include "hg_gemm_tc.cuh"

namespace hg {

static bool same_shape(const hg_problem& a, const hg_problem& b) {
  return a.rows == b.rows && a.tokens == b.tokens && a.k == b.k && a.outputs == b.outputs;
}

// Counterpart of the reference's Runner (runtime.cu:20-44).  The reference owns
// two kernels, a side stream and fork/join events; here one persistent launch
// covers both partitions, so the stream policies 0-3 all enqueue that launch.
constexpr int kReferenceVariants = 45, kLastSimtVariant = 34;

struct Runner {
  hg_problem low{}, high{};
  int low_id = 0, high_id = 0, dtype = HG_DTYPE_F16;
  TcGemm* tc = nullptr;

  Runner(int li, int hi, const hg_problem& l, const hg_problem& h, cudaStream_t s, int dt)
      : low(l), high(h), low_id(li), high_id(hi), dtype(dt) {
    if (li < 0 || hi < 0) throw std::runtime_error("Negative schedule id");
    if (l.rows == 0 && h.rows == 0) throw std::runtime_error("Hybrid GEMM needs at least one weight row");
    // The partitions share one launch: the low partition's id decides unless it is absent or AUTO.
    int schedule = l.rows && li ? li : (h.rows && hi ? hi : (li ? li : hi));
    // Ids above the three schedules of this library are the reference's variant ids (45 of them,
    // src/kernel/output_channel_gemm.h:41): 28-34, its SIMT family, select the SIMT kernel here; the rest name
    // CUTLASS and cp.async tile shapes that have no counterpart, so a plan tuned on the reference's GPU still
    // loads and runs with the schedule chosen from the shape.  The tensor-core handle always exists: it serves
    // policies 0-3 whatever the id.
    if (schedule >= kReferenceVariants) throw std::runtime_error("Unknown schedule id " + std::to_string(schedule));
    if (schedule > HG_SCHEDULE_STREAM_K) schedule = HG_SCHEDULE_AUTO;
    tc = tc_create(l, h, schedule, dt, s);
  }
  ~Runner() { tc_destroy(tc); }

  bool simt_only() const {
    const int id = low.rows ? low_id : high_id;
    return id >= HG_SCHEDULE_SIMT && id <= kLastSimtVariant;
  }

  void run(const hg_problem& l, const hg_problem& h, cudaStream_t s, int policy) {
    if (!same_shape(l, low) || !same_shape(h, high)) throw std::runtime_error("Kernel cannot rebind to a different shape");
    if (policy < 0 || policy > HG_POLICY_GEMV_PAIR4) throw std::runtime_error("Unknown launch policy");
    validate(l, h);   // every path, the SIMT kernel included: a bad pointer is an error, never a launch
    if (policy >= HG_POLICY_GEMV_PAIR1) run_simt_pair(l, h, s, 1 << (policy - HG_POLICY_GEMV_PAIR1), dtype);
    else if (simt_only()) run_simt_pair(l, h, s, 4, dtype);
    else tc_run(tc, l, h, s);
  }

  // Quantise-and-multiply in one launch (decode sizes): see hg_run_x.
  void run_x(const hg_problem& l, const hg_problem& h, const void* x, int x_dtype, cudaStream_t s) {
    if (!same_shape(l, low) || !same_shape(h, high)) throw std::runtime_error("Kernel cannot rebind to a different shape");
    if (!x) throw std::runtime_error("Null activations");
    tc_run(tc, l, h, s, x, x_dtype);
  }

  // Row-parallel tensor parallelism: the partial result goes to this rank's exchange buffer (see hg_run_partial).
  void run_partial(const hg_problem& l, const hg_problem& h, const void* x, int x_dtype, const PartialTarget& target, cudaStream_t s) {
    if (!same_shape(l, low) || !same_shape(h, high)) throw std::runtime_error("Kernel cannot rebind to a different shape");
    tc_run(tc, l, h, s, x, x_dtype, &target);
  }
};

static std::string& fused_error() {
  static thread_local std::string message;
  return message;
}

// Fixed-operand wrapper behind the hg_fused_* symbols.
struct FusedRunner {
  std::unique_ptr<Runner> runner;
  hg_problem low{}, high{};
};

}  // namespace hg

extern "C" {

int hg_create_dtype(int low_id, int high_id, const hg_problem* l, const hg_problem* h, void* stream, int dtype,
                    void** handle) {
  HG_TRY
  if (!l || !h || !handle) throw std::runtime_error("Null argument to hg_create");
  *handle = new hg::Runner(low_id, high_id, *l, *h, static_cast<cudaStream_t>(stream), dtype);
  HG_CATCH
}

int hg_create(int low_id, int high_id, const hg_problem* l, const hg_problem* h, void* stream, void** handle) {
  return hg_create_dtype(low_id, high_id, l, h, stream, HG_DTYPE_F16, handle);
}

int hg_run(void* handle, const hg_problem* l, const hg_problem* h, void* stream, int policy) {
  HG_TRY
  if (!handle || !l || !h) throw std::runtime_error("Null argument to hg_run");
  static_cast<hg::Runner*>(handle)->run(*l, *h, static_cast<cudaStream_t>(stream), policy);
  HG_CATCH
}

int hg_run_x(void* handle, const hg_problem* l, const hg_problem* h, const void* x, int x_dtype, void* stream) {
  HG_TRY
  if (!handle || !l || !h) throw std::runtime_error("Null argument to hg_run_x");
  static_cast<hg::Runner*>(handle)->run_x(*l, *h, x, x_dtype, static_cast<cudaStream_t>(stream));
  HG_CATCH
}

int hg_run_partial(void* handle, const hg_problem* l, const hg_problem* h, const void* x, int x_dtype,
                   void* buffer, int64_t half_bytes, int f32, const int* state, void* stream) {
  HG_TRY
  if (!handle || !l || !h) throw std::runtime_error("Null argument to hg_run_partial");
  const hg::PartialTarget target{buffer, half_bytes, f32, state};
  static_cast<hg::Runner*>(handle)->run_partial(*l, *h, x, x_dtype, target, static_cast<cudaStream_t>(stream));
  HG_CATCH
}

int hg_info(void* handle, int* out) {
  HG_TRY
  if (!handle || !out) throw std::runtime_error("Null argument to hg_info");
  auto* r = static_cast<hg::Runner*>(handle);
  std::fill(out, out + 20, -1);
  int regs = 0, local = 0;
  hg::tc_kernel_attributes(&regs, &local);
  const hg::Plan& plan = hg::tc_plan(r->tc);
  for (int part = 0; part < 2; ++part) {
    if (!(part ? r->high.rows : r->low.rows)) continue;
    const int values[10] = {plan.schedule, hg::kTileRows, plan.n_tile, 2 * hg::kTileK, plan.stages,
                            regs, plan.smem_bytes, local, part, 0};
    std::copy(values, values + 10, out + part * 10);
  }
  HG_CATCH
}

void hg_destroy(void* handle) { delete static_cast<hg::Runner*>(handle); }

int hg_status(void* handle, void* stream, int* status) {
  HG_TRY
  if (!handle || !status) throw std::runtime_error("Null argument to hg_status");
  hg::tc_status(static_cast<hg::Runner*>(handle)->tc, static_cast<cudaStream_t>(stream), status);
  HG_CATCH
}

int hg_trace(void* handle, void* stream, unsigned long long* out, int max_values, int* values) {
  HG_TRY
  if (!handle || !out || !values || max_values <= 0) throw std::runtime_error("Invalid hg_trace arguments");
  auto* runner = static_cast<hg::Runner*>(handle);
  if (!runner->tc) throw std::runtime_error("hg_trace: the handle has no tensor-core GEMM");
  *values = hg::tc_trace(runner->tc, static_cast<cudaStream_t>(stream), out, max_values);
  HG_CATCH
}

int hg_plan(int rows_low, int rows_high, int tokens, int k, int sms, int schedule, int* header, int* units,
            int max_units) {
  HG_TRY
  if (!header || rows_low < 0 || rows_high < 0 || rows_low + rows_high == 0 || tokens <= 0 || k <= 0 || k % 128 || sms <= 0)
    throw std::runtime_error("Invalid hg_plan arguments");
  const hg::Plan plan = hg::make_plan(rows_low, rows_high, tokens, k, sms, schedule);
  const int values[12] = {plan.schedule, plan.grid, plan.n_tile, plan.token_tiles, plan.stages, plan.smem_bytes,
                          plan.tmem_cols, plan.ws_slots, plan.counters, int(plan.units.size()),
                          plan.external_reduce ? 1 : 0, plan.issuers};
  std::copy(values, values + 12, header);
  if (units) {
    if (int(plan.units.size()) > max_units) throw std::runtime_error("hg_plan: unit buffer too small");
    for (int c = 0; c < plan.grid; ++c)
      for (int u = plan.cta_begin[c]; u < plan.cta_begin[c + 1]; ++u) {
        const hg::WorkUnit& w = plan.units[u];
        const int row[9] = {c, w.tile, w.token_tile, w.kb_begin, w.kb_end, w.split, w.nsplit, w.ws_slot, w.counter};
        std::copy(row, row + 9, units + 9 * u);
      }
  }
  HG_CATCH
}

const char* hg_fused_error(void) { return hg::fused_error().c_str(); }

#define HG_FUSED_TRY try {
#define HG_FUSED_CATCH                          \
  }                                             \
  catch (std::exception const& e) {             \
    hg::fused_error() = e.what();               \
    return -1;                                  \
  }                                             \
  return 0;

int hg_fused_create_dtype(int id, const hg_problem* l, const hg_problem* h, void* stream, int dtype, void** handle) {
  HG_FUSED_TRY
  if (!l || !h || !handle) throw std::runtime_error("Null argument to hg_fused_create");
  auto f = std::make_unique<hg::FusedRunner>();
  f->low = *l; f->high = *h;
  f->runner = std::make_unique<hg::Runner>(id, id, *l, *h, static_cast<cudaStream_t>(stream), dtype);
  *handle = f.release();
  HG_FUSED_CATCH
}
int hg_fused_create(int id, const hg_problem* l, const hg_problem* h, void* stream, void** handle) {
  return hg_fused_create_dtype(id, l, h, stream, HG_DTYPE_F16, handle);
}
int hg_fused_update(void* handle, const hg_problem* l, const hg_problem* h) {
  HG_FUSED_TRY
  auto* f = static_cast<hg::FusedRunner*>(handle);
  if (!f || !l || !h) throw std::runtime_error("Null argument to hg_fused_update");
  if (!hg::same_shape(*l, f->low) || !hg::same_shape(*h, f->high)) throw std::runtime_error("Fused rebind unsupported");
  f->low = *l; f->high = *h;
  HG_FUSED_CATCH
}
int hg_fused_run(void* handle, void* stream) {
  HG_FUSED_TRY
  auto* f = static_cast<hg::FusedRunner*>(handle);
  if (!f) throw std::runtime_error("Null argument to hg_fused_run");
  f->runner->run(f->low, f->high, static_cast<cudaStream_t>(stream), HG_POLICY_SERIAL);
  HG_FUSED_CATCH
}
// id, tile_m, tile_n, tile_k, stages, registers, shared bytes, local bytes, low and high
// TMA transaction bytes per K stage, virtual rows (fused_probe.cu:18-26).
int hg_fused_info(void* handle, int* data) {
  HG_FUSED_TRY
  auto* f = static_cast<hg::FusedRunner*>(handle);
  if (!f || !data) throw std::runtime_error("Null argument to hg_fused_info");
  int regs = 0, local = 0;
  hg::tc_kernel_attributes(&regs, &local);
  const hg::Plan& plan = hg::tc_plan(f->runner->tc);
  // Bytes per K256 stage: MXFP4 weights arrive by cp.async (16 KiB packed), MXFP8 by TMA (32 KiB).
  const int common = 2 * (plan.n_tile * 128 + 1024);
  const int tiles = (f->low.rows + 127) / 128 + (f->high.rows + 127) / 128;
  const int values[11] = {plan.schedule, hg::kTileRows, plan.n_tile, 2 * hg::kTileK, plan.stages, regs,
                          plan.smem_bytes, local, 16384 + common, 32768 + common, tiles * 128};
  std::copy(values, values + 11, data);
  HG_FUSED_CATCH
}
void hg_fused_destroy(void* handle) { delete static_cast<hg::FusedRunner*>(handle); }

}  // extern "C"
