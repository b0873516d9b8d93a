// Second half of a row-parallel exchange: every rank's GEMM has written its partial [tokens, outputs] into
// its OWN exchange buffer (hg_run_partial: plain local stores from the scatter epilogue); this kernel tells
// the peers so, waits (bounded) until every peer has said the same, pulls the partials of all ranks with
// 16-byte loads over NVLink and adds them in rank order, so that every rank ends with identical bits.
//
// The reference has no tensor parallelism (integrations/vllm/hygemm_vllm/quantization.py:81-83 refuses
// it); the sum it would need is the all-reduce vLLM's RowParallelLinear performs after the layer.
#include <algorithm>
#include <cstdlib>

#include "hg_tp.cuh"

namespace hg {

template <typename T>
__global__ void __launch_bounds__(256)
tp_allreduce_kernel(const TpExchange x) {
  pdl_trigger();
  pdl_wait();  // the GEMM that wrote this rank's partial has finished and its stores are performed
  const int epoch = *reinterpret_cast<volatile int*>(x.state) + 1;
  if (blockIdx.x == 0) tp_publish(x, epoch, int(threadIdx.x));
  // Every block waits by itself until every rank has published this exchange here.
  const int ok = __syncthreads_and(tp_wait(x, epoch, int(threadIdx.x)));
  tp_sum<T>(x, epoch, ok, int64_t(blockIdx.x) * blockDim.x + threadIdx.x, int64_t(gridDim.x) * blockDim.x);
  // The last block to finish advances the exchange count (every block has read it by then).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(x.state + 1, 1) == int(gridDim.x) - 1) {
      x.state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(x.state) = epoch;
    }
  }
}

unsigned long long tp_wait_limit_ns() {
  static const unsigned long long value = [] {
    const char* text = std::getenv("HYGEMM_TP_WAIT_MS");
    const long ms = text && *text ? std::atol(text) : 1000;
    return (unsigned long long)(std::max<long>(1, std::min<long>(ms, 60000))) * 1000000ull;
  }();
  return value;
}

TpExchange make_exchange(void* const* buffers, void* out, int64_t elems, int64_t half_bytes, int f32, int world, int rank,
                         int* const* flags, int* state) {
  if (!buffers || !out || !flags || !state) throw std::runtime_error("Null argument to the tensor-parallel exchange");
  if (world < 1 || world > HG_TP_MAX_WORLD || rank < 0 || rank >= world) throw std::runtime_error("Tensor-parallel world must be 1..8 with rank inside it");
  if (elems <= 0 || elems % 8 || half_bytes % 16 || elems * (f32 ? 4 : 2) > half_bytes)
    throw std::runtime_error("Element count must be a multiple of 8 and fit half an exchange buffer");
  if (reinterpret_cast<uintptr_t>(out) & 15) throw std::runtime_error("Buffers must be 16-byte aligned");
  TpExchange x{};
  for (int w = 0; w < world; ++w) {
    if (!buffers[w] || (reinterpret_cast<uintptr_t>(buffers[w]) & 15)) throw std::runtime_error("Exchange buffers must be 16-byte aligned");
    if (!flags[w]) throw std::runtime_error("Null flag array");
    x.buffers[w] = static_cast<const unsigned char*>(buffers[w]);
    x.flags[w] = flags[w];
  }
  x.out = static_cast<uint16_t*>(out);
  x.vectors = elems / 8;
  x.half_bytes = half_bytes;
  x.world = world;
  x.rank = rank;
  x.f32 = f32 ? 1 : 0;
  x.state = state;
  x.wait_ns = tp_wait_limit_ns();
  return x;
}

}  // namespace hg

extern "C" {

int hg_tp_allreduce(void* const* buffers, void* out, int64_t elems, int64_t half_bytes, int f32, int world, int rank,
                    int* const* flags, int* state, int dtype, void* stream) {
  HG_TRY
  using namespace hg;
  if (dtype != HG_DTYPE_F16 && dtype != HG_DTYPE_BF16) throw std::runtime_error("Unknown dtype");
  const TpExchange x = make_exchange(buffers, out, elems, half_bytes, f32, world, rank, flags, state);
  int device = 0, sms = 0;
  check(cudaGetDevice(&device), "cudaGetDevice");
  check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "SM count");
  const int64_t blocks = (x.vectors + 255) / 256;
  const dim3 grid(unsigned(std::max<int64_t>(1, std::min<int64_t>(blocks, 2 * sms)))), block(256);
  auto s = static_cast<cudaStream_t>(stream);
  check(dtype == HG_DTYPE_BF16 ? launch_kernel(tp_allreduce_kernel<__nv_bfloat16>, grid, block, 0, s, x)
                               : launch_kernel(tp_allreduce_kernel<__half>, grid, block, 0, s, x), "tensor-parallel all-reduce launch");
  HG_CATCH
}

int hg_tp_status(int* state, void* stream, int* status) {
  HG_TRY
  if (!state || !status) throw std::runtime_error("Null argument to hg_tp_status");
  auto s = static_cast<cudaStream_t>(stream);
  hg::check(cudaMemcpyAsync(status, state + 2, sizeof(int), cudaMemcpyDeviceToHost, s), "status read");
  hg::check(cudaMemsetAsync(state + 2, 0, sizeof(int), s), "status clear");
  hg::check(cudaStreamSynchronize(s), "status sync");
  HG_CATCH
}

}  // extern "C"
