// Second half of a row-parallel exchange: publish, wait (bounded) and sum the partial results that the
// GEMM epilogues of all ranks pushed into this rank's receive buffer over NVLink (see hg_run_push).
//
// The reference has no tensor parallelism (integrations/vllm/hygemm_vllm/quantization.py:81-83 refuses
// it); the sum it would need is the all-reduce vLLM's RowParallelLinear performs after the layer.
#include <algorithm>

#include "hg_common.cuh"

namespace hg {

struct TpReduceParams {
  const uint16_t* recv;        // own receive buffer: [2][world][slot_elems]
  uint16_t* out;
  int64_t vectors;             // 8-element vectors to reduce
  int64_t slot_elems;
  int world, rank;
  int* flags[HG_TP_MAX_WORLD]; // flag array of every rank as mapped here; [rank] is the own one
  int* state;                  // [0] finished exchanges, [1] block ticket, [2] status
};

constexpr unsigned long long kTpWaitNanoseconds = 1000000000ull;

__device__ __forceinline__ int load_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_nanoseconds() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <typename T>
__global__ void __launch_bounds__(256)
tp_reduce_kernel(const TpReduceParams p) {
  pdl_trigger();
  pdl_wait();  // the GEMM that pushed this rank's partials has finished and its stores are performed
  const int epoch = *reinterpret_cast<volatile int*>(p.state) + 1;

  // Publish: one thread per peer tells it that slot `rank` of its receive buffer is complete.
  if (blockIdx.x == 0 && int(threadIdx.x) < p.world) {
    __threadfence_system();
    store_release_sys(p.flags[threadIdx.x] + p.rank, epoch);
  }
  // Wait until every rank has published this exchange here.  Bounded: a peer that never arrives leaves
  // a status word behind and the kernel returns without summing.
  int ok = 1;
  if (int(threadIdx.x) < p.world) {
    const int* flag = p.flags[p.rank] + threadIdx.x;
    int polls = 0;
    unsigned long long start = 0;
    while (load_acquire_sys(flag) - epoch < 0) {
      if (++polls < 64) continue;
      if (!start) start = global_nanoseconds();
      if (global_nanoseconds() - start > kTpWaitNanoseconds) {
        ok = 0;
        atomicCAS(p.state + 2, 0, 1000 + int(threadIdx.x));
        break;
      }
      __nanosleep(200);
    }
  }
  ok = __syncthreads_and(ok);

  if (ok) {
    const uint4* base = reinterpret_cast<const uint4*>(p.recv + int64_t(epoch & 1) * p.world * p.slot_elems);
    const int64_t slot_vectors = p.slot_elems >> 3;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.vectors; i += int64_t(gridDim.x) * blockDim.x) {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int w = 0; w < p.world; ++w) {   // rank order: every rank computes the same bits
        const uint4 v = __ldcg(base + w * slot_vectors + i);
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sum[2 * j] += to_float<T>(uint16_t(words[j] & 0xffffu));
          sum[2 * j + 1] += to_float<T>(uint16_t(words[j] >> 16));
        }
      }
      uint4 r;
      r.x = uint32_t(from_float<T>(sum[0])) | uint32_t(from_float<T>(sum[1])) << 16;
      r.y = uint32_t(from_float<T>(sum[2])) | uint32_t(from_float<T>(sum[3])) << 16;
      r.z = uint32_t(from_float<T>(sum[4])) | uint32_t(from_float<T>(sum[5])) << 16;
      r.w = uint32_t(from_float<T>(sum[6])) | uint32_t(from_float<T>(sum[7])) << 16;
      reinterpret_cast<uint4*>(p.out)[i] = r;
    }
  }
  // The last block to finish advances the exchange count (every block has read it by then).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.state + 1, 1) == int(gridDim.x) - 1) {
      p.state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(p.state) = epoch;
    }
  }
}

}  // namespace hg

extern "C" {

int hg_tp_reduce(const void* recv_own, void* out, int64_t elems, int64_t slot_elems, int world, int rank,
                 int* const* flags, int* state, int dtype, void* stream) {
  HG_TRY
  using namespace hg;
  if (!recv_own || !out || !flags || !state) throw std::runtime_error("Null argument to hg_tp_reduce");
  if (world < 1 || world > HG_TP_MAX_WORLD || rank < 0 || rank >= world) throw std::runtime_error("Tensor-parallel world must be 1..8 with rank inside it");
  if (elems <= 0 || elems % 8 || slot_elems % 8 || elems > slot_elems) throw std::runtime_error("Element counts must be multiples of 8 with elems <= slot_elems");
  if ((reinterpret_cast<uintptr_t>(recv_own) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) throw std::runtime_error("Buffers must be 16-byte aligned");
  if (dtype != HG_DTYPE_F16 && dtype != HG_DTYPE_BF16) throw std::runtime_error("Unknown dtype");
  TpReduceParams p{};
  p.recv = static_cast<const uint16_t*>(recv_own);
  p.out = static_cast<uint16_t*>(out);
  p.vectors = elems / 8;
  p.slot_elems = slot_elems;
  p.world = world;
  p.rank = rank;
  for (int w = 0; w < world; ++w) {
    if (!flags[w]) throw std::runtime_error("Null flag array");
    p.flags[w] = flags[w];
  }
  p.state = state;
  int device = 0, sms = 0;
  check(cudaGetDevice(&device), "cudaGetDevice");
  check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "SM count");
  const int64_t blocks = (p.vectors + 255) / 256;
  const dim3 grid(unsigned(std::max<int64_t>(1, std::min<int64_t>(blocks, sms)))), block(256);
  auto s = static_cast<cudaStream_t>(stream);
  check(dtype == HG_DTYPE_BF16 ? launch_kernel(tp_reduce_kernel<__nv_bfloat16>, grid, block, 0, s, p)
                               : launch_kernel(tp_reduce_kernel<__half>, grid, block, 0, s, p), "tensor-parallel reduce launch");
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
