// Second half of a row-parallel exchange: every rank's GEMM has written its partial [tokens, outputs] into
// its OWN exchange buffer (hg_run_partial: plain local stores from the scatter epilogue); this kernel tells
// the peers so, waits (bounded) until every peer has said the same, pulls the partials of all ranks with
// 16-byte loads over NVLink and adds them in rank order, so that every rank ends with identical bits.
//
// The reference has no tensor parallelism (integrations/vllm/hygemm_vllm/quantization.py:81-83 refuses
// it); the sum it would need is the all-reduce vLLM's RowParallelLinear performs after the layer.
#include <algorithm>
#include <cstdlib>

#include "hg_common.cuh"

namespace hg {

struct TpReduceParams {
  const unsigned char* buffers[HG_TP_MAX_WORLD];  // exchange buffer of every rank as mapped here ([rank] = own)
  int* flags[HG_TP_MAX_WORLD];                    // flag array of every rank as mapped here
  uint16_t* out;
  int64_t vectors;             // 8-element vectors to reduce
  int64_t half_bytes;          // distance between the two halves of an exchange buffer
  int world, rank, f32;
  int* state;                  // [0] finished exchanges, [1] block ticket, [2] status
  unsigned long long wait_ns;
};

__device__ __forceinline__ int load_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// 16 bytes of a peer's (or the own) buffer; never through L1, where a line of an earlier exchange could linger.
__device__ __forceinline__ uint4 load_peer(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_nanoseconds() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <typename T>
__global__ void __launch_bounds__(256)
tp_allreduce_kernel(const TpReduceParams p) {
  pdl_trigger();
  pdl_wait();  // the GEMM that wrote this rank's partial has finished and its stores are performed
  const int epoch = *reinterpret_cast<volatile int*>(p.state) + 1;

  // Publish: one thread per peer tells it that this rank's partial of exchange `epoch` is complete.
  if (blockIdx.x == 0 && int(threadIdx.x) < p.world) {
    __threadfence_system();
    store_release_sys(p.flags[threadIdx.x] + p.rank, epoch);
  }
  // Wait until every rank has published this exchange here.  Bounded: a peer that never arrives leaves
  // a status word behind and the output is filled with NaN instead of a sum.
  int ok = 1;
  if (int(threadIdx.x) < p.world) {
    const int* flag = p.flags[p.rank] + threadIdx.x;
    int polls = 0;
    unsigned long long start = 0;
    while (load_acquire_sys(flag) - epoch < 0) {
      if (++polls < 64) continue;
      if (!start) start = global_nanoseconds();
      if (global_nanoseconds() - start > p.wait_ns) {
        ok = 0;
        atomicCAS(p.state + 2, 0, 1000 + int(threadIdx.x));
        break;
      }
      __nanosleep(200);
    }
  }
  ok = __syncthreads_and(ok);

  const int64_t half = int64_t(epoch & 1) * p.half_bytes;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.vectors; i += int64_t(gridDim.x) * blockDim.x) {
    uint4 r;
    if (!ok) {
      r.x = r.y = r.z = r.w = 0x7fff7fffu;   // NaN in bf16 and in fp16: a missing peer never looks like a result
    } else {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (p.f32) {
        // All loads of all ranks first (independent NVLink round trips), then the additions in rank order.
        uint4 a[HG_TP_MAX_WORLD], b[HG_TP_MAX_WORLD];
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < p.world) {
            const unsigned char* src = p.buffers[w] + half + i * 32;
            a[w] = load_peer(src);
            b[w] = load_peer(src + 16);
          }
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < p.world) {
            sum[0] += __uint_as_float(a[w].x); sum[1] += __uint_as_float(a[w].y);
            sum[2] += __uint_as_float(a[w].z); sum[3] += __uint_as_float(a[w].w);
            sum[4] += __uint_as_float(b[w].x); sum[5] += __uint_as_float(b[w].y);
            sum[6] += __uint_as_float(b[w].z); sum[7] += __uint_as_float(b[w].w);
          }
      } else {
        uint4 a[HG_TP_MAX_WORLD];
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < p.world) a[w] = load_peer(p.buffers[w] + half + i * 16);
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < p.world) {
            const uint32_t words[4] = {a[w].x, a[w].y, a[w].z, a[w].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              sum[2 * j] += to_float<T>(uint16_t(words[j] & 0xffffu));
              sum[2 * j + 1] += to_float<T>(uint16_t(words[j] >> 16));
            }
          }
      }
      r.x = uint32_t(from_float<T>(sum[0])) | uint32_t(from_float<T>(sum[1])) << 16;
      r.y = uint32_t(from_float<T>(sum[2])) | uint32_t(from_float<T>(sum[3])) << 16;
      r.z = uint32_t(from_float<T>(sum[4])) | uint32_t(from_float<T>(sum[5])) << 16;
      r.w = uint32_t(from_float<T>(sum[6])) | uint32_t(from_float<T>(sum[7])) << 16;
    }
    reinterpret_cast<uint4*>(p.out)[i] = r;
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

// How long a rank waits for its peers, read once: HYGEMM_TP_WAIT_MS (default one second).
static unsigned long long wait_limit_ns() {
  static const unsigned long long value = [] {
    const char* text = std::getenv("HYGEMM_TP_WAIT_MS");
    const long ms = text && *text ? std::atol(text) : 1000;
    return (unsigned long long)(std::max<long>(1, std::min<long>(ms, 60000))) * 1000000ull;
  }();
  return value;
}

}  // namespace hg

extern "C" {

int hg_tp_allreduce(void* const* buffers, void* out, int64_t elems, int64_t half_bytes, int f32, int world, int rank,
                    int* const* flags, int* state, int dtype, void* stream) {
  HG_TRY
  using namespace hg;
  if (!buffers || !out || !flags || !state) throw std::runtime_error("Null argument to hg_tp_allreduce");
  if (world < 1 || world > HG_TP_MAX_WORLD || rank < 0 || rank >= world) throw std::runtime_error("Tensor-parallel world must be 1..8 with rank inside it");
  if (elems <= 0 || elems % 8 || half_bytes % 16 || elems * (f32 ? 4 : 2) > half_bytes)
    throw std::runtime_error("Element count must be a multiple of 8 and fit half an exchange buffer");
  if (reinterpret_cast<uintptr_t>(out) & 15) throw std::runtime_error("Buffers must be 16-byte aligned");
  if (dtype != HG_DTYPE_F16 && dtype != HG_DTYPE_BF16) throw std::runtime_error("Unknown dtype");
  TpReduceParams p{};
  for (int w = 0; w < world; ++w) {
    if (!buffers[w] || (reinterpret_cast<uintptr_t>(buffers[w]) & 15)) throw std::runtime_error("Exchange buffers must be 16-byte aligned");
    if (!flags[w]) throw std::runtime_error("Null flag array");
    p.buffers[w] = static_cast<const unsigned char*>(buffers[w]);
    p.flags[w] = flags[w];
  }
  p.out = static_cast<uint16_t*>(out);
  p.vectors = elems / 8;
  p.half_bytes = half_bytes;
  p.world = world;
  p.rank = rank;
  p.f32 = f32 ? 1 : 0;
  p.state = state;
  p.wait_ns = wait_limit_ns();
  int device = 0, sms = 0;
  check(cudaGetDevice(&device), "cudaGetDevice");
  check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "SM count");
  const int64_t blocks = (p.vectors + 255) / 256;
  const dim3 grid(unsigned(std::max<int64_t>(1, std::min<int64_t>(blocks, 2 * sms)))), block(256);
  auto s = static_cast<cudaStream_t>(stream);
  check(dtype == HG_DTYPE_BF16 ? launch_kernel(tp_allreduce_kernel<__nv_bfloat16>, grid, block, 0, s, p)
                               : launch_kernel(tp_allreduce_kernel<__half>, grid, block, 0, s, p), "tensor-parallel all-reduce launch");
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
