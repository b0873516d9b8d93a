// Device side of the row-parallel exchange, shared by the stand-alone all-reduce kernel (hg_tp.cu) and by the
// tail of the GEMM kernel that does the exchange itself (hg_gemm_tc.cu).
#pragma once
#include "hg_common.cuh"

namespace hg {

// What a rank needs to take part in one exchange.
struct TpExchange {
  const unsigned char* buffers[HG_TP_MAX_WORLD];  // exchange buffer of every rank as mapped here ([rank] = own)
  int* flags[HG_TP_MAX_WORLD];                    // flag array of every rank as mapped here
  uint16_t* out;               // summed [tokens, outputs], 16-bit
  int64_t vectors;             // 8-element vectors to reduce
  int64_t half_bytes;          // distance between the two halves of an exchange buffer
  int world, rank, f32;        // world == 0: no exchange
  int* state;                  // [0] finished exchanges, [1] block ticket, [2] status, [3] second block ticket
  unsigned long long wait_ns;  // how long to wait for the peers
};

#ifdef __CUDACC__
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

// One thread per peer tells it that this rank's partial of exchange `epoch` is complete.
__device__ __forceinline__ void tp_publish(const TpExchange& x, int epoch, int lane) {
  if (lane < x.world) {
    __threadfence_system();
    store_release_sys(x.flags[lane] + x.rank, epoch);
  }
}

// Thread `lane` (< world) waits until rank `lane` has published exchange `epoch` here.  Bounded: on expiry a
// status word is left behind and 0 returned.  Threads with lane >= world return 1 at once.
__device__ __forceinline__ int tp_wait(const TpExchange& x, int epoch, int lane) {
  if (lane >= x.world) return 1;
  const int* flag = x.flags[x.rank] + lane;
  int polls = 0;
  unsigned long long start = 0;
  while (load_acquire_sys(flag) - epoch < 0) {
    if (++polls < 64) continue;
    if (!start) start = global_nanoseconds();
    if (global_nanoseconds() - start > x.wait_ns) {
      atomicCAS(x.state + 2, 0, 1000 + lane);
      return 0;
    }
    __nanosleep(200);
  }
  return 1;
}

// Vectors first, first + stride, ... of the result: the partials of all ranks are loaded (all loads of a vector in
// flight together: independent NVLink round trips) and added in rank order, so every rank computes identical
// bits; `ok` == 0 (a peer never arrived) fills the vectors with NaN instead, so a failure never passes for a result.
template <typename T>
__device__ __forceinline__ void tp_sum(const TpExchange& x, int epoch, int ok, int64_t first, int64_t stride) {
  const int64_t half = int64_t(epoch & 1) * x.half_bytes;
  for (int64_t i = first; i < x.vectors; i += stride) {
    uint4 r;
    if (!ok) {
      r.x = r.y = r.z = r.w = 0x7fff7fffu;   // NaN in bf16 and in fp16
    } else {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (x.f32) {
        uint4 a[HG_TP_MAX_WORLD], b[HG_TP_MAX_WORLD];
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < x.world) {
            const unsigned char* src = x.buffers[w] + half + i * 32;
            a[w] = load_peer(src);
            b[w] = load_peer(src + 16);
          }
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < x.world) {
            sum[0] += __uint_as_float(a[w].x); sum[1] += __uint_as_float(a[w].y);
            sum[2] += __uint_as_float(a[w].z); sum[3] += __uint_as_float(a[w].w);
            sum[4] += __uint_as_float(b[w].x); sum[5] += __uint_as_float(b[w].y);
            sum[6] += __uint_as_float(b[w].z); sum[7] += __uint_as_float(b[w].w);
          }
      } else {
        uint4 a[HG_TP_MAX_WORLD];
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < x.world) a[w] = load_peer(x.buffers[w] + half + i * 16);
#pragma unroll
        for (int w = 0; w < HG_TP_MAX_WORLD; ++w)
          if (w < x.world) {
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
    reinterpret_cast<uint4*>(x.out)[i] = r;
  }
}
#endif  // __CUDACC__

// How long a rank waits for its peers, read once: HYGEMM_TP_WAIT_MS (default one second).
unsigned long long tp_wait_limit_ns();
// Fills and checks a TpExchange from the arguments of the C entry points (throws on a bad argument).
TpExchange make_exchange(void* const* buffers, void* out, int64_t elems, int64_t half_bytes, int f32, int world, int rank,
                         int* const* flags, int* state);

}  // namespace hg
