// Shared host/device helpers of the hybrid MX linear library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>

#include "../../include/hygemm.h"

namespace hg {

// Thread-local message behind hg_last_error(); the error convention follows
// integrations/vllm/native/runtime.cu:15-18 of the reference.
std::string& last_error();

inline void check(cudaError_t e, const char* what = "CUDA") {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

#define HG_TRY try {
#define HG_CATCH                                   \
  }                                                \
  catch (std::exception const& e) {                \
    hg::last_error() = e.what();                   \
    return -1;                                     \
  }                                                \
  return 0;

// Bytes of the padded E8M0 buffer: 512-byte atoms of 128 rows x 4 K32 groups.
__host__ __device__ inline int64_t scale_size(int rows, int k) {
  return rows <= 0 || k <= 0 ? 0 : int64_t((rows + 127) / 128) * (k / 128) * 512;
}

// Byte offset of the 32-bit word holding the four K32 scales of (row, K128 block kb).
__host__ __device__ inline int64_t scale_word_offset(int row, int kb, int k) {
  return (int64_t(row / 128) * (k / 128) + kb) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4;
}

#ifdef __CUDACC__
// Programmatic dependent launch.  Every kernel of the library is launched with the
// programmatic-stream-serialization attribute (unless HYGEMM_PDL=0): it may start while its
// predecessor in the stream drains, does its set-up and any work that does not depend on the
// predecessor, and calls pdl_wait() before it reads the predecessor's output or writes global memory.
// pdl_trigger() lets the next kernel in the stream do the same.  Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool pdl_enabled();

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, KernelArgs(std::forward<Args>(args))...);
}

// Smallest e with amax * 2^-e <= MAX (448 for E4M3, 6 for E2M1), clamped to
// [-127,127]; e = 0 for an all-zero block.  Equals ceil(log2(amax/MAX)) of
// integrations/vllm/native/runtime.cu:71-72 for every 16-bit input (proved
// exhaustively by the CPU tests) without a transcendental.
template <bool FP4>
__device__ __forceinline__ int mx_exponent(float amax) {
  uint32_t b = __float_as_uint(amax);
  if (b == 0) return 0;
  int ef = int(b >> 23);
  if (ef == 0) return -127;
  uint32_t man = b & 0x7fffffu;
  int x = ef - 127;
  int e = FP4 ? (man <= 0x400000u ? x - 2 : x - 1) : (man <= 0x600000u ? x - 8 : x - 7);
  return max(-127, min(127, e));
}

// 2^-e as an fp32 factor (e in [-127,127]; 2^-127 is a subnormal constant).
__device__ __forceinline__ float mx_inverse_scale(int e) {
  return e == 127 ? __uint_as_float(0x00400000u) : __uint_as_float(uint32_t(127 - e) << 23);
}

// Two floats -> two E4M3 bytes (lo in bits 0-7), round-to-nearest-even, saturating.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// Eight floats -> eight E2M1 nibbles (element 0 in the lowest nibble).
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&v)[8]) {
  uint32_t r;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return r;
}

template <typename T> __device__ __forceinline__ float to_float(uint16_t bits);
template <> __device__ __forceinline__ float to_float<__half>(uint16_t bits) {
  return __half2float(__ushort_as_half(bits));
}
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(uint16_t bits) {
  return __uint_as_float(uint32_t(bits) << 16);
}
template <typename T> __device__ __forceinline__ uint16_t from_float(float v);
template <> __device__ __forceinline__ uint16_t from_float<__half>(float v) {
  return __half_as_ushort(__float2half_rn(v));
}
template <> __device__ __forceinline__ uint16_t from_float<__nv_bfloat16>(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
#endif  // __CUDACC__

}  // namespace hg
