// Offline MXFP4 weight quantiser with an exponent search per K32 group (load-time work).
//
// Follows integrations/vllm/allocation/fp4_quant.py:28-58 of the reference (`quantize`): the
// round-to-nearest result of hg_pack is the baseline; for every non-zero offset, in the order given, the
// group's scale byte is moved by the offset (clamped to [0,254]), the 32 values are re-rounded to E2M1 at
// that scale (saturating at 6, i.e. clipped when the scale shrinks) and the candidate replaces the best
// so far if its importance-weighted squared error is strictly smaller.  The reference runs this as a
// chain of torch ops over whole tensors (several full-size fp32 temporaries per offset); here one pass
// reads each 16-bit weight once and writes 4.25 bits per weight.
//
// Layout as mx_quant_kernel: sixteen threads own one (row, K128 block), four threads one K32 group, eight
// consecutive values per thread.  The error sum has a fixed order (eight terms left to right per thread,
// then a two-step butterfly over the four threads) so that the CPU oracle reproduces every decision.
#include "hg_common.cuh"

namespace hg {

constexpr int kMaxClipOffsets = 8;
struct ClipOffsets {
  int count;
  int value[kMaxClipOffsets];
};

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // 0, .5, 1, 1.5, 2, 3, 4, 6 by the low three bits; bit 3 is the sign.
  const uint32_t m = code & 7u;
  const float mag = m < 2u ? 0.5f * float(m) : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (code & 8u) ? -mag : mag;
}

// Codes of eight values at scale 2^e and the thread's part of the weighted squared error.
__device__ __forceinline__ uint32_t clip_candidate(const float (&v)[8], const float (&weight)[8], int e, float& error) {
  const float inv = mx_inverse_scale(e);
  // 2^e as a factor: e in [-127,127]; 2^-127 is the subnormal 0x00400000.
  const float scale = e == -127 ? __uint_as_float(0x00400000u) : __uint_as_float(uint32_t(e + 127) << 23);
  float scaled[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) scaled[i] = v[i] * inv;
  const uint32_t codes = cvt_e2m1x8(scaled);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float diff = __fsub_rn(__fmul_rn(e2m1_value((codes >> (4 * i)) & 15u), scale), v[i]);
    sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(diff, diff), weight[i]));
  }
  error = sum;
  return codes;
}

template <typename T>
__global__ void __launch_bounds__(256)
mx_clip_search_kernel(const uint16_t* __restrict__ in, const float* __restrict__ importance, uint8_t* __restrict__ q4,
                      uint8_t* __restrict__ scales, int rows, int k, ClipOffsets offsets) {
  const int64_t thread = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = k >> 3;
  if (thread >= int64_t(rows) * per_row) return;   // whole groups leave together: k % 32 == 0 and 4 | blockDim
  const int row = int(thread / per_row), col = int(thread % per_row) << 3;
  const uint4 raw = *reinterpret_cast<const uint4*>(in + int64_t(row) * k + col);
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8], weight[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = to_float<T>(uint16_t(words[i] & 0xffffu));
    v[2 * i + 1] = to_float<T>(uint16_t(words[i] >> 16));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) weight[i] = importance ? importance[col + i] : 1.f;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const uint32_t mask = 0xfu << (threadIdx.x & 28);   // the four threads of this K32 group (groups never straddle the tail)
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
  const int base = mx_exponent<true>(amax);

  auto group_error = [&](float part) {
    part = __fadd_rn(part, __shfl_xor_sync(mask, part, 1));
    return __fadd_rn(part, __shfl_xor_sync(mask, part, 2));
  };
  float part;
  uint32_t best_codes = clip_candidate(v, weight, base, part);
  float best = group_error(part);
  int best_e = base;
  for (int o = 0; o < offsets.count; ++o) {
    if (offsets.value[o] == 0) continue;
    const int e = max(-127, min(127, base + offsets.value[o]));
    const uint32_t codes = clip_candidate(v, weight, e, part);
    const float error = group_error(part);
    if (error < best) { best = error; best_e = e; best_codes = codes; }
  }
  *reinterpret_cast<uint32_t*>(q4 + (int64_t(row) * k + col) / 2) = best_codes;
  if ((col & 31) == 0) scales[int64_t(row) * (k >> 5) + (col >> 5)] = uint8_t(best_e + 127);
}

}  // namespace hg

extern "C" int hg_clip_pack(const void* in, const float* importance, void* q4, void* scales, int rows, int k,
                            const int* offsets, int n_offsets, int dtype, void* stream) {
  HG_TRY
  using namespace hg;
  if (!in || !q4 || !scales || rows <= 0 || k <= 0 || k % 128) throw std::runtime_error("Invalid MX clip-pack arguments");
  if (n_offsets < 0 || n_offsets > kMaxClipOffsets || (n_offsets && !offsets)) throw std::runtime_error("At most 8 exponent offsets");
  if (dtype != HG_DTYPE_F16 && dtype != HG_DTYPE_BF16) throw std::runtime_error("Unknown input dtype");
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(q4) & 3)) throw std::runtime_error("Weights must be 16-byte aligned");
  ClipOffsets list{};
  list.count = n_offsets;
  for (int i = 0; i < n_offsets; ++i) {
    if (offsets[i] < -254 || offsets[i] > 254) throw std::runtime_error("Exponent offset out of range");
    list.value[i] = offsets[i];
  }
  const int64_t threads = int64_t(rows) * (k / 8);
  const dim3 grid(unsigned((threads + 255) / 256)), block(256);
  auto s = static_cast<cudaStream_t>(stream);
  const auto* src = static_cast<const uint16_t*>(in);
  auto* codes = static_cast<uint8_t*>(q4);
  auto* bytes = static_cast<uint8_t*>(scales);
  if (dtype == HG_DTYPE_BF16) mx_clip_search_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(src, importance, codes, bytes, rows, k, list);
  else mx_clip_search_kernel<__half><<<grid, block, 0, s>>>(src, importance, codes, bytes, rows, k, list);
  check(cudaGetLastError(), "clip-pack launch");
  HG_CATCH
}
