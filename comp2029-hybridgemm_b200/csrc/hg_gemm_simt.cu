// SIMT pair kernel: both precision partitions in one launch, one warp per weight row.
//
// Covers the reference's GEMV family and its `pair_kernel`
// (src/kernel/output_channel_gemv.cu:32-86, launch policies gemv_pair1/2/4):
// codes are expanded with cvt (e2m1x2 / e4m3x2 -> f16x2), every K32 group is
// accumulated in fp32 and scaled by 2^(sw+sx-254) exactly as
// output_channel_gemv.cu:53, then a fixed-order warp reduction.  It is the
// independent second implementation the tcgen05 kernel is checked against on
// the device and the path behind schedule id 28 / policies 4-6; the tensor-core
// kernel is the one the performance claims are about.
#include "hg_common.cuh"

namespace hg {

__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t pair) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(pair));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

// Four packed E2M1 bytes (8 codes) -> 8 floats, element 0 from the lowest nibble.
__device__ __forceinline__ void e2m1x8_to_float(uint32_t packed, float (&out)[8]) {
  uint32_t h[4];
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(packed));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&h[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// 2^(b-127) for an E8M0 byte (b = 0 is the fp32 subnormal 2^-127).
__device__ __forceinline__ float e8m0_to_float(uint32_t b) {
  return b ? __uint_as_float(b << 23) : __uint_as_float(0x00400000u);
}

__device__ __forceinline__ int64_t scale_offset(int row, int g, int k) {
  return scale_word_offset(row, g >> 2, k) + (g & 3);
}

struct SimtParams {
  const uint8_t* weight[2];
  const uint8_t* weight_scales[2];
  const int32_t* ids[2];
  int rows[2];
  const uint8_t* activation;
  const uint8_t* activation_scales;
  uint16_t* output;
  int tokens, k, outputs;
};

template <typename T, int NT>
__global__ void __launch_bounds__(128)
simt_pair_kernel(SimtParams p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int vrow = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (vrow >= p.rows[0] + p.rows[1]) return;
  const int part = vrow >= p.rows[0];
  const int row = part ? vrow - p.rows[0] : vrow;
  const int groups = p.k >> 5;
  const uint8_t* w = p.weight[part];
  const uint8_t* ws = p.weight_scales[part];
  const int channel = p.ids[part][row];

  for (int t0 = 0; t0 < p.tokens; t0 += NT) {
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.f;
    for (int g = lane; g < groups; g += 32) {
      float wv[32];
      if (part) {
        const uint4* src = reinterpret_cast<const uint4*>(w + int64_t(row) * p.k + g * 32);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 raw = src[h];
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float2 f = e4m3x2_to_float2(uint16_t(words[i >> 1] >> ((i & 1) * 16)));
            wv[h * 16 + 2 * i] = f.x;
            wv[h * 16 + 2 * i + 1] = f.y;
          }
        }
      } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(w + (int64_t(row) * p.k + g * 32) / 2);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float f[8];
          e2m1x8_to_float(words[i], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[i * 8 + j] = f[j];
        }
      }
      const float sw = e8m0_to_float(ws[scale_offset(row, g, p.k)]);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int token = t0 + t;
        if (token >= p.tokens) break;
        const uint4* xs = reinterpret_cast<const uint4*>(p.activation + int64_t(token) * p.k + g * 32);
        float dot = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 raw = xs[h];
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float2 f = e4m3x2_to_float2(uint16_t(words[i >> 1] >> ((i & 1) * 16)));
            dot = fmaf(wv[h * 16 + 2 * i], f.x, dot);
            dot = fmaf(wv[h * 16 + 2 * i + 1], f.y, dot);
          }
        }
        const float sx = e8m0_to_float(p.activation_scales[scale_offset(token, g, p.k)]);
        acc[t] += dot * sw * sx;
      }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      float v = acc[t];
#pragma unroll
      for (int d = 16; d; d >>= 1) v += __shfl_down_sync(0xffffffffu, v, d);
      if (lane == 0 && t0 + t < p.tokens) p.output[int64_t(t0 + t) * p.outputs + channel] = from_float<T>(v);
    }
  }
}

void run_simt_pair(const hg_problem& l, const hg_problem& h, cudaStream_t stream, int tokens_per_pass, int dtype) {
  SimtParams p{};
  const hg_problem* parts[2] = {&l, &h};
  const hg_problem& any = l.rows ? l : h;
  for (int i = 0; i < 2; ++i) {
    p.weight[i] = static_cast<const uint8_t*>(parts[i]->weight);
    p.weight_scales[i] = static_cast<const uint8_t*>(parts[i]->weight_scales);
    p.ids[i] = static_cast<const int32_t*>(parts[i]->ids);
    p.rows[i] = parts[i]->rows;
  }
  p.activation = static_cast<const uint8_t*>(any.activation);
  p.activation_scales = static_cast<const uint8_t*>(any.activation_scales);
  p.output = static_cast<uint16_t*>(any.output);
  p.tokens = any.tokens; p.k = any.k; p.outputs = any.outputs;
  const int total = p.rows[0] + p.rows[1];
  if (!total) return;
  const dim3 grid((total + 3) / 4), block(128);
#define HG_SIMT(T)                                                             \
  switch (tokens_per_pass) {                                                   \
    case 1: simt_pair_kernel<T, 1><<<grid, block, 0, stream>>>(p); break;      \
    case 2: simt_pair_kernel<T, 2><<<grid, block, 0, stream>>>(p); break;      \
    default: simt_pair_kernel<T, 4><<<grid, block, 0, stream>>>(p); break;     \
  }
  if (dtype == HG_DTYPE_BF16) { HG_SIMT(__nv_bfloat16) } else { HG_SIMT(__half) }
#undef HG_SIMT
  check(cudaGetLastError(), "SIMT pair launch");
}

}  // namespace hg
