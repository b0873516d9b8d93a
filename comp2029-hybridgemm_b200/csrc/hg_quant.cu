// MXFP8 / MXFP4 quantiser and fused SwiGLU+MXFP8 producer (memory-bound kernels).
//
// One kernel family replaces the reference's pack_mx / pack_mx_vector
// (integrations/vllm/native/runtime.cu:46-113) and silu_mx
// (integrations/vllm/native/producer.cu:10-45).  Sixteen threads own one
// (row, K128 block): each loads 8 contiguous 16-bit values with one 16-byte
// load, four neighbouring threads reduce the K32 amax with two shuffles, and
// the sixteen threads emit the block's four E8M0 bytes as ONE aligned 32-bit
// word of the 512-byte scale atom.  Threads past the real work write the 0x7f
// padding words of the last 128-row scale block, so no memset node precedes
// the kernel and every byte of the scale buffer is rewritten on every call.
#include <cstdlib>

#include "hg_common.cuh"

namespace hg {

std::string& last_error() {
  static thread_local std::string message;
  return message;
}

bool pdl_enabled() {
  static const bool enabled = [] {
    const char* v = std::getenv("HYGEMM_PDL");
    return !(v && v[0] == '0');
  }();
  return enabled;
}

template <typename T, bool FP4, bool SILU, int MATH>
__global__ void __launch_bounds__(256)
mx_quant_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ out, uint8_t* __restrict__ sf,
                uint16_t* __restrict__ debug, int rows, int k) {
  pdl_trigger();
  pdl_wait();   // the input is usually the previous kernel's output
  const int kblocks = k >> 7;
  const int64_t real = int64_t(rows) * kblocks * 16;
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= real) {
    // Padding words of the last 128-row scale block (rows .. roundup128(rows)-1).
    const int pad_rows = ((rows + 127) & ~127) - rows;
    const int64_t p = tid - real;
    if (pad_rows == 0 || p >= int64_t(pad_rows) * kblocks) return;
    const int row = rows + int(p % pad_rows), kb = int(p / pad_rows);
    *reinterpret_cast<uint32_t*>(sf + scale_word_offset(row, kb, k)) = 0x7f7f7f7fu;
    return;
  }
  const int lane = threadIdx.x & 31;
  const unsigned mask = 0xffffu << (lane & 16);        // the 16 threads of this (row, K128 block)
  const int sub = int(tid & 15);
  const int64_t item = tid >> 4;
  const int row = int(item / kblocks), kb = int(item % kblocks);
  const int col = kb * 128 + sub * 8;

  float v[8];
  if constexpr (SILU) {
    const uint4 g4 = *reinterpret_cast<const uint4*>(in + int64_t(row) * 2 * k + col);
    const uint4 u4 = *reinterpret_cast<const uint4*>(in + int64_t(row) * 2 * k + k + col);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
    uint32_t dw[4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float g = to_float<T>(uint16_t(gw[i >> 1] >> ((i & 1) * 16)));
      const float u = to_float<T>(uint16_t(uw[i >> 1] >> ((i & 1) * 16)));
      const float e = MATH == 0 ? expf(-g) : __expf(-g);
      const float act = MATH == 1 ? __fdividef(g, 1.f + e) : g / (1.f + e);
      // The consumer this replaces adds a zero beta to `up` before multiplying;
      // keeping the addition preserves +0 + -0 -> +0 and with it the sign bit
      // of a zero product (integrations/vllm/native/producer.cu:30-32).
      const float up = __fadd_rn(u, 0.f);
      const uint16_t a16 = from_float<T>(act);
      const uint16_t p16 = from_float<T>(to_float<T>(a16) * up);
      v[i] = to_float<T>(p16);
      if (i & 1) dw[i >> 1] |= uint32_t(p16) << 16; else dw[i >> 1] = p16;
    }
    if (debug) *reinterpret_cast<uint4*>(debug + int64_t(row) * k + col) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
  } else {
    const uint4 x4 = *reinterpret_cast<const uint4*>(in + int64_t(row) * k + col);
    const uint32_t xw[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_float<T>(uint16_t(xw[i >> 1] >> ((i & 1) * 16)));
  }

  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
  const int e = mx_exponent<FP4>(amax);
  const float inv = mx_inverse_scale(e);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] *= inv;

  if constexpr (FP4) {
    *reinterpret_cast<uint32_t*>(out + (int64_t(row) * k + col) / 2) = cvt_e2m1x8(v);
  } else {
    uint2 codes;
    codes.x = cvt_e4m3x2(v[0], v[1]) | (cvt_e4m3x2(v[2], v[3]) << 16);
    codes.y = cvt_e4m3x2(v[4], v[5]) | (cvt_e4m3x2(v[6], v[7]) << 16);
    *reinterpret_cast<uint2*>(out + int64_t(row) * k + col) = codes;
  }

  // Gather the four K32 exponents of this K128 block into one scale word.
  const int base = lane & 16;
  const uint32_t byte = uint32_t(e + 127);
  const uint32_t word = __shfl_sync(mask, byte, base) | (__shfl_sync(mask, byte, base + 4) << 8) |
                        (__shfl_sync(mask, byte, base + 8) << 16) | (__shfl_sync(mask, byte, base + 12) << 24);
  if (sub == 0) *reinterpret_cast<uint32_t*>(sf + scale_word_offset(row, kb, k)) = word;
}

template <typename T, bool FP4, bool SILU, int MATH>
static cudaError_t launch_quant(const void* in, void* out, void* sf, void* debug, int rows, int k, cudaStream_t s) {
  const int kblocks = k / 128;
  const int64_t pad_rows = ((rows + 127) & ~127) - rows;
  const int64_t threads = int64_t(rows) * kblocks * 16 + pad_rows * kblocks;
  const int64_t blocks = (threads + 255) / 256;
  return launch_kernel(mx_quant_kernel<T, FP4, SILU, MATH>, dim3(unsigned(blocks)), dim3(256), 0, s,
                       static_cast<const uint16_t*>(in), static_cast<uint8_t*>(out), static_cast<uint8_t*>(sf),
                       static_cast<uint16_t*>(debug), rows, k);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static void pack_any(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream, bool bf16) {
  // Argument rule of integrations/vllm/native/runtime.cu:121.
  if (rows <= 0 || k <= 0 || k % 128 || !in || !out || !sf) throw std::runtime_error("Invalid MX pack arguments");
  if (!aligned16(in) || !aligned16(out) || !aligned16(sf))
    throw std::runtime_error("MX pack pointers must be 16-byte aligned");
  auto s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (bf16) e = fp4 ? launch_quant<__nv_bfloat16, true, false, 0>(in, out, sf, nullptr, rows, k, s)
                    : launch_quant<__nv_bfloat16, false, false, 0>(in, out, sf, nullptr, rows, k, s);
  else      e = fp4 ? launch_quant<__half, true, false, 0>(in, out, sf, nullptr, rows, k, s)
                    : launch_quant<__half, false, false, 0>(in, out, sf, nullptr, rows, k, s);
  check(e, "MX pack launch");
}

static int silu_any(const void* in, void* q, void* sf, void* debug, int rows, int k, void* stream, int math, bool bf16) {
  // Argument rule and return convention of integrations/vllm/native/producer.cu:46-54.
  if (!in || !q || !sf || rows <= 0 || k <= 0 || k % 128 || math < 0 || math > 2) return int(cudaErrorInvalidValue);
  if (!aligned16(in) || !aligned16(q) || !aligned16(sf) || (debug && !aligned16(debug))) return int(cudaErrorMisalignedAddress);
  auto s = static_cast<cudaStream_t>(stream);
#define HG_SILU(T)                                                                     \
  (math == 0 ? launch_quant<T, false, true, 0>(in, q, sf, debug, rows, k, s)           \
   : math == 1 ? launch_quant<T, false, true, 1>(in, q, sf, debug, rows, k, s)         \
               : launch_quant<T, false, true, 2>(in, q, sf, debug, rows, k, s))
  return int(bf16 ? HG_SILU(__nv_bfloat16) : HG_SILU(__half));
#undef HG_SILU
}

}  // namespace hg

extern "C" {

const char* hg_last_error(void) { return hg::last_error().c_str(); }

int64_t hg_scale_size(int rows, int k) { return hg::scale_size(rows, k); }

// `mode` selected among kernels in the reference; every mode wrote the same
// bytes, so here all modes run the one kernel.
int hg_pack(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream) {
  HG_TRY hg::pack_any(in, out, sf, rows, k, fp4, stream, false); HG_CATCH
}
int hg_pack_mode(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream, int mode) {
  (void)mode;
  HG_TRY hg::pack_any(in, out, sf, rows, k, fp4, stream, false); HG_CATCH
}
int hg_pack_bf16(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream) {
  HG_TRY hg::pack_any(in, out, sf, rows, k, fp4, stream, true); HG_CATCH
}
int hg_pack_mode_bf16(const void* in, void* out, void* sf, int rows, int k, int fp4, void* stream, int mode) {
  (void)mode;
  HG_TRY hg::pack_any(in, out, sf, rows, k, fp4, stream, true); HG_CATCH
}

int hg_silu_pack(const void* in, void* q, void* sf, void* debug, int rows, int k, void* stream, int math) {
  return hg::silu_any(in, q, sf, debug, rows, k, stream, math, false);
}
int hg_silu_pack_bf16(const void* in, void* q, void* sf, void* debug, int rows, int k, void* stream, int math) {
  return hg::silu_any(in, q, sf, debug, rows, k, stream, math, true);
}

}  // extern "C"
