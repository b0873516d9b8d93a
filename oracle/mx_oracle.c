/*
 * CPU oracle for the hybrid MXFP4/MXFP8 output-channel linear layer.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference algorithm; it is linked by the test-suite, by the smoke check and
 * by the CPU-baseline leg of the benchmark, never by the product path (the
 * product path is the CUDA library and has no CPU fallback).
 *
 * Parity status: pinned.  The decode/dequantise/matmul half is checked against
 * outputs of the reference's own Python (decode_mx, codes_rne, pack_codes,
 * decode_logical, scale_indices) stored under tests/golden/; the E4M3
 * conversion is checked against the CPU float8_e4m3fn cast of PyTorch and
 * against the host conversion of the CUTLASS headers for every 16-bit input;
 * the exponent rule is checked exhaustively against its closed form.  The
 * reference's CUDA quantiser itself cannot execute off an SM120 GPU.
 *
 * Each function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ------------------------------------------------------------------------- */
/* Minimal pthread parallel-for (row ranges), so the timed CPU baseline can   */
/* use every host core without an OpenMP runtime.                             */
/* ------------------------------------------------------------------------- */

static int g_threads = 0;
void hgo_set_threads(int n) { g_threads = n; }
int hgo_threads(void) {
  if (g_threads > 0) return g_threads;
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}
typedef void (*row_fn)(int begin, int end, void* ctx);
typedef struct { row_fn fn; void* ctx; int begin, end; } row_job;
static void* row_thread(void* p) { row_job* j = (row_job*)p; j->fn(j->begin, j->end, j->ctx); return NULL; }
static void parallel_rows(int n, row_fn fn, void* ctx) {
  int threads = hgo_threads();
  if (threads > n) threads = n;
  if (threads <= 1) { fn(0, n, ctx); return; }
  pthread_t tid[256]; row_job job[256];
  if (threads > 256) threads = 256;
  int chunk = (n + threads - 1) / threads, started = 0;
  for (int t = 0; t < threads; ++t) {
    int b = t * chunk, e = b + chunk > n ? n : b + chunk;
    if (b >= e) break;
    job[t] = (row_job){fn, ctx, b, e};
    if (pthread_create(&tid[t], NULL, row_thread, &job[t]) != 0) { fn(b, e, ctx); tid[t] = 0; }
    started = t + 1;
  }
  for (int t = 0; t < started; ++t) if (tid[t]) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------------- */
/* 16-bit float helpers                                                       */
/* ------------------------------------------------------------------------- */

static inline float bits_to_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t float_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float hgo_half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_to_float(sign);
    float v = ldexpf((float)man, -24);
    return sign ? -v : v;
  }
  if (exp == 31) return bits_to_float(sign | 0x7f800000u | (man << 13));
  return bits_to_float(sign | ((exp + 112) << 23) | (man << 13));
}

float hgo_bf16_to_float(uint16_t h) { return bits_to_float((uint32_t)h << 16); }

/* round-to-nearest-even float -> IEEE half (matches __float2half_rn) */
uint16_t hgo_float_to_half(float f) {
  uint32_t x = float_to_bits(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t a = x & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);          /* NaN */
  if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);         /* overflow -> inf (>= 65536) */
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);         /* rounds up to inf */
  if (a < 0x33000001u) return (uint16_t)sign;                      /* < 2^-25 (or ==) -> 0 */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift = (e < -14) ? (13 + (-14 - e)) : 13;
  uint32_t half_m = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (half_m & 1))) half_m++;
  uint32_t out;
  if (e < -14) out = half_m;                                       /* subnormal (may carry to normal) */
  else out = ((uint32_t)(e + 15) << 10) + (half_m - 0x400u);       /* carry propagates into exponent */
  return (uint16_t)(sign | out);
}

/* round-to-nearest-even float -> bfloat16 (matches __float2bfloat16_rn) */
uint16_t hgo_float_to_bf16(float f) {
  uint32_t x = float_to_bits(f);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7fffu + lsb;
  return (uint16_t)(x >> 16);
}

static inline float load16(const uint16_t* p, int64_t i, int bf16) {
  return bf16 ? hgo_bf16_to_float(p[i]) : hgo_half_to_float(p[i]);
}
static inline uint16_t round16(float v, int bf16) {
  return bf16 ? hgo_float_to_bf16(v) : hgo_float_to_half(v);
}

/* ------------------------------------------------------------------------- */
/* Element codecs                                                             */
/* ------------------------------------------------------------------------- */

/* E4M3 (fn: no inf, 0x7f/0xff NaN, max 448), round-to-nearest-even,
 * saturating to +-448.  Follows the conversion the reference applies in
 * integrations/vllm/native/runtime.cu:79 (cutlass::float_e4m3_t(float)). */
uint8_t hgo_e4m3_from_float(float f) {
  uint32_t x = float_to_bits(f);
  uint8_t sign = (uint8_t)((x >> 24) & 0x80u);
  uint32_t a = x & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint8_t)(sign | 0x7f);
  float v = bits_to_float(a);
  if (v >= 464.0f) return (uint8_t)(sign | 0x7e);                  /* saturate (464 = tie above 448) */
  if (v < 0.0009765625f) {                                         /* below 2^-10: 0 or tie */
    /* smallest subnormal is 2^-9; halfway is 2^-10, ties to even (0). */
    return sign;
  }
  int e; float m = frexpf(v, &e);                                  /* v = m*2^e, m in [0.5,1) */
  e -= 1;                                                          /* v = (2m)*2^e, 2m in [1,2) */
  int q_exp = e < -6 ? -6 : e;                                     /* subnormals share exponent -6 */
  float scaled = ldexpf(v, 3 - q_exp);                             /* units of the 3-bit mantissa */
  float r = nearbyintf(scaled);                                    /* default mode: ties-to-even */
  (void)m;
  int mant = (int)r;                                               /* in [0,16] */
  int expo = q_exp + 7;
  if (e < -6) {                                                    /* subnormal: mant in [0,8] */
    if (mant >= 8) return (uint8_t)(sign | (1 << 3) | (mant - 8));
    return (uint8_t)(sign | mant);
  }
  if (mant >= 16) { mant = 8; expo += 1; }
  uint32_t code = ((uint32_t)expo << 3) | (uint32_t)(mant - 8);
  if (code > 0x7e) code = 0x7e;
  return (uint8_t)(sign | code);
}

float hgo_e4m3_to_float(uint8_t c) {
  int sign = c & 0x80, e = (c >> 3) & 0xf, m = c & 7;
  float v;
  if (e == 15 && m == 7) v = NAN;
  else if (e == 0) v = ldexpf((float)m, -9);
  else v = ldexpf((float)(8 + m), e - 10);
  return sign ? -v : v;
}

/* E2M1 round-to-nearest-even, saturating at 6, sign bit kept for -0.
 * Follows integrations/vllm/allocation/fp4_quant.py:10-16 (codes_rne): the
 * decision boundaries .25,.75,1.25,1.75,2.5,3.5,5 with ties resolved to the
 * even code. */
uint8_t hgo_e2m1_from_float(float f) {
  static const float bound[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  uint8_t sign = signbit(f) ? 8 : 0;
  float a = fabsf(f);
  int code = 0;
  while (code < 7 && a > bound[code]) code++;                      /* bucketize(right=False) */
  if (code < 7 && a == bound[code] && (code & 1)) code++;          /* tie on an odd code -> even */
  return (uint8_t)(sign | code);
}

static const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
float hgo_e2m1_to_float(uint8_t c) { return kE2M1[c & 15]; }
/* decode_mx's table (integrations/vllm/test_components.py:16) holds +0 at code 8. */
static const float kE2M1Decode[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                      0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

/* ------------------------------------------------------------------------- */
/* Scale layout                                                               */
/* ------------------------------------------------------------------------- */

/* Physical byte offset of the E8M0 scale for (row r, K32 group g): 512-byte
 * atoms of 128 rows x 4 groups.  integrations/vllm/hygemm_vllm/offline_weights.py:6-9,
 * integrations/vllm/native/producer.cu:7-9. */
int64_t hgo_scale_index(int r, int g, int k) {
  return ((int64_t)(r / 128) * (k / 128) + g / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + g % 4;
}

/* Size in bytes of the padded scale buffer (integrations/vllm/native/runtime.cu:117-119,
 * integrations/vllm/hygemm_vllm/quality_worker.py:29). */
int64_t hgo_scale_size(int rows, int k) {
  if (rows <= 0 || k <= 0) return 0;
  return (int64_t)((rows + 127) / 128) * (k / 128) * 512;
}

/* ------------------------------------------------------------------------- */
/* Exponent rule                                                              */
/* ------------------------------------------------------------------------- */

/* Literal form: integrations/vllm/native/runtime.cu:71-72
 *   e = amax>0 ? int(ceilf(log2f(amax/max))) : 0 ; clamp to [-127,127]. */
int hgo_exponent_literal(float amax, int fp4) {
  if (!(amax > 0)) return 0;
  float q = amax / (fp4 ? 6.0f : 448.0f);
  float l = ceilf(log2f(q));
  if (l < -127.f) return -127;
  if (l > 127.f) return 127;
  return (int)l;
}

/* Closed form used by the CUDA kernels: the smallest e with amax*2^-e <= max,
 * computed from the fp32 bit pattern (no transcendental). */
int hgo_exponent_exact(float amax, int fp4) {
  if (!(amax > 0)) return 0;
  uint32_t b = float_to_bits(amax);
  int ef = (int)(b >> 23);
  if (ef == 0) return -127;                                        /* fp32 subnormal */
  uint32_t man = b & 0x7fffffu;
  int x = ef - 127, e;
  if (fp4) e = (man <= 0x400000u) ? x - 2 : x - 1;                 /* max 6   = 1.5  * 2^2 */
  else     e = (man <= 0x600000u) ? x - 8 : x - 7;                 /* max 448 = 1.75 * 2^8 */
  if (e < -127) e = -127;
  if (e > 127) e = 127;
  return e;
}

/* ------------------------------------------------------------------------- */
/* Quantiser: integrations/vllm/native/runtime.cu:46-80 (pack_mx) and         */
/* :84-113 (pack_mx_vector); both produce identical bytes.                    */
/* ------------------------------------------------------------------------- */

typedef struct {
  const uint16_t* in; uint8_t* out; uint8_t* sf; uint16_t* debug;
  int k, fp4, bf16, silu;
} pack_ctx;

static void pack_rows(int begin, int end, void* p) {
  pack_ctx* c = (pack_ctx*)p;
  const int k = c->k, fp4 = c->fp4, bf16 = c->bf16, groups = k / 32;
  for (int r = begin; r < end; ++r) {
    for (int g = 0; g < groups; ++g) {
      float v[32], amax = 0.f;
      for (int i = 0; i < 32; ++i) {
        int col = g * 32 + i;
        if (c->silu) {
          /* integrations/vllm/native/producer.cu:24-35 */
          float gate = load16(c->in, (int64_t)r * 2 * k + col, bf16);
          float up = load16(c->in, (int64_t)r * 2 * k + k + col, bf16) + 0.0f;
          float act = gate / (1.f + expf(-gate));
          uint16_t a16 = round16(act, bf16);
          float a = bf16 ? hgo_bf16_to_float(a16) : hgo_half_to_float(a16);
          uint16_t v16 = round16(a * up, bf16);
          if (c->debug) c->debug[(int64_t)r * k + col] = v16;
          v[i] = bf16 ? hgo_bf16_to_float(v16) : hgo_half_to_float(v16);
        } else {
          v[i] = load16(c->in, (int64_t)r * k + col, bf16);
        }
        amax = fmaxf(amax, fabsf(v[i]));
      }
      int e = hgo_exponent_literal(amax, fp4);
      c->sf[hgo_scale_index(r, g, k)] = (uint8_t)(e + 127);
      if (fp4) {
        for (int i = 0; i < 32; i += 2) {
          uint8_t lo = hgo_e2m1_from_float(ldexpf(v[i], -e));
          uint8_t hi = hgo_e2m1_from_float(ldexpf(v[i + 1], -e));
          c->out[((int64_t)r * k + g * 32 + i) / 2] = (uint8_t)(lo | (hi << 4));
        }
      } else {
        for (int i = 0; i < 32; ++i)
          c->out[(int64_t)r * k + g * 32 + i] = hgo_e4m3_from_float(ldexpf(v[i], -e));
      }
    }
  }
}

/* in: [rows,k] 16-bit floats (bf16 != 0 selects bfloat16, else IEEE half).
 * out: [rows,k] E4M3 bytes, or [rows,k/2] packed E2M1 (even k in the low
 * nibble, runtime.cu:77-78).  sf: hgo_scale_size(rows,k) bytes; every byte
 * that is not a valid (row,group) scale is 0x7f (runtime.cu:60-63,:130). */
int hgo_pack(const uint16_t* in, uint8_t* out, uint8_t* sf, int rows, int k, int fp4, int bf16) {
  if (rows <= 0 || k <= 0 || k % 128 || !in || !out || !sf) return -1;
  memset(sf, 127, (size_t)hgo_scale_size(rows, k));
  pack_ctx ctx = {in, out, sf, NULL, k, fp4, bf16, 0};
  parallel_rows(rows, pack_rows, &ctx);
  return 0;
}

/* SwiGLU + quantiser: integrations/vllm/native/producer.cu:10-45.
 * in: [rows, 2k] = gate || up.  act = round16(g/(1+expf(-g)));
 * v = round16(float(act) * (up + 0.0f)); then the K32 quantisation of v.
 * debug (optional): [rows,k] receives the 16-bit v. */
int hgo_silu_pack(const uint16_t* in, uint8_t* q, uint8_t* sf, uint16_t* debug, int rows, int k, int bf16) {
  if (rows <= 0 || k <= 0 || k % 128 || !in || !q || !sf) return -1;
  memset(sf, 127, (size_t)hgo_scale_size(rows, k));
  pack_ctx ctx = {in, q, sf, debug, k, 0, bf16, 1};
  parallel_rows(rows, pack_rows, &ctx);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Offline MXFP4 exponent search: integrations/vllm/allocation/fp4_quant.py   */
/* :28-58 (quantize).  Per K32 group the round-to-nearest result of hgo_pack  */
/* is the baseline; for every non-zero offset in the given order the scale    */
/* byte is moved by that offset (clamped to [0,254]), the group re-rounded    */
/* with codes_rne and kept if its importance-weighted squared error is        */
/* STRICTLY smaller than the best so far.  Output: packed codes [rows,k/2]    */
/* and logical scale bytes [rows,k/32].                                       */
/*                                                                            */
/* The reference sums the 32 error terms with a torch reduction whose order   */
/* is not specified; here the order is fixed: four runs of eight terms added  */
/* left to right, then (r0+r1)+(r2+r3).  The two can differ only where two    */
/* candidates tie to within fp32 rounding of the sum.                         */
/* ------------------------------------------------------------------------- */

typedef struct {
  const uint16_t* in; const float* importance; uint8_t* q4; uint8_t* scales;
  int k, bf16, n_offsets; const int* offsets;
} clip_ctx;

static float group_error(const float* v, const uint8_t* code, float scale, const float* weight) {
  float run[4];
  for (int j = 0; j < 4; ++j) {
    float sum = 0.f;
    for (int i = 0; i < 8; ++i) {
      float diff = kE2M1[code[8 * j + i]] * scale - v[8 * j + i];
      float term = diff * diff;
      term = term * (weight ? weight[8 * j + i] : 1.f);
      sum = sum + term;
    }
    run[j] = sum;
  }
  return (run[0] + run[1]) + (run[2] + run[3]);
}

static void clip_rows(int begin, int end, void* p) {
  clip_ctx* c = (clip_ctx*)p;
  const int k = c->k, groups = k / 32;
  for (int r = begin; r < end; ++r)
    for (int g = 0; g < groups; ++g) {
      float v[32], amax = 0.f;
      for (int i = 0; i < 32; ++i) {
        v[i] = load16(c->in, (int64_t)r * k + g * 32 + i, c->bf16);
        amax = fmaxf(amax, fabsf(v[i]));
      }
      const float* weight = c->importance ? c->importance + g * 32 : NULL;
      const int base = hgo_exponent_literal(amax, 1) + 127;
      uint8_t best_code[32], code[32];
      int best_byte = base;
      for (int i = 0; i < 32; ++i) best_code[i] = hgo_e2m1_from_float(ldexpf(v[i], -(base - 127)));
      float best = group_error(v, best_code, ldexpf(1.f, base - 127), weight);
      for (int o = 0; o < c->n_offsets; ++o) {
        if (c->offsets[o] == 0) continue;
        int byte = base + c->offsets[o];
        byte = byte < 0 ? 0 : (byte > 254 ? 254 : byte);
        for (int i = 0; i < 32; ++i) code[i] = hgo_e2m1_from_float(ldexpf(v[i], -(byte - 127)));
        float err = group_error(v, code, ldexpf(1.f, byte - 127), weight);
        if (err < best) { best = err; best_byte = byte; memcpy(best_code, code, 32); }
      }
      c->scales[(int64_t)r * groups + g] = (uint8_t)best_byte;
      for (int i = 0; i < 32; i += 2)
        c->q4[((int64_t)r * k + g * 32 + i) / 2] = (uint8_t)(best_code[i] | (best_code[i + 1] << 4));
    }
}

int hgo_clip_pack(const uint16_t* in, const float* importance, uint8_t* q4, uint8_t* scales, int rows, int k,
                  const int* offsets, int n_offsets, int bf16) {
  if (rows <= 0 || k <= 0 || k % 128 || !in || !q4 || !scales || n_offsets < 0 || (n_offsets && !offsets)) return -1;
  clip_ctx ctx = {in, importance, q4, scales, k, bf16, n_offsets, offsets};
  parallel_rows(rows, clip_rows, &ctx);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Dequantise: integrations/vllm/test_components.py:10-24 (decode_mx)         */
/* ------------------------------------------------------------------------- */

typedef struct { const uint8_t* q; const uint8_t* sf; float* out; int k, fp4; } decode_ctx;

static void decode_rows(int begin, int end, void* p) {
  decode_ctx* d = (decode_ctx*)p;
  const int k = d->k;
  for (int r = begin; r < end; ++r)
    for (int c = 0; c < k; ++c) {
      float scale = exp2f((float)d->sf[hgo_scale_index(r, c / 32, k)] - 127.f);
      float v;
      if (d->fp4) {
        uint8_t byte = d->q[((int64_t)r * k + c) / 2];
        v = kE2M1Decode[(c & 1) ? (byte >> 4) : (byte & 15)];
      } else {
        v = hgo_e4m3_to_float(d->q[(int64_t)r * k + c]);
      }
      d->out[(int64_t)r * k + c] = v * scale;
    }
}

int hgo_decode(const uint8_t* q, const uint8_t* sf, float* out, int rows, int k, int fp4) {
  if (rows < 0 || k <= 0 || k % 128) return -1;
  decode_ctx ctx = {q, sf, out, k, fp4};
  parallel_rows(rows, decode_rows, &ctx);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Hybrid linear: integrations/vllm/test_components.py:27-38 (reference)      */
/* ------------------------------------------------------------------------- */

typedef struct {
  const float* dw; const float* dx; const int32_t* ids;
  int tokens, k, outputs, bf16; uint16_t* y; float* y_f32;
} gemm_ctx;

static void gemm_rows(int begin, int end, void* p) {
  gemm_ctx* g = (gemm_ctx*)p;
  for (int r = begin; r < end; ++r) {
    const float* wr = g->dw + (int64_t)r * g->k;
    for (int t = 0; t < g->tokens; ++t) {
      const float* xr = g->dx + (int64_t)t * g->k;
      float acc = 0.f;
      for (int c = 0; c < g->k; ++c) acc += wr[c] * xr[c];
      int64_t at = (int64_t)t * g->outputs + g->ids[r];
      if (g->y) g->y[at] = round16(acc, g->bf16);
      if (g->y_f32) g->y_f32[at] = acc;
    }
  }
}

/* y[t, ids[r]] = round16( sum_k dw[r,k] * dx[t,k] ) with fp32 accumulation over
 * the dequantised operands.  Both partitions scatter into y [tokens,outputs]
 * (16-bit) and/or y_f32.  Accumulation order is k ascending (the tolerance of
 * the parity tests absorbs the order; the exact-representable cases are
 * order-free). */
int hgo_hybrid_linear(const uint8_t* w4, const uint8_t* sf4, const int32_t* lo, int rows_lo,
                      const uint8_t* w8, const uint8_t* sf8, const int32_t* hi, int rows_hi,
                      const uint8_t* xq, const uint8_t* xsf, int tokens, int k, int outputs,
                      uint16_t* y, int bf16, float* y_f32) {
  if (tokens <= 0 || k <= 0 || k % 128 || outputs <= 0) return -1;
  float* dx = (float*)malloc(sizeof(float) * (size_t)tokens * k);
  if (!dx) return -2;
  hgo_decode(xq, xsf, dx, tokens, k, 0);
  for (int part = 0; part < 2; ++part) {
    int rows = part ? rows_hi : rows_lo;
    if (!rows) continue;
    float* dw = (float*)malloc(sizeof(float) * (size_t)rows * k);
    if (!dw) { free(dx); return -2; }
    hgo_decode(part ? w8 : w4, part ? sf8 : sf4, dw, rows, k, part ? 0 : 1);
    gemm_ctx ctx = {dw, dx, part ? hi : lo, tokens, k, outputs, bf16, y, y_f32};
    parallel_rows(rows, gemm_rows, &ctx);
    free(dw);
  }
  free(dx);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Exact-representable generator: src/kernel/output_channel_bench.cu:48-57    */
/* ------------------------------------------------------------------------- */

uint32_t hgo_hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; return x ^ (x >> 16);
}
float hgo_raw_weight(int row, int k, int fp8) {
  static const float f4[8] = {-2, -1.5f, -1, -.5f, .5f, 1, 1.5f, 2};
  uint32_t h = hgo_hash32((uint32_t)row * 0x9e3779b9u + (uint32_t)k + 17u);
  return fp8 ? (float)((int)(h % 31) - 15) / 8 : f4[h & 7];
}
float hgo_raw_activation(int token, int k) {
  return (float)((int)(hgo_hash32((uint32_t)token * 0x85ebca6bu + (uint32_t)k + 29u) % 31) - 15) / 8;
}
float hgo_raw_scale(int row, int group, int seed) {
  static const float v[3] = {.5f, 1.f, 2.f};
  return v[hgo_hash32((uint32_t)row * 0x9e3779b9u + (uint32_t)group + (uint32_t)seed) % 3];
}
static uint8_t scale_byte(float s) { return s == .5f ? 126 : (s == 1.f ? 127 : 128); }

/* Fills one partition of an exact case (output_channel_bench.cu:99-110):
 * ids[r] are original channel numbers; weights and scales are functions of
 * the channel number, not of the partition row. */
int hgo_exact_weights(const int32_t* ids, int rows, int k, int fp8, uint8_t* w, uint8_t* sf) {
  if (rows <= 0) return 0;
  memset(sf, 127, (size_t)hgo_scale_size(rows, k));
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < k; ++c) {
      float v = hgo_raw_weight(ids[r], c, fp8);
      if (fp8) w[(int64_t)r * k + c] = hgo_e4m3_from_float(v);
      else {
        uint8_t code = hgo_e2m1_from_float(v);
        uint8_t* b = &w[((int64_t)r * k + c) / 2];
        *b = (c & 1) ? (uint8_t)((*b & 15) | (code << 4)) : (uint8_t)((*b & 0xf0) | code);
      }
      if (c % 32 == 0) sf[hgo_scale_index(r, c / 32, k)] = scale_byte(hgo_raw_scale(ids[r], c / 32, 88));
    }
  return 0;
}
int hgo_exact_activations(int tokens, int k, uint8_t* x, uint8_t* sf) {
  memset(sf, 127, (size_t)hgo_scale_size(tokens, k));
  for (int t = 0; t < tokens; ++t)
    for (int c = 0; c < k; ++c) {
      x[(int64_t)t * k + c] = hgo_e4m3_from_float(hgo_raw_activation(t, c));
      if (c % 32 == 0) sf[hgo_scale_index(t, c / 32, k)] = scale_byte(hgo_raw_scale(t, c / 32, 100));
    }
  return 0;
}
/* Expected output element (output_channel_bench.cu:121-125), before the
 * 16-bit rounding; every partial sum is exactly representable in fp32. */
float hgo_exact_reference(int out, int token, int k, int is_high) {
  float sum = 0;
  for (int c = 0; c < k; ++c)
    sum += hgo_raw_weight(out, c, is_high) * hgo_raw_scale(out, c / 32, 88) *
           hgo_raw_activation(token, c) * hgo_raw_scale(token, c / 32, 100);
  return sum;
}

typedef struct { const uint8_t* is_high; int tokens, k, outputs, bf16; uint16_t* y; } exact_ctx;
static void exact_rows(int begin, int end, void* p) {
  exact_ctx* e = (exact_ctx*)p;
  for (int o = begin; o < end; ++o)
    for (int t = 0; t < e->tokens; ++t)
      e->y[(int64_t)t * e->outputs + o] = round16(hgo_exact_reference(o, t, e->k, e->is_high[o]), e->bf16);
}
void hgo_exact_expected(const uint8_t* is_high, int outputs, int tokens, int k, uint16_t* y, int bf16) {
  exact_ctx ctx = {is_high, tokens, k, outputs, bf16, y};
  parallel_rows(outputs, exact_rows, &ctx);
}
